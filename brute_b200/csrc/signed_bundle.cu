// signed_bundle: int8 weights x bit1 values -> bit1 votes.
//   out[b, m, d] = ( sum_n W[b, m, n] * pm1(V[b, n, d]) >= 0 ),  pm1(bit) = bit ? +1 : -1,
// W int8 [B, M, N], V packed [B, N, ceil(D/64)], out packed [B, M, ceil(D/64)], pad bits 0.
//
// With v in {0,1}: sum_n w*pm1(v) = 2*T - S, T[m,d] = sum_n w[m,n]*v[n,d], S[m] = sum_n w[m,n].
// T is an int8 x {0,1} contraction done with dp4a: a block owns 32 rows of W and one 64-bit
// output word; V's words are stored to shared memory byte-transposed ([8 bytes of the word][n]),
// so that 4 consecutive n of one byte column are one 32-bit load, and the 8 bits of that column
// spread into 8 dp4a operands with a shift and a mask each (0.75 ALU op per MAC). Each thread
// keeps 8 accumulators (its 8 bits of the word), not 64.
#include "signed_bundle_tcgen05.cuh"

namespace bb {

constexpr int SB_ROWS = 32, SB_NCHUNK = 128, SB_THREADS = 256;

__global__ void __launch_bounds__(SB_THREADS)
k_signed_bundle(const int8_t* __restrict__ W, const uint64_t* __restrict__ V, uint64_t* __restrict__ out,
                int64_t M, int64_t N, int64_t Dp, int64_t D) {
    __shared__ __align__(16) int8_t Ws[SB_ROWS][SB_NCHUNK];
    __shared__ __align__(16) uint8_t Vb[8][SB_NCHUNK];
    const int tid = threadIdx.x, lane = tid & 31;
    // lane = (row & 3) * 8 + byte column, so the 8 byte columns of a row are 8 neighbouring lanes
    const int col = tid & 7, row = tid >> 3;                 // row 0..31
    const int64_t b = blockIdx.z, dp = blockIdx.x, m0 = (int64_t)blockIdx.y * SB_ROWS;
    const int8_t* Wb = W + b * M * N;
    const uint64_t* Vbat = V + b * N * Dp;

    int acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int wsum = 0;
    for (int64_t n0 = 0; n0 < N; n0 += SB_NCHUNK) {
        // W tile: 32 rows x 128 n (bytes), zero filled past the edges
        for (int i = tid; i < SB_ROWS * SB_NCHUNK; i += SB_THREADS) {
            const int r = i / SB_NCHUNK, c = i % SB_NCHUNK;
            Ws[r][c] = (m0 + r < M && n0 + c < N) ? Wb[(m0 + r) * N + n0 + c] : (int8_t)0;
        }
        // V words of this chunk, byte-transposed
        if (tid < SB_NCHUNK) {
            const uint64_t w = (n0 + tid < N) ? __ldg(Vbat + (n0 + tid) * Dp + dp) : 0ull;
#pragma unroll
            for (int g = 0; g < 8; ++g) Vb[g][tid] = (uint8_t)(w >> (8 * g));
        }
        __syncthreads();
#pragma unroll 4
        for (int c = 0; c < SB_NCHUNK; c += 4) {
            const int w4 = *reinterpret_cast<const int*>(&Ws[row][c]);
            const uint32_t x = *reinterpret_cast<const uint32_t*>(&Vb[col][c]);
            wsum = __dp4a(w4, 0x01010101, wsum);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = __dp4a(w4, (int)((x >> j) & 0x01010101u), acc[j]);
        }
        __syncthreads();
    }
    uint32_t byte = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int64_t d = dp * 64 + col * 8 + j;
        if (d < D && 2 * acc[j] - wsum >= 0) byte |= 1u << j;
    }
    uint64_t word = (uint64_t)byte << (8 * col);
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    word |= __shfl_xor_sync(0xffffffffu, word, 2);
    word |= __shfl_xor_sync(0xffffffffu, word, 4);
    if ((lane & 7) == 0 && m0 + row < M) out[(b * M + m0 + row) * Dp + dp] = word;
}

}  // namespace bb

using namespace bb;

extern "C" int brute_b200_signed_bundle(const int8_t* W, const uint64_t* V, uint64_t* out,
                                        int64_t B, int64_t M, int64_t N, int64_t Dp, int64_t D, void* stream) {
    BB_REQUIRE(B >= 0 && M >= 0 && N >= 0 && Dp >= 0 && D >= 0 && D <= 64 * Dp, BRUTE_ERR_INVALID_ARG);
    if (B * M * Dp == 0) return BRUTE_OK;
    BB_REQUIRE(out != nullptr && (N == 0 || (W != nullptr && V != nullptr)), BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(V) && aligned8(out), BRUTE_ERR_MISALIGNED);
    // The tensor-core kernel with the bit transpose of V fused into its expander warps: one launch,
    // no scratch. Shapes outside the TMA rules, and rows padded beyond ceil(D/64) words (the tensor
    // path writes only that many words of every output row), take the CUDA-core kernel below.
    if (st_accepts(W, B, M, N, D) && Dp == (D + 63) / 64)
        return st_run(W, V, out, B, M, N, Dp, D, as_stream(stream), /*fused=*/true);
    BB_REQUIRE(B <= 65535 && (M + SB_ROWS - 1) / SB_ROWS <= 65535, BRUTE_ERR_UNSUPPORTED);
    const dim3 grid((unsigned)Dp, (unsigned)((M + SB_ROWS - 1) / SB_ROWS), (unsigned)B);
    k_signed_bundle<<<grid, SB_THREADS, 0, as_stream(stream)>>>(W, V, out, M, N, Dp, D);
    return launch_status();
}

namespace bb { int sb_status_bridge() { return tc5_device_status(); } }

extern "C" int brute_b200_transpose_bits(const uint64_t* in, uint64_t* out, int64_t batch, int64_t R, int64_t C, void* stream);

extern "C" int64_t brute_b200_signed_bundle_workspace_bytes(int64_t B, int64_t N, int64_t D) {
    if (B <= 0 || N <= 0 || D <= 0) return 0;
    return B * D * ((N + 63) / 64) * 8;          // V transposed: [B, D, ceil(N/64)] words
}

extern "C" int brute_b200_signed_bundle_ws(const int8_t* W, const uint64_t* V, uint64_t* out,
                                           int64_t B, int64_t M, int64_t N, int64_t Dp, int64_t D,
                                           void* workspace, int64_t workspace_bytes, void* stream) {
    BB_REQUIRE(B >= 0 && M >= 0 && N >= 0 && Dp >= 0 && D >= 0 && D <= 64 * Dp, BRUTE_ERR_INVALID_ARG);
    if (B * M * Dp == 0) return BRUTE_OK;
    // Shapes outside the TMA rules take the CUDA-core kernel, no workspace. So do rows that are padded
    // beyond ceil(D/64) words: the bit transpose reads V with a pitch of ceil(D/64) words per row, and
    // the tensor path writes only that many words of every output row.
    if (!st_accepts(W, B, M, N, D) || Dp != (D + 63) / 64)
        return brute_b200_signed_bundle(W, V, out, B, M, N, Dp, D, stream);
    BB_REQUIRE(out != nullptr && W != nullptr && V != nullptr, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(V) && aligned8(out), BRUTE_ERR_MISALIGNED);
    BB_REQUIRE(workspace != nullptr && workspace_bytes >= brute_b200_signed_bundle_workspace_bytes(B, N, D),
               BRUTE_ERR_WORKSPACE);
    BB_REQUIRE(aligned8(workspace), BRUTE_ERR_MISALIGNED);
    uint64_t* Vt = static_cast<uint64_t*>(workspace);
    // V [B, N, Dp] holds D valid bits per row: transpose the [N x D] bit matrices into [D x N]
    const int rc = brute_b200_transpose_bits(V, Vt, B, N, D, stream);
    if (rc != BRUTE_OK) return rc;
    return st_run(W, Vt, out, B, M, N, Dp, D, as_stream(stream), /*fused=*/false);
}

// ---------------------------------------------------------------------------
// The same call for callers that cannot hand over a workspace: the scratch for the bit-transposed V
// is a fixed array in device memory that belongs to the library image.
namespace bb {
constexpr int64_t SB_STATIC_SCRATCH_BYTES = 1 << 20;            // 1 MiB: B * D * ceil(N/64) * 8 must fit
static __device__ __align__(256) uint64_t g_sb_static_scratch[SB_STATIC_SCRATCH_BYTES / 8];
constexpr int SB_MAX_DEVICES = 64;
static uint64_t* g_sb_static_ptr[SB_MAX_DEVICES];               // device address of the array, per device
}  // namespace bb

extern "C" int64_t brute_b200_signed_bundle_static_max_bytes(void) { return SB_STATIC_SCRATCH_BYTES; }

extern "C" int brute_b200_signed_bundle_static(const int8_t* W, const uint64_t* V, uint64_t* out,
                                               int64_t B, int64_t M, int64_t N, int64_t Dp, int64_t D,
                                               void* stream) {
    BB_REQUIRE(B >= 0 && M >= 0 && N >= 0 && Dp >= 0 && D >= 0 && D <= 64 * Dp, BRUTE_ERR_INVALID_ARG);
    if (B * M * Dp == 0) return BRUTE_OK;
    if (!st_accepts(W, B, M, N, D) || Dp != (D + 63) / 64)     // the CUDA-core kernel uses no scratch, whatever the size
        return brute_b200_signed_bundle(W, V, out, B, M, N, Dp, D, stream);
    const int64_t need = brute_b200_signed_bundle_workspace_bytes(B, N, D);
    BB_REQUIRE(need <= SB_STATIC_SCRATCH_BYTES, BRUTE_ERR_WORKSPACE);
    int dev = -1;
    BB_REQUIRE(cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < SB_MAX_DEVICES, BRUTE_ERR_LAUNCH);
    if (g_sb_static_ptr[dev] == nullptr) {
        // once per device, with that device current: where this device keeps the array
        void* p = nullptr;
        BB_REQUIRE(cudaGetSymbolAddress(&p, g_sb_static_scratch) == cudaSuccess && p != nullptr, BRUTE_ERR_LAUNCH);
        g_sb_static_ptr[dev] = static_cast<uint64_t*>(p);
    }
    // Nothing in the scratch has to start at zero: the transpose writes every word that the GEMM
    // reads (all ceil(N/64) words of all D rows of all B batches, pad bits included).
    return brute_b200_signed_bundle_ws(W, V, out, B, M, N, Dp, D, g_sb_static_ptr[dev], SB_STATIC_SCRATCH_BYTES, stream);
}
