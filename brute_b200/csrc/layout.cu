// Layout kernels on packed words: bit-matrix transpose and OR/AND over a non-packed axis.
//
// transpose_bits: in [batch, R, ceil(C/64)] -> out [batch, C, ceil(R/64)], out bit (c, r) = in bit
// (r, c). A 64 x 64 bit block is transposed in registers by the butterfly (swap the off-diagonal
// 32 x 32 quadrants, then 16 x 16 inside each, ... down to 1 x 1): lane L holds rows L and L + 32
// of the block, the first round is inside the lane and the other five exchange with lane L ^ j
// through shuffles, about a hundred instructions per 64 x 64 block instead of 4096 single-bit moves. A CTA
// of 8 warps owns a 512 x 512 bit tile; warp w transposes the eight blocks of row-block w, and the
// transposed words go through shared memory so that every input and output row of the tile is one
// contiguous 64-byte run. HBM bound: 2 * R * C / 8 bytes.
//
// reduce_rows: in [outer, R, inner] words -> out [outer, inner] words, OR or AND over R. One
// thread per inner word (coalesced), R cut into chunks across blockIdx.y, partial results merged
// with 64-bit atomics into an output that the launcher presets (0 for OR, ~0 for AND).
#include "common.cuh"

namespace bb {

// lane L holds rows L (lo) and L + 32 (hi) of a 64 x 64 bit block; afterwards it holds rows L and
// L + 32 of the transposed block
__device__ __forceinline__ void transpose64x64(uint64_t& lo, uint64_t& hi, int lane) {
    {
        const uint64_t t = ((lo >> 32) ^ hi) & 0x00000000FFFFFFFFull;
        lo ^= t << 32;
        hi ^= t;
    }
    const uint64_t masks[5] = {0x0000FFFF0000FFFFull, 0x00FF00FF00FF00FFull, 0x0F0F0F0F0F0F0F0Full,
                               0x3333333333333333ull, 0x5555555555555555ull};
#pragma unroll
    for (int s = 0; s < 5; ++s) {
        const int j = 16 >> s;
        const uint64_t m = masks[s];
        // Rows k (lane bit j clear) and k + j (set) swap the bit blocks (m << j) of the first with
        // the blocks m of the second. Both lanes compute the same t = ((x_k >> j) ^ x_{k+j}) & m
        // from what they send and what they receive, and differ only in a shift amount.
        const int sh = (lane & j) ? 0 : j;
        const uint64_t slo = lo >> sh, shi = hi >> sh;
        const uint64_t tlo = (slo ^ __shfl_xor_sync(0xffffffffu, slo, j)) & m;
        const uint64_t thi = (shi ^ __shfl_xor_sync(0xffffffffu, shi, j)) & m;
        lo ^= tlo << sh;
        hi ^= thi << sh;
    }
}

constexpr int TB_TILE = 512;            // bits per tile side = 8 blocks of 64: 64-byte runs on both sides
constexpr int TB_BLOCKS = TB_TILE / 64;
constexpr int TB_THREADS = 32 * TB_BLOCKS;
constexpr int TB_PITCH = TB_BLOCKS + 1; // words per staged output row (+1 pad: conflict-free 8-byte accesses)

__global__ void __launch_bounds__(TB_THREADS)
k_transpose_bits(const uint64_t* __restrict__ in, uint64_t* __restrict__ out,
                 int64_t R, int64_t C, int64_t wpr_in, int64_t wpr_out, int64_t gx, int64_t gy, int64_t sgx) {
    __shared__ uint64_t stage[TB_TILE * TB_PITCH];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t b = blockIdx.y;
    // Tiles run in 8 x 8 groups: the CTAs that are resident together then read 512-byte runs of
    // the input rows and write 512-byte runs of the output rows between them, instead of one
    // 64-byte run per DRAM page.
    const int64_t grp = (int64_t)blockIdx.x >> 6;
    const int in_grp = (int)(blockIdx.x & 63);
    const int64_t tx = (grp % sgx) * 8 + (in_grp & 7), ty = (grp / sgx) * 8 + (in_grp >> 3);
    if (tx >= gx || ty >= gy) return;
    const int64_t r0 = ty * TB_TILE;                               // first input row of the tile
    const int64_t cw0 = tx * TB_BLOCKS;                            // first input word (column block) of the tile
    const uint64_t* inb = in + b * R * wpr_in;
    uint64_t* outb = out + b * C * wpr_out;

    // warp w: rows [r0 + 64 w, +64) of the tile, all TB_BLOCKS column blocks; lane L: rows L and L + 32
    uint64_t lo[TB_BLOCKS], hi[TB_BLOCKS];
    {
        const int64_t ra = r0 + 64 * warp + lane, rb = ra + 32;
        const uint64_t* pa = inb + ra * wpr_in + cw0;
        const uint64_t* pb = inb + rb * wpr_in + cw0;
        const bool full = cw0 + TB_BLOCKS <= wpr_in && (wpr_in & 1) == 0 && (reinterpret_cast<uintptr_t>(inb) & 15u) == 0;
        if (full && rb < R) {
#pragma unroll
            for (int cb = 0; cb < TB_BLOCKS; cb += 2) {
                const uint4 va = ldg_stream(pa + cb), vb = ldg_stream(pb + cb);
                lo[cb] = (uint64_t)va.x | ((uint64_t)va.y << 32); lo[cb + 1] = (uint64_t)va.z | ((uint64_t)va.w << 32);
                hi[cb] = (uint64_t)vb.x | ((uint64_t)vb.y << 32); hi[cb + 1] = (uint64_t)vb.z | ((uint64_t)vb.w << 32);
            }
        } else {
#pragma unroll
            for (int cb = 0; cb < TB_BLOCKS; ++cb) {
                const bool okw = cw0 + cb < wpr_in;
                lo[cb] = (ra < R && okw) ? __ldg(pa + cb) : 0ull;
                hi[cb] = (rb < R && okw) ? __ldg(pb + cb) : 0ull;
            }
        }
    }
#pragma unroll
    for (int cb = 0; cb < TB_BLOCKS; ++cb) {
        transpose64x64(lo[cb], hi[cb], lane);
        stage[(64 * cb + lane) * TB_PITCH + warp] = lo[cb];
        stage[(64 * cb + 32 + lane) * TB_PITCH + warp] = hi[cb];
    }
    __syncthreads();
    const int64_t ow0 = ty * TB_BLOCKS;                             // first output word of the tile's rows
#pragma unroll
    for (int k = 0; k < TB_TILE / TB_THREADS; ++k) {
        const int orow = tid + TB_THREADS * k;
        const int64_t c = cw0 * 64 + orow;                          // output row = input bit column
        if (c >= C) continue;
        uint64_t* dst = outb + c * wpr_out + ow0;
        const uint64_t* src = stage + orow * TB_PITCH;
        if (ow0 + TB_BLOCKS <= wpr_out && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
            for (int w = 0; w < TB_BLOCKS; w += 2)
                stg_stream(dst + w, make_uint4((uint32_t)src[w], (uint32_t)(src[w] >> 32), (uint32_t)src[w + 1], (uint32_t)(src[w + 1] >> 32)));
        } else {
#pragma unroll
            for (int w = 0; w < TB_BLOCKS; ++w) if (ow0 + w < wpr_out) dst[w] = src[w];
        }
    }
}

template <bool IS_OR>
__global__ void __launch_bounds__(256)
k_reduce_rows(const uint64_t* __restrict__ in, unsigned long long* __restrict__ out,
              int64_t R, int64_t inner, int64_t rows_per_chunk) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= inner) return;
    const int64_t o = blockIdx.z;
    const int64_t ra = (int64_t)blockIdx.y * rows_per_chunk;
    const int64_t rb = ra + rows_per_chunk < R ? ra + rows_per_chunk : R;
    const uint64_t* p = in + (o * R + ra) * inner + i;
    uint64_t acc = IS_OR ? 0ull : ~0ull;
    int64_t r = ra;
    for (; r + 4 <= rb; r += 4, p += 4 * inner) {         // four independent loads in flight
        const uint64_t a = __ldg(p), b = __ldg(p + inner), c = __ldg(p + 2 * inner), d = __ldg(p + 3 * inner);
        acc = IS_OR ? (acc | a | b | c | d) : (acc & a & b & c & d);
    }
    for (; r < rb; ++r, p += inner) acc = IS_OR ? (acc | __ldg(p)) : (acc & __ldg(p));
    if (IS_OR) { if (acc != 0ull) atomicOr(out + o * inner + i, acc); }
    else       { if (acc != ~0ull) atomicAnd(out + o * inner + i, acc); }
}

}  // namespace bb

using namespace bb;

extern "C" int brute_b200_transpose_bits(const uint64_t* in, uint64_t* out,
                                         int64_t batch, int64_t R, int64_t C, void* stream) {
    BB_REQUIRE(batch >= 0 && R >= 0 && C >= 0, BRUTE_ERR_INVALID_ARG);
    if (batch == 0 || C == 0) return BRUTE_OK;
    const int64_t wpr_in = (C + 63) / 64, wpr_out = (R + 63) / 64;
    if (R == 0) return BRUTE_OK;                           // output rows have no words
    BB_REQUIRE(in != nullptr && out != nullptr && in != out, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(in) && aligned8(out), BRUTE_ERR_MISALIGNED);
    const int64_t gx = (wpr_in + TB_BLOCKS - 1) / TB_BLOCKS, gy = (R + TB_TILE - 1) / TB_TILE;
    const int64_t sgx = (gx + 7) / 8, sgy = (gy + 7) / 8;
    BB_REQUIRE(sgx * sgy * 64 <= 0x7fffffffll && batch <= 65535, BRUTE_ERR_UNSUPPORTED);
    k_transpose_bits<<<dim3((unsigned)(sgx * sgy * 64), (unsigned)batch), TB_THREADS, 0, as_stream(stream)>>>(
        in, out, R, C, wpr_in, wpr_out, gx, gy, sgx);
    return launch_status();
}

extern "C" int brute_b200_reduce_rows(int op, const uint64_t* in, uint64_t* out,
                                      int64_t outer, int64_t R, int64_t inner, void* stream) {
    BB_REQUIRE(op == BRUTE_OP_OR || op == BRUTE_OP_AND, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(outer >= 0 && R >= 0 && inner >= 0, BRUTE_ERR_INVALID_ARG);
    if (outer == 0 || inner == 0) return BRUTE_OK;
    BB_REQUIRE(out != nullptr && (R == 0 || in != nullptr), BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(in) && aligned8(out), BRUTE_ERR_MISALIGNED);
    BB_REQUIRE(outer <= 65535, BRUTE_ERR_UNSUPPORTED);
    cudaStream_t st = as_stream(stream);
    // identity of the reduction; an empty axis leaves it (any -> 0, all -> ~0, as torch does)
    if (cudaMemsetAsync(out, op == BRUTE_OP_OR ? 0x00 : 0xFF, (size_t)(outer * inner) * 8, st) != cudaSuccess)
        return BRUTE_ERR_LAUNCH;
    if (R == 0) return BRUTE_OK;
    const int64_t gx = (inner + 255) / 256;
    BB_REQUIRE(gx <= 0x7fffffffll, BRUTE_ERR_UNSUPPORTED);
    // enough row chunks to put about 8 blocks on every SM, at least 16 rows each
    int64_t chunks = (8 * (int64_t)kNumSMs + gx * outer - 1) / (gx * outer);
    if (chunks > (R + 15) / 16) chunks = (R + 15) / 16;
    if (chunks < 1) chunks = 1;
    if (chunks > 65535) chunks = 65535;
    const int64_t rows_per_chunk = (R + chunks - 1) / chunks;
    const dim3 grid((unsigned)gx, (unsigned)((R + rows_per_chunk - 1) / rows_per_chunk), (unsigned)outer);
    if (op == BRUTE_OP_OR)
        k_reduce_rows<true><<<grid, 256, 0, st>>>(in, reinterpret_cast<unsigned long long*>(out), R, inner, rows_per_chunk);
    else
        k_reduce_rows<false><<<grid, 256, 0, st>>>(in, reinterpret_cast<unsigned long long*>(out), R, inner, rows_per_chunk);
    return launch_status();
}
