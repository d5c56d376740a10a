// Transport form of the GEMM result for the all-gather of a column-sharded GEMM.
//
// C = K - 2H lies in [-K, K]: for K <= 32767 an int16 carries it exactly, so the ranks exchange
// int16 blocks (half the NVLink bytes of the int32 result) and every rank widens what it received
// straight into its replicated int32 matrix. The widening pass also does the layout change that the
// gather leaves behind: NCCL delivers the rank blocks stacked, [world, rows, n_loc], and the result
// is row major [rows, world * n_loc].
// Both kernels are HBM bound; 128-bit loads and stores, grid sized to the SMs.
#include "common.cuh"

namespace bb {

// 8 int32 -> 8 int16 per thread trip
__global__ void __launch_bounds__(256)
k_narrow_i32_i16(const int32_t* __restrict__ in, int16_t* __restrict__ out, int64_t n8) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
        const uint4 a = ldg_stream(in + i * 8), b = ldg_stream(in + i * 8 + 4);
        uint4 o;
        o.x = (a.x & 0xFFFFu) | (a.y << 16);
        o.y = (a.z & 0xFFFFu) | (a.w << 16);
        o.z = (b.x & 0xFFFFu) | (b.y << 16);
        o.w = (b.z & 0xFFFFu) | (b.w << 16);
        stg_stream(out + i * 8, o);
    }
}

__global__ void __launch_bounds__(256)
k_narrow_i32_i16_tail(const int32_t* __restrict__ in, int16_t* __restrict__ out, int64_t from, int64_t n) {
    const int64_t i = from + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = (int16_t)in[i];
}

__device__ __forceinline__ int32_t sx16(uint32_t v) { return (int32_t)(int16_t)(v & 0xFFFFu); }

// in [world, rows, n_loc] (ELEM = int16 or int32) -> out[m * ldc + r * n_loc + j] int32.
// One thread moves 8 consecutive j of one (r, m); n_loc is a multiple of 8 here.
template <typename ELEM>
__global__ void __launch_bounds__(256)
k_unstack_rank_blocks(const ELEM* __restrict__ in, int32_t* __restrict__ out,
                      int64_t world, int64_t rows, int64_t n_loc, int64_t ldc) {
    const int64_t v_per_row = n_loc / 8;                     // vectors of 8 per (r, m)
    const int64_t total = world * rows * v_per_row;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        // i walks the OUTPUT in row-major order, so that stores of a warp are contiguous
        const int64_t m = i / (world * v_per_row);
        const int64_t rem = i - m * (world * v_per_row);
        const int64_t r = rem / v_per_row, v = rem - r * v_per_row;
        const ELEM* src = in + ((r * rows + m) * n_loc + v * 8);
        int32_t* dst = out + m * ldc + r * n_loc + v * 8;
        if (sizeof(ELEM) == 2) {
            const uint4 a = ldg_stream(src);
            stg_stream(dst,     make_uint4((uint32_t)sx16(a.x), (uint32_t)sx16(a.x >> 16), (uint32_t)sx16(a.y), (uint32_t)sx16(a.y >> 16)));
            stg_stream(dst + 4, make_uint4((uint32_t)sx16(a.z), (uint32_t)sx16(a.z >> 16), (uint32_t)sx16(a.w), (uint32_t)sx16(a.w >> 16)));
        } else {
            stg_stream(dst, ldg_stream(src));
            stg_stream(dst + 4, ldg_stream(reinterpret_cast<const int32_t*>(src) + 4));
        }
    }
}

template <typename ELEM>
__global__ void __launch_bounds__(256)
k_unstack_rank_blocks_scalar(const ELEM* __restrict__ in, int32_t* __restrict__ out,
                             int64_t world, int64_t rows, int64_t n_loc, int64_t ldc) {
    const int64_t total = world * rows * n_loc;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t m = i / (world * n_loc);
        const int64_t rem = i - m * (world * n_loc);
        const int64_t r = rem / n_loc, j = rem - r * n_loc;
        out[m * ldc + r * n_loc + j] = (int32_t)in[(r * rows + m) * n_loc + j];
    }
}

}  // namespace bb

using namespace bb;

extern "C" int brute_b200_narrow_i32_i16(const int32_t* in, int16_t* out, int64_t n, void* stream) {
    BB_REQUIRE(n >= 0, BRUTE_ERR_INVALID_ARG);
    if (n == 0) return BRUTE_OK;
    BB_REQUIRE(in != nullptr && out != nullptr, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE((reinterpret_cast<uintptr_t>(in) & 3u) == 0 && (reinterpret_cast<uintptr_t>(out) & 1u) == 0,
               BRUTE_ERR_MISALIGNED);
    cudaStream_t st = as_stream(stream);
    const int64_t n8 = (aligned16(in) && aligned16(out)) ? n / 8 : 0;
    if (n8 > 0) {
        k_narrow_i32_i16<<<stream_grid(n8, 256, 8), 256, 0, st>>>(in, out, n8);
        if (int rc = launch_status()) return rc;
    }
    const int64_t rest = n - n8 * 8;
    if (rest > 0) {
        k_narrow_i32_i16_tail<<<(unsigned)((rest + 255) / 256), 256, 0, st>>>(in, out, n8 * 8, n);
    }
    return launch_status();
}

extern "C" int brute_b200_unstack_rank_blocks(const void* in, int elem_bytes, int32_t* out,
                                              int64_t world, int64_t rows, int64_t n_loc, int64_t ldc, void* stream) {
    BB_REQUIRE(world >= 0 && rows >= 0 && n_loc >= 0 && ldc >= world * n_loc, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(elem_bytes == 2 || elem_bytes == 4, BRUTE_ERR_UNSUPPORTED);
    if (world * rows * n_loc == 0) return BRUTE_OK;
    BB_REQUIRE(in != nullptr && out != nullptr && in != out, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE((reinterpret_cast<uintptr_t>(in) & (uintptr_t)(elem_bytes - 1)) == 0 &&
               (reinterpret_cast<uintptr_t>(out) & 3u) == 0, BRUTE_ERR_MISALIGNED);
    cudaStream_t st = as_stream(stream);
    const bool vec = (n_loc % 8 == 0) && (ldc % 4 == 0) && aligned16(in) && aligned16(out);
    if (vec) {
        const int grid = stream_grid(world * rows * (n_loc / 8), 256, 8);
        if (elem_bytes == 2) k_unstack_rank_blocks<int16_t><<<grid, 256, 0, st>>>(static_cast<const int16_t*>(in), out, world, rows, n_loc, ldc);
        else                 k_unstack_rank_blocks<int32_t><<<grid, 256, 0, st>>>(static_cast<const int32_t*>(in), out, world, rows, n_loc, ldc);
    } else {
        const int grid = stream_grid(world * rows * n_loc, 256, 8);
        if (elem_bytes == 2) k_unstack_rank_blocks_scalar<int16_t><<<grid, 256, 0, st>>>(static_cast<const int16_t*>(in), out, world, rows, n_loc, ldc);
        else                 k_unstack_rank_blocks_scalar<int32_t><<<grid, 256, 0, st>>>(static_cast<const int32_t*>(in), out, world, rows, n_loc, ldc);
    }
    return launch_status();
}
