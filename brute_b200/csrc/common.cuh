// Shared helpers for the brute_b200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/brute_b200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "brute_b200 kernels are written for sm_100a only"
#endif

namespace bb {

constexpr int kNumSMs = 148;           // B200: 2 dies x 74 SMs
constexpr int kWarp   = 32;

// ---- host-side argument checks ------------------------------------------
#define BB_REQUIRE(cond, code) do { if (!(cond)) return (code); } while (0)

inline int launch_status() {
    return cudaGetLastError() == cudaSuccess ? BRUTE_OK : BRUTE_ERR_LAUNCH;
}

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned8(const void* p)  { return (reinterpret_cast<uintptr_t>(p) & 7u) == 0; }

// Grid for a streaming kernel: a whole number of waves over the SMs, never
// more blocks than there is work for.
inline int stream_grid(int64_t work_items, int items_per_block, int blocks_per_sm) {
    int64_t need = (work_items + items_per_block - 1) / items_per_block;
    int64_t cap  = (int64_t)kNumSMs * blocks_per_sm;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

// ---- device helpers ------------------------------------------------------
#ifdef __CUDACC__

// Grid of a persistent grid-stride kernel: exactly the blocks that are resident
// at once (SMs x occupancy), so there is no second, partial wave.
template <class Kernel>
inline int resident_grid(Kernel kernel, int block_threads, int64_t blocks_needed) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, block_threads, 0) != cudaSuccess || per_sm < 1)
        per_sm = 1;
    const int64_t cap = (int64_t)kNumSMs * per_sm;
    if (blocks_needed < 1) blocks_needed = 1;
    return (int)(blocks_needed < cap ? blocks_needed : cap);
}

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device setting of a kernel: remember per
// device (not per process) where it has been made, so that one process may drive several GPUs.
template <auto Kernel>
inline bool kernel_smem_ready(int bytes) {
    static unsigned long long done_mask = 0;       // bit d: device d is set up (devices >= 64: every call)
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess) return false;
    if (d >= 0 && d < 64 && ((done_mask >> d) & 1ull)) return true;
    if (cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
    if (d >= 0 && d < 64) done_mask |= 1ull << d;
    return true;
}

// 128-bit streaming load that does not allocate in L1.
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void stg_stream(void* p, uint4 v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// 4 bytes (each zero / nonzero) -> 4 bits, bit i = (byte i != 0).
__device__ __forceinline__ uint32_t nonzero_bytes_to_bits(uint32_t w) {
    // high bit of each byte set iff the byte is nonzero
    uint32_t nz = (((w & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | w) & 0x80808080u;
    // gather bits 7,15,23,31 into bits 24..27: one multiply, no carries collide
    return (((nz >> 7) * 0x01020408u) >> 24) & 0xFu;
}

// 16 bytes -> 16 bits
__device__ __forceinline__ uint32_t nonzero_bytes_to_bits16(uint4 v) {
    return nonzero_bytes_to_bits(v.x) | (nonzero_bytes_to_bits(v.y) << 4) |
           (nonzero_bytes_to_bits(v.z) << 8) | (nonzero_bytes_to_bits(v.w) << 12);
}

// 4 bits -> 4 bytes of 0/1, byte i = bit i.
__device__ __forceinline__ uint32_t bits4_to_bytes01(uint32_t nib) {
    return ((nib & 0xFu) * 0x00204081u) & 0x01010101u;
}

__device__ __forceinline__ uint64_t warp_sum_u64(uint64_t v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Block-wide sum; result valid in thread 0. `red` holds 32 slots.
__device__ __forceinline__ uint64_t block_sum_u64(uint64_t v, uint64_t* red) {
    v = warp_sum_u64(v);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) red[wid] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    v = (threadIdx.x < nw) ? red[threadIdx.x] : 0;
    if (wid == 0) v = warp_sum_u64(v);
    return v;
}

// 64 x 64 bit-matrix transpose in registers (the butterfly: swap the off-diagonal 32 x 32 quadrants,
// then 16 x 16 inside each, ... down to 1 x 1).
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

#endif  // __CUDACC__

}  // namespace bb
