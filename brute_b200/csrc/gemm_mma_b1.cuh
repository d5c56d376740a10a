// xnor-popcount GEMM on the legacy warp-level binary MMA:
//   mma.sync.aligned.m16n8k256.row.col.s32.b1.b1.s32.xor.popc
// which accumulates popcount(a ^ b) directly, so C = K - 2*acc needs no side
// vectors. 128x128 CTA tile, 8 warps of 64x32, K slices of 512 bits staged with
// cp.async (3 stages). Rows are padded to 96 bytes in shared memory so that the
// 8-byte fragment loads of a half-warp fall in 16 distinct bank pairs.
//
// The k index inside a 256-bit step is permuted (a thread loads 8 adjacent
// bytes for its two k-registers); A and B use the same permutation, which a
// popcount contraction cannot see.
#pragma once
#include "common.cuh"

namespace bb {

constexpr int MB_BM = 128, MB_BN = 128, MB_THREADS = 256, MB_STAGES = 3;
constexpr int MB_BK_BYTES = 64;             // 512 bits of K per stage
constexpr int MB_ROW = 96;                  // padded row pitch in shared memory
constexpr int MB_STAGE_BYTES = (MB_BM + MB_BN) * MB_ROW;
constexpr int MB_SMEM = MB_STAGES * MB_STAGE_BYTES;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory");
}

__device__ __forceinline__ void mma_b1_xor(int32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k256.row.col.s32.b1.b1.s32.xor.popc "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// PACK = false: C int32 [M, ldc]. PACK = true: bits sign(scale[n]*c) to out32
// (the packed output viewed as 32-bit halves, 2*wpr_out per row).
template <bool PACK>
__global__ void __launch_bounds__(MB_THREADS)
k_xnor_gemm_mma_b1(const uint8_t* __restrict__ A, const uint8_t* __restrict__ B,
                   int64_t M, int64_t N, int64_t Kbytes /* 8*Kp */, int32_t K,
                   int32_t* __restrict__ C, int64_t ldc,
                   const float* __restrict__ scale, uint32_t* __restrict__ out32, int64_t halves_per_row,
                   int mode) {
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 2, wn = warp & 3;            // 2 x 4 warps
    const int g = lane >> 2, t = lane & 3;
    const int64_t m0 = (int64_t)blockIdx.y * MB_BM, n0 = (int64_t)blockIdx.x * MB_BN;
    const int64_t nslices = (Kbytes + MB_BK_BYTES - 1) / MB_BK_BYTES;

    auto load_stage = [&](int stage, int64_t slice) {
        // 256 rows x 4 chunks of 16 bytes; 4 chunks per thread
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = tid + it * MB_THREADS;      // 0..1023
            const int row = idx >> 2, ch = idx & 3;     // row 0..127: A, 128..255: B
            const bool isA = row < MB_BM;
            const int64_t grow = isA ? m0 + row : n0 + (row - MB_BM);
            const int64_t kb = slice * MB_BK_BYTES + ch * 16;
            int bytes = 0;
            if (grow < (isA ? M : N) && kb < Kbytes) bytes = (int)((Kbytes - kb) < 16 ? (Kbytes - kb) : 16);
            const uint8_t* src = (isA ? A : B) + (bytes ? grow * Kbytes + kb : 0);
            cp_async16(smem_base + stage * MB_STAGE_BYTES + row * MB_ROW + ch * 16, src, bytes);
        }
    };

    int32_t acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[i][j][c] = 0;

#pragma unroll
    for (int s = 0; s < MB_STAGES - 1; ++s) {
        if (s < nslices) load_stage(s, s);
        cp_async_commit();
    }
    for (int64_t sl = 0; sl < nslices; ++sl) {
        cp_async_wait<MB_STAGES - 2>();
        __syncthreads();
        const int64_t nxt = sl + MB_STAGES - 1;
        if (nxt < nslices) load_stage((int)(nxt % MB_STAGES), nxt);
        cp_async_commit();
        const uint8_t* st = smem + (sl % MB_STAGES) * MB_STAGE_BYTES;
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            uint2 bf[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                bf[j] = *reinterpret_cast<const uint2*>(st + (MB_BM + wn * 32 + j * 8 + g) * MB_ROW + kk * 32 + t * 8);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint8_t* ar = st + (wm * 64 + i * 16 + g) * MB_ROW + kk * 32 + t * 8;
                const uint2 lo = *reinterpret_cast<const uint2*>(ar);
                const uint2 hi = *reinterpret_cast<const uint2*>(ar + 8 * MB_ROW);
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_b1_xor(acc[i][j], lo.x, hi.x, lo.y, hi.y, bf[j].x, bf[j].y);
            }
        }
    }
    cp_async_wait<0>();

    // epilogue: thread holds rows (g, g+8) and columns (2t, 2t+1) of each 16x8 tile
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int64_t m = m0 + wm * 64 + i * 16 + g + 8 * h;
            if (!PACK) {
                if (m < M) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int64_t n = n0 + wn * 32 + j * 8 + 2 * t;
                        const int32_t v0 = K - 2 * acc[i][j][2 * h], v1 = K - 2 * acc[i][j][2 * h + 1];
                        int32_t* dst = C + m * ldc + n;
                        if (n + 1 < N && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0)
                            *reinterpret_cast<int2*>(dst) = make_int2(v0, v1);
                        else { if (n < N) dst[0] = v0; if (n + 1 < N) dst[1] = v1; }
                    }
                }
            } else {
                uint32_t bits = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int64_t n = n0 + wn * 32 + j * 8 + 2 * t + e;
                        if (n < N) {
                            const float y = __ldg(scale + n) * (float)(K - 2 * acc[i][j][2 * h + e]);
                            const bool b = mode == BRUTE_SIGN_GE0 ? (y >= 0.0f) : (y > 0.0f);
                            bits |= (b ? 1u : 0u) << (j * 8 + 2 * t + e);
                        }
                    }
                }
                bits |= __shfl_xor_sync(0xffffffffu, bits, 1);
                bits |= __shfl_xor_sync(0xffffffffu, bits, 2);
                const int64_t half = (n0 + wn * 32) >> 5;
                if (t == 0 && m < M && half < halves_per_row) out32[m * halves_per_row + half] = bits;
            }
        }
    }
}

}  // namespace bb
