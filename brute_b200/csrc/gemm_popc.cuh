// CUDA-core xnor-popcount GEMM: register-blocked __popcll, any shape.
//
// This is the instruction path that needs no tensor-core mapping of the binary
// contraction. A 128x128 tile of C per CTA, 8x8 outputs per thread, operands
// staged through shared memory in 8-word (512-bit) K slices, so every packed
// word is read from L2 once per CTA and reused 128 times. The POPC pipe bounds
// it (two 32-bit POPC per 64 bit-MACs).
#pragma once
#include "common.cuh"

namespace bb {

constexpr int PG_BM = 128, PG_BN = 128, PG_BK = 8, PG_THREADS = 256;

// Epilogue functor interface: store(m, n0, vals[8]) for 8 consecutive n.
struct EpilogueInt32 {
    int32_t* C; int64_t ldc; int64_t M, N;
    __device__ __forceinline__ void tile_row(int64_t m, int64_t n0, const int32_t* v) const {
        if (m >= M) return;
        int32_t* dst = C + m * ldc + n0;
        if (n0 + 8 <= N && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
            *reinterpret_cast<int4*>(dst)     = make_int4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<int4*>(dst + 4) = make_int4(v[4], v[5], v[6], v[7]);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) if (n0 + j < N) dst[j] = v[j];
        }
    }
};

// Fused binarised-MLP epilogue: bit = sign(scale[n] * c), 8 threads of a warp
// (consecutive lanes) own the 64 columns of one output word.
struct EpilogueScaleSignPack {
    const float* scale; uint64_t* out; int64_t wpr_out; int64_t M, N; int mode;
    __device__ __forceinline__ void tile_row(int64_t m, int64_t n0, const int32_t* v) const {
        uint32_t byte = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (n0 + j < N) {
                const float y = __ldg(scale + n0 + j) * (float)v[j];
                const bool b = mode == BRUTE_SIGN_GE0 ? (y >= 0.0f) : (y > 0.0f);
                byte |= (b ? 1u : 0u) << j;
            }
        }
        // lanes l..l+7 (l % 8 == 0) hold bytes 0..7 of the word
        const int lane = threadIdx.x & 31;
        uint64_t w = (uint64_t)byte << (8 * (lane & 7));
        w |= __shfl_xor_sync(0xffffffffu, w, 1);
        w |= __shfl_xor_sync(0xffffffffu, w, 2);
        w |= __shfl_xor_sync(0xffffffffu, w, 4);
        if ((lane & 7) == 0 && m < M && n0 < N) out[m * wpr_out + (n0 >> 6)] = w;
    }
};

template <class Epilogue>
__global__ void __launch_bounds__(PG_THREADS)
k_xnor_gemm_popc(const uint64_t* __restrict__ A, const uint64_t* __restrict__ B,
                 int64_t M, int64_t N, int64_t Kp, int32_t K, Epilogue ep) {
    // [k][row] so that a thread's 8 consecutive rows are one 64-byte span
    __shared__ __align__(16) uint64_t As[PG_BK][PG_BM];
    __shared__ __align__(16) uint64_t Bs[PG_BK][PG_BN];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 8 x 8 outputs each
    const int64_t m0 = (int64_t)blockIdx.y * PG_BM, n0 = (int64_t)blockIdx.x * PG_BN;

    int32_t acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0;

    for (int64_t k0 = 0; k0 < Kp; k0 += PG_BK) {
        // 128 rows x 8 words per operand = 1024 words; 4 per thread and operand
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = tid + it * PG_THREADS;   // 0..1023
            const int row = idx >> 3, kk = idx & 7;
            const int64_t k = k0 + kk;
            uint64_t a = 0, b = 0;
            if (k < Kp) {
                if (m0 + row < M) a = __ldg(A + (m0 + row) * Kp + k);
                if (n0 + row < N) b = __ldg(B + (n0 + row) * Kp + k);
            }
            As[kk][row] = a;
            Bs[kk][row] = b;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < PG_BK; ++kk) {
            uint64_t a[8], b[8];
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
                const ulonglong2 va = *reinterpret_cast<const ulonglong2*>(&As[kk][ty * 8 + i]);
                const ulonglong2 vb = *reinterpret_cast<const ulonglong2*>(&Bs[kk][tx * 8 + i]);
                a[i] = va.x; a[i + 1] = va.y; b[i] = vb.x; b[i + 1] = vb.y;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] += __popcll(a[i] ^ b[j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int32_t v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = K - 2 * acc[i][j];
        ep.tile_row(m0 + ty * 8 + i, n0 + tx * 8, v);
    }
}

}  // namespace bb
