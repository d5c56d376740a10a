// Fused binary attention forward.
//
//   score(i,j) = (D - 2*popcount(q_i ^ k_j)) * scale      (integer popcount scores)
//   P = softmax_j(score) in fp32, optional causal mask
//   O = P @ V, V and O in bf16, fp32 accumulation on the tensor cores
//
// A score takes only D+1 values, one per Hamming distance h, so
// exp(score - rowmax) = rowfactor * T[h] with T[h] = exp(-2*scale*h) and the row
// factor cancels between numerator and denominator of the softmax. The TABLE
// kernel therefore keeps T in shared memory (fp32, T <= 1, every term positive)
// and needs no running maximum, no exp and no rescaling of O: blockwise softmax
// without the "online" bookkeeping. It is used while exp(-2*|scale|*D) stays a
// normal fp32 number; steeper scales take the ONLINE kernel (running max, exp2).
//
// One CTA owns 128 query rows of one (batch, head); 8 warps of 16 rows. K (packed
// words) and V (bf16) stream through shared memory in 64-key tiles with a
// two-deep cp.async pipeline. Each thread computes the scores that land in ITS
// lanes of the m16n8k16 A-fragment directly with XOR + POPC from the packed Q
// words it keeps in registers, so P never leaves registers between the score
// stage and the P@V MMA. V fragments come from ldmatrix.trans on a 16-byte
// XOR-swizzled tile.
#include "common.cuh"
#include <cstdlib>
#include <cstring>

namespace bb {

constexpr int AT_BM = 128, AT_BN = 64, AT_THREADS = 256;

__device__ __forceinline__ void at_cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void at_cp_async8(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" :: "r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// D = 64*W. V tile row = D bf16 = 2*D bytes = D/8 chunks of 16 bytes; chunk c of
// row r is stored at chunk (c ^ (r & 7)).
template <int W>
__global__ void __launch_bounds__(AT_THREADS)
k_binary_attention_fwd(const uint64_t* __restrict__ Qp, const uint64_t* __restrict__ Kp,
                       const __nv_bfloat16* __restrict__ V, __nv_bfloat16* __restrict__ O,
                       int64_t S, int causal, float scale_log2, int64_t q_tiles) {
    constexpr int D = 64 * W;
    constexpr int VROW = D * 2;                 // bytes per V row
    constexpr int VCH = D / 8;                  // 16-byte chunks per V row
    constexpr int NT = D / 8;                   // n8 tiles of the output
    __shared__ __align__(16) uint64_t Ks[2][AT_BN * W];
    __shared__ __align__(128) uint8_t Vs[2][AT_BN * VROW];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    // heavy (late) query tiles first: under a causal mask they have the most keys
    const int64_t qt = q_tiles - 1 - (int64_t)blockIdx.x;
    const int64_t bh = blockIdx.y;
    const int64_t q0 = qt * AT_BM;
    const uint64_t* Qb = Qp + bh * S * W;
    const uint64_t* Kb = Kp + bh * S * W;
    const __nv_bfloat16* Vb = V + bh * S * D;
    __nv_bfloat16* Ob = O + bh * S * D;

    const int64_t row_lo = q0 + warp * 16 + g, row_hi = row_lo + 8;
    uint64_t q[2][W];
#pragma unroll
    for (int w = 0; w < W; ++w) {
        q[0][w] = row_lo < S ? __ldg(Qb + row_lo * W + w) : 0ull;
        q[1][w] = row_hi < S ? __ldg(Qb + row_hi * W + w) : 0ull;
    }

    const int64_t kend = causal ? (q0 + AT_BM < S ? q0 + AT_BM : S) : S;   // keys [0, kend)
    const int64_t ntiles = (kend + AT_BN - 1) / AT_BN;
    const uint32_t ks_base = (uint32_t)__cvta_generic_to_shared(&Ks[0][0]);
    const uint32_t vs_base = (uint32_t)__cvta_generic_to_shared(&Vs[0][0]);

    auto load_tile = [&](int buf, int64_t tile) {
        const int64_t k0 = tile * AT_BN;
        // K: 64 keys x W words
        if (tid < AT_BN * W) {
            const int key = tid / W, w = tid % W;
            const bool ok = k0 + key < S;
            at_cp_async8(ks_base + (buf * AT_BN * W + tid) * 8, Kb + (ok ? (k0 + key) * W + w : 0), ok ? 8 : 0);
        }
        // V: 64 rows x VCH chunks
#pragma unroll
        for (int it = 0; it < (AT_BN * VCH) / AT_THREADS; ++it) {
            const int idx = tid + it * AT_THREADS;
            const int row = idx / VCH, ch = idx % VCH;
            const bool ok = k0 + row < S;
            const int sch = (ch & ~7) | ((ch ^ row) & 7);
            at_cp_async16(vs_base + buf * AT_BN * VROW + row * VROW + sch * 16,
                          Vb + (ok ? (k0 + row) * D + ch * 8 : 0), ok ? 16 : 0);
        }
    };

    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};

    if (ntiles > 0) load_tile(0, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");

    for (int64_t tile = 0; tile < ntiles; ++tile) {
        const int buf = (int)(tile & 1);
        if (tile + 1 < ntiles) load_tile(buf ^ 1, tile + 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();

        const int64_t k0 = tile * AT_BN;
        // a warp whose rows all precede this tile has nothing to add
        const bool active = !(causal && k0 > q0 + warp * 16 + 15);
        if (active) {
            // ---- scores: s[h][kb][c], h = row half, kb = 16-key block, c: 0,1 -> cols 2t,2t+1; 2,3 -> 2t+8,2t+9
            float s[2][4][4];
            const bool need_mask = (causal && k0 + AT_BN - 1 > q0 + warp * 16) || (k0 + AT_BN > S);
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int key = kb * 16 + 2 * t + (c & 1) + ((c >> 1) << 3);
                    int h0 = 0, h1 = 0;
#pragma unroll
                    for (int w = 0; w < W; ++w) {
                        const uint64_t kw = Ks[buf][key * W + w];
                        h0 += __popcll(q[0][w] ^ kw);
                        h1 += __popcll(q[1][w] ^ kw);
                    }
                    float s0 = (float)(D - 2 * h0) * scale_log2;
                    float s1 = (float)(D - 2 * h1) * scale_log2;
                    if (need_mask) {
                        const int64_t kidx = k0 + key;
                        if (kidx >= S || (causal && kidx > row_lo)) s0 = -INFINITY;
                        if (kidx >= S || (causal && kidx > row_hi)) s1 = -INFINITY;
                    }
                    s[0][kb][c] = s0;
                    s[1][kb][c] = s1;
                }
            }
            // ---- online softmax (log2 domain)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float mx = -INFINITY;
#pragma unroll
                for (int kb = 0; kb < 4; ++kb)
#pragma unroll
                    for (int c = 0; c < 4; ++c) mx = fmaxf(mx, s[h][kb][c]);
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float mnew = fmaxf(mrow[h], mx);
                // mnew stays -inf only if every key so far was masked for this row
                const float msafe = mnew == -INFINITY ? 0.f : mnew;
                const float alpha = exp2f(mrow[h] - msafe);
                float sum = 0.f;
#pragma unroll
                for (int kb = 0; kb < 4; ++kb)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float p = exp2f(s[h][kb][c] - msafe);
                        s[h][kb][c] = p;
                        sum += p;
                    }
                lrow[h] = lrow[h] * alpha + sum;
                mrow[h] = mnew;
#pragma unroll
                for (int j = 0; j < NT; ++j) { o[j][2 * h] *= alpha; o[j][2 * h + 1] *= alpha; }
            }
            // ---- O += P @ V
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
                const uint32_t a0 = pack_bf16x2(s[0][kb][0], s[0][kb][1]);
                const uint32_t a1 = pack_bf16x2(s[1][kb][0], s[1][kb][1]);
                const uint32_t a2 = pack_bf16x2(s[0][kb][2], s[0][kb][3]);
                const uint32_t a3 = pack_bf16x2(s[1][kb][2], s[1][kb][3]);
                const int vrow = kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
                for (int j = 0; j < NT; j += 2) {
                    const int ch = j + (lane >> 4);
                    const int sch = (ch & ~7) | ((ch ^ vrow) & 7);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(vs_base + buf * AT_BN * VROW + vrow * VROW + sch * 16, b0, b1, b2, b3);
                    mma_bf16_16816(o[j], a0, a1, a2, a3, b0, b1);
                    mma_bf16_16816(o[j + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
        __syncthreads();   // everyone is done with `buf` before it is refilled
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // ---- finalise: divide by the row sums, stage through shared memory, 16-byte stores
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float l = lrow[h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int r = warp * 16 + g + 8 * h;         // row within the CTA tile
        if (AT_BM * VROW <= 2 * AT_BN * VROW) {
            uint8_t* srow = &Vs[0][0] + r * VROW;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int sch = (j & ~7) | ((j ^ r) & 7);
                *reinterpret_cast<uint32_t*>(srow + sch * 16 + t * 4) =
                    pack_bf16x2(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < (AT_BM * VCH) / AT_THREADS; ++it) {
        const int idx = tid + it * AT_THREADS;
        const int r = idx / VCH, ch = idx % VCH;
        const int sch = (ch & ~7) | ((ch ^ r) & 7);
        if (q0 + r < S) {
            const uint4 v = *reinterpret_cast<const uint4*>(&Vs[0][0] + r * VROW + sch * 16);
            *reinterpret_cast<uint4*>(Ob + (q0 + r) * D + ch * 8) = v;
        }
    }
}


// Hamming distance of two D-bit vectors; for D = 128 a carry-save step turns four
// 32-bit popcounts into three (the POPC pipe is the narrow one).
template <int W> __device__ __forceinline__ int hamming_bits(const uint32_t* q, const uint32_t* k);
template <> __device__ __forceinline__ int hamming_bits<1>(const uint32_t* q, const uint32_t* k) {
    return __popc(q[0] ^ k[0]) + __popc(q[1] ^ k[1]);
}
template <> __device__ __forceinline__ int hamming_bits<2>(const uint32_t* q, const uint32_t* k) {
    const uint32_t x0 = q[0] ^ k[0], x1 = q[1] ^ k[1], x2 = q[2] ^ k[2], x3 = q[3] ^ k[3];
    const uint32_t s = x0 ^ x1 ^ x2;
    const uint32_t c = (x0 & x1) | (x0 & x2) | (x1 & x2);
    return __popc(s) + __popc(x3) + 2 * __popc(c);
}

template <int W>
__global__ void __launch_bounds__(AT_THREADS, 2)
k_binary_attention_fwd_table(const uint64_t* __restrict__ Qp, const uint64_t* __restrict__ Kp,
                             const __nv_bfloat16* __restrict__ V, __nv_bfloat16* __restrict__ O,
                             int64_t S, int causal, float neg2c_log2 /* -2*scale*log2(e) */, float bias_log2,
                             int64_t q_tiles) {
    constexpr int D = 64 * W;
    constexpr int VROW = D * 2;
    constexpr int VCH = D / 8;
    constexpr int NT = D / 8;
    __shared__ __align__(16) uint64_t Ks[2][AT_BN * W];
    __shared__ __align__(128) uint8_t Vs[2][AT_BN * VROW];
    __shared__ float T[D + 1];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int64_t qt = q_tiles - 1 - (int64_t)blockIdx.x;
    const int64_t bh = blockIdx.y;
    const int64_t q0 = qt * AT_BM;
    const uint64_t* Qb = Qp + bh * S * W;
    const uint64_t* Kb = Kp + bh * S * W;
    const __nv_bfloat16* Vb = V + bh * S * D;
    __nv_bfloat16* Ob = O + bh * S * D;

    if (tid <= D) T[tid] = exp2f(neg2c_log2 * (float)tid - bias_log2);

    const int64_t row_lo = q0 + warp * 16 + g, row_hi = row_lo + 8;
    uint32_t q[2][2 * W];
#pragma unroll
    for (int w = 0; w < W; ++w) {
        const uint64_t a = row_lo < S ? __ldg(Qb + row_lo * W + w) : 0ull;
        const uint64_t b = row_hi < S ? __ldg(Qb + row_hi * W + w) : 0ull;
        q[0][2 * w] = (uint32_t)a; q[0][2 * w + 1] = (uint32_t)(a >> 32);
        q[1][2 * w] = (uint32_t)b; q[1][2 * w + 1] = (uint32_t)(b >> 32);
    }

    const int64_t kend = causal ? (q0 + AT_BM < S ? q0 + AT_BM : S) : S;
    const int64_t ntiles = (kend + AT_BN - 1) / AT_BN;
    const uint32_t ks_base = (uint32_t)__cvta_generic_to_shared(&Ks[0][0]);
    const uint32_t vs_base = (uint32_t)__cvta_generic_to_shared(&Vs[0][0]);

    auto load_tile = [&](int buf, int64_t tile) {
        const int64_t k0 = tile * AT_BN;
        if (tid < AT_BN * W) {
            const int key = tid / W, w = tid % W;
            const bool ok = k0 + key < S;
            at_cp_async8(ks_base + (buf * AT_BN * W + tid) * 8, Kb + (ok ? (k0 + key) * W + w : 0), ok ? 8 : 0);
        }
#pragma unroll
        for (int it = 0; it < (AT_BN * VCH) / AT_THREADS; ++it) {
            const int idx = tid + it * AT_THREADS;
            const int row = idx / VCH, ch = idx % VCH;
            const bool ok = k0 + row < S;
            const int sch = (ch & ~7) | ((ch ^ row) & 7);
            at_cp_async16(vs_base + buf * AT_BN * VROW + row * VROW + sch * 16,
                          Vb + (ok ? (k0 + row) * D + ch * 8 : 0), ok ? 16 : 0);
        }
    };

    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float lrow[2] = {0.f, 0.f};

    if (ntiles > 0) load_tile(0, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");

    for (int64_t tile = 0; tile < ntiles; ++tile) {
        const int buf = (int)(tile & 1);
        if (tile + 1 < ntiles) load_tile(buf ^ 1, tile + 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();

        const int64_t k0 = tile * AT_BN;
        const bool active = !(causal && k0 > q0 + warp * 16 + 15);
        if (active) {
            const bool need_mask = (causal && k0 + AT_BN - 1 > q0 + warp * 16) || (k0 + AT_BN > S);
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
                float p[2][4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int key = kb * 16 + 2 * t + (c & 1) + ((c >> 1) << 3);
                    uint32_t kw[2 * W];
                    if (W == 2) {
                        const uint4 kv = *reinterpret_cast<const uint4*>(&Ks[buf][key * 2]);
                        kw[0] = kv.x; kw[1] = kv.y; kw[2 * W - 2] = kv.z; kw[2 * W - 1] = kv.w;
                    } else {
                        const uint2 kv = *reinterpret_cast<const uint2*>(&Ks[buf][key]);
                        kw[0] = kv.x; kw[1] = kv.y;
                    }
                    float p0 = T[hamming_bits<W>(q[0], kw)];
                    float p1 = T[hamming_bits<W>(q[1], kw)];
                    if (need_mask) {
                        const int64_t kidx = k0 + key;
                        if (kidx >= S || (causal && kidx > row_lo)) p0 = 0.f;
                        if (kidx >= S || (causal && kidx > row_hi)) p1 = 0.f;
                    }
                    p[0][c] = p0; p[1][c] = p1;
                }
                const uint32_t a0 = pack_bf16x2(p[0][0], p[0][1]);
                const uint32_t a1 = pack_bf16x2(p[1][0], p[1][1]);
                const uint32_t a2 = pack_bf16x2(p[0][2], p[0][3]);
                const uint32_t a3 = pack_bf16x2(p[1][2], p[1][3]);
                // the denominator sums the SAME bf16-rounded weights that enter the MMA,
                // so the normalised weights of a row add up to exactly one
                lrow[0] += (__uint_as_float(a0 << 16) + __uint_as_float(a0 & 0xFFFF0000u)) +
                           (__uint_as_float(a2 << 16) + __uint_as_float(a2 & 0xFFFF0000u));
                lrow[1] += (__uint_as_float(a1 << 16) + __uint_as_float(a1 & 0xFFFF0000u)) +
                           (__uint_as_float(a3 << 16) + __uint_as_float(a3 & 0xFFFF0000u));
                const int vrow = kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
                for (int j = 0; j < NT; j += 2) {
                    const int ch = j + (lane >> 4);
                    const int sch = (ch & ~7) | ((ch ^ vrow) & 7);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(vs_base + buf * AT_BN * VROW + vrow * VROW + sch * 16, b0, b1, b2, b3);
                    mma_bf16_16816(o[j], a0, a1, a2, a3, b0, b1);
                    mma_bf16_16816(o[j + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
        __syncthreads();
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float l = lrow[h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int r = warp * 16 + g + 8 * h;
        uint8_t* srow = &Vs[0][0] + r * VROW;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int sch = (j & ~7) | ((j ^ r) & 7);
            *reinterpret_cast<uint32_t*>(srow + sch * 16 + t * 4) =
                pack_bf16x2(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
        }
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < (AT_BM * VCH) / AT_THREADS; ++it) {
        const int idx = tid + it * AT_THREADS;
        const int r = idx / VCH, ch = idx % VCH;
        const int sch = (ch & ~7) | ((ch ^ r) & 7);
        if (q0 + r < S) {
            const uint4 v = *reinterpret_cast<const uint4*>(&Vs[0][0] + r * VROW + sch * 16);
            *reinterpret_cast<uint4*>(Ob + (q0 + r) * D + ch * 8) = v;
        }
    }
}


// ---------------------------------------------------------------------------
// Table softmax with the SCORES on the tensor cores as well.
//
// The keys of a tile are expanded once per CTA from packed bits to int8 in shared memory
// (bit 1 -> -2, bit 0 -> +2), the queries once per warp into m16n8k32 A-fragments (bit 1 -> +1,
// bit 0 -> -1), so that mma.sync s8 x s8 accumulates acc = 4*h - 2*D for Hamming distance h.
// T[h] is a float table, so acc + 2*D IS the byte offset of T[h]: a score costs one shared-memory
// load and half a bf16x2 convert, against ~18 XOR/POPC/ALU instructions on the CUDA cores. The
// accumulator layout of the score MMA is the A-fragment layout of the P.V MMA, so P still never
// leaves registers. The row sums come from one more MMA per 16 keys against a column of ones,
// which sums exactly the bf16-rounded weights that enter P.V. The d positions inside every
// 32-bit word are permuted (byte 4j+i <- bit 8i+j) identically for Q and K.
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_s8_16832(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 4 bits (j, 8+j, 16+j, 24+j of h) -> 4 int8: query side +1 / -1, key side -2 / +2
__device__ __forceinline__ uint32_t at_enc_q(uint32_t h, int j) { return 0xFFFFFFFFu ^ (((h >> j) & 0x01010101u) * 0xFEu); }
__device__ __forceinline__ uint32_t at_enc_k(uint32_t h, int j) { return 0x02020202u ^ (((h >> j) & 0x01010101u) * 0xFCu); }

template <int W> constexpr int at_mma_smem() { return 2 * AT_BN * 64 * W + 2 * AT_BN * 128 * W + 4 * (64 * W + 4); }

template <int W>
__global__ void __launch_bounds__(AT_THREADS, 2)
k_binary_attention_fwd_mma(const uint64_t* __restrict__ Qp, const uint64_t* __restrict__ Kp,
                           const __nv_bfloat16* __restrict__ V, __nv_bfloat16* __restrict__ O,
                           int64_t S, int causal, float neg2c_log2 /* -2*scale*log2(e) */, float bias_log2,
                           int64_t q_tiles) {
    constexpr int D = 64 * W;
    constexpr int VROW = D * 2, VCH = D / 8, NT = D / 8;
    constexpr int KROW = D;                     // bytes per expanded key row
    constexpr int KS = D / 32;                  // k-steps of the score MMA = 32-bit words per row
    extern __shared__ __align__(128) uint8_t at_smem[];
    uint8_t* Ke = at_smem;                                   // [2][AT_BN][KROW] int8, 16-byte chunks swizzled
    uint8_t* Vs = at_smem + 2 * AT_BN * KROW;                // [2][AT_BN][VROW] bf16, 16-byte chunks swizzled
    float* T = reinterpret_cast<float*>(Vs + 2 * AT_BN * VROW);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int64_t qt = q_tiles - 1 - (int64_t)blockIdx.x;    // heavy (late) causal tiles first
    const int64_t bh = blockIdx.y;
    const int64_t q0 = qt * AT_BM;
    const uint32_t* Qw = reinterpret_cast<const uint32_t*>(Qp + bh * S * W);
    const uint32_t* Kw = reinterpret_cast<const uint32_t*>(Kp + bh * S * W);
    const __nv_bfloat16* Vb = V + bh * S * D;
    __nv_bfloat16* Ob = O + bh * S * D;

    if (tid <= D) T[tid] = exp2f(neg2c_log2 * (float)tid - bias_log2);
    const char* Tc = reinterpret_cast<const char*>(T) + 2 * D;     // acc = 4*h - 2*D -> T[h]

    const int64_t row_lo = q0 + warp * 16 + g, row_hi = row_lo + 8;
    uint32_t qa[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        const uint32_t lo = row_lo < S ? __ldg(Qw + row_lo * KS + ks) : 0u;
        const uint32_t hi = row_hi < S ? __ldg(Qw + row_hi * KS + ks) : 0u;
        qa[ks][0] = at_enc_q(lo, t);     qa[ks][1] = at_enc_q(hi, t);
        qa[ks][2] = at_enc_q(lo, 4 + t); qa[ks][3] = at_enc_q(hi, 4 + t);
    }

    const int64_t kend = causal ? (q0 + AT_BM < S ? q0 + AT_BM : S) : S;
    const int64_t ntiles = (kend + AT_BN - 1) / AT_BN;
    const uint32_t ke_base = (uint32_t)__cvta_generic_to_shared(Ke);
    const uint32_t vs_base = (uint32_t)__cvta_generic_to_shared(Vs);

    // this thread's packed word of a key tile: key ekey, 32-bit word ew
    const bool expander = tid < AT_BN * KS;
    const int ekey = tid / KS, ew = tid % KS;
    auto key_swz = [](int key) { return W == 2 ? (key & 7) : ((key >> 1) & 3); };
    auto load_k = [&](int64_t tile) -> uint32_t {
        const int64_t k = tile * AT_BN + ekey;
        return (expander && k < S) ? __ldg(Kw + k * KS + ew) : 0u;
    };
    auto expand_k = [&](int buf, uint32_t h) {
        if (!expander) return;
        uint8_t* row = Ke + (buf * AT_BN + ekey) * KROW;
        const int sw = key_swz(ekey);
        *reinterpret_cast<uint4*>(row + (((2 * ew) ^ sw) << 4)) =
            make_uint4(at_enc_k(h, 0), at_enc_k(h, 1), at_enc_k(h, 2), at_enc_k(h, 3));
        *reinterpret_cast<uint4*>(row + (((2 * ew + 1) ^ sw) << 4)) =
            make_uint4(at_enc_k(h, 4), at_enc_k(h, 5), at_enc_k(h, 6), at_enc_k(h, 7));
    };
    auto load_v = [&](int buf, int64_t tile) {
        const int64_t k0 = tile * AT_BN;
#pragma unroll
        for (int it = 0; it < (AT_BN * VCH) / AT_THREADS; ++it) {
            const int idx = tid + it * AT_THREADS;
            const int row = idx / VCH, ch = idx % VCH;
            const bool ok = k0 + row < S;
            const int sch = (ch & ~7) | ((ch ^ row) & 7);
            at_cp_async16(vs_base + buf * AT_BN * VROW + row * VROW + sch * 16,
                          Vb + (ok ? (k0 + row) * D + ch * 8 : 0), ok ? 16 : 0);
        }
    };

    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float ol[4] = {0.f, 0.f, 0.f, 0.f};         // row sums: P against a column of ones
    constexpr uint32_t ONES = 0x3F803F80u;      // bf16 (1.0, 1.0)

    uint32_t knext = 0u;
    if (ntiles > 0) {
        load_v(0, 0);
        expand_k(0, load_k(0));
        if (ntiles > 1) knext = load_k(1);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");

    for (int64_t tile = 0; tile < ntiles; ++tile) {
        const int buf = (int)(tile & 1);
        if (tile + 1 < ntiles) {
            load_v(buf ^ 1, tile + 1);
            expand_k(buf ^ 1, knext);            // read again only after the barrier that ends this iteration
            if (tile + 2 < ntiles) knext = load_k(tile + 2);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();

        const int64_t k0 = tile * AT_BN;
        const bool active = !(causal && k0 > q0 + warp * 16 + 15);
        if (active) {
            const bool need_mask = (causal && k0 + AT_BN - 1 > q0 + warp * 16) || (k0 + AT_BN > S);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                int c[4][4];
#pragma unroll
                for (int nbi = 0; nbi < 4; ++nbi) {
                    c[nbi][0] = c[nbi][1] = c[nbi][2] = c[nbi][3] = 0;
                    const int krow = 8 * (4 * half + nbi) + (lane & 7);
                    const uint32_t rowaddr = ke_base + (uint32_t)((buf * AT_BN + krow) * KROW);
                    const int sw = key_swz(krow);
#pragma unroll
                    for (int cq = 0; cq < KS / 2; ++cq) {
                        uint32_t b0, b1, b2, b3;
                        ldmatrix_x4(rowaddr + (uint32_t)((((4 * cq + (lane >> 3))) ^ sw) << 4), b0, b1, b2, b3);
                        mma_s8_16832(c[nbi], qa[2 * cq], b0, b1);
                        mma_s8_16832(c[nbi], qa[2 * cq + 1], b2, b3);
                    }
                }
#pragma unroll
                for (int kbi = 0; kbi < 2; ++kbi) {
                    const int kb = 2 * half + kbi;
                    float p[2][4];          // [n-block of the pair][accumulator slot]
#pragma unroll
                    for (int x = 0; x < 2; ++x) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            float v = *reinterpret_cast<const float*>(Tc + c[2 * kbi + x][e]);
                            if (need_mask) {
                                const int64_t kidx = k0 + kb * 16 + x * 8 + 2 * t + (e & 1);
                                const int64_t row = (e & 2) ? row_hi : row_lo;
                                if (kidx >= S || (causal && kidx > row)) v = 0.f;
                            }
                            p[x][e] = v;
                        }
                    }
                    const uint32_t a0 = pack_bf16x2(p[0][0], p[0][1]);
                    const uint32_t a1 = pack_bf16x2(p[0][2], p[0][3]);
                    const uint32_t a2 = pack_bf16x2(p[1][0], p[1][1]);
                    const uint32_t a3 = pack_bf16x2(p[1][2], p[1][3]);
                    mma_bf16_16816(ol, a0, a1, a2, a3, ONES, ONES);
                    const int vrow = kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
                    for (int j = 0; j < NT; j += 2) {
                        const int ch = j + (lane >> 4);
                        const int sch = (ch & ~7) | ((ch ^ vrow) & 7);
                        uint32_t b0, b1, b2, b3;
                        ldmatrix_x4_trans(vs_base + buf * AT_BN * VROW + vrow * VROW + sch * 16, b0, b1, b2, b3);
                        mma_bf16_16816(o[j], a0, a1, a2, a3, b0, b1);
                        mma_bf16_16816(o[j + 1], a0, a1, a2, a3, b2, b3);
                    }
                }
            }
        }
        __syncthreads();
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // normalise, stage the 128 x D output tile through the V buffers, coalesced 16-byte stores
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const float l = ol[2 * h];
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int r = warp * 16 + g + 8 * h;
        uint8_t* srow = Vs + r * VROW;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int sch = (j & ~7) | ((j ^ r) & 7);
            *reinterpret_cast<uint32_t*>(srow + sch * 16 + t * 4) =
                pack_bf16x2(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
        }
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < (AT_BM * VCH) / AT_THREADS; ++it) {
        const int idx = tid + it * AT_THREADS;
        const int r = idx / VCH, ch = idx % VCH;
        const int sch = (ch & ~7) | ((ch ^ r) & 7);
        if (q0 + r < S) {
            const uint4 v = *reinterpret_cast<const uint4*>(Vs + r * VROW + sch * 16);
            *reinterpret_cast<uint4*>(Ob + (q0 + r) * D + ch * 8) = v;
        }
    }
}

}  // namespace bb

#include "attention_tcgen05.cuh"

namespace bb { int at_status_bridge() { return tc5_device_status(); } }

using namespace bb;

extern "C" int brute_b200_binary_attention_fwd(const uint64_t* Qp, const uint64_t* Kp_,
                                               const void* V, void* O,
                                               int64_t B, int64_t H, int64_t S, int64_t D,
                                               int causal, float scale, void* stream) {
    BB_REQUIRE(B >= 0 && H >= 0 && S >= 0, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(D == 64 || D == 128, BRUTE_ERR_UNSUPPORTED);
    if (B * H == 0 || S == 0) return BRUTE_OK;
    BB_REQUIRE(Qp && Kp_ && V && O, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(Qp) && aligned8(Kp_) && aligned16(V) && aligned16(O), BRUTE_ERR_MISALIGNED);
    BB_REQUIRE(B * H <= 65535, BRUTE_ERR_UNSUPPORTED);
    BB_REQUIRE(scale == scale, BRUTE_ERR_INVALID_ARG);
    const int64_t q_tiles = (S + AT_BM - 1) / AT_BM;
    const dim3 grid((unsigned)q_tiles, (unsigned)(B * H));
    const float scale_log2 = scale * 1.4426950408889634f;
    cudaStream_t st = as_stream(stream);
    auto* v = static_cast<const __nv_bfloat16*>(V);
    auto* o = static_cast<__nv_bfloat16*>(O);
    // table kernel while T[D] = exp2(-2*|scale|*log2(e)*D) is a normal fp32 number
    const float span_log2 = 2.0f * fabsf(scale_log2) * (float)D;
    if (span_log2 <= 100.0f) {
        const float neg2c = -2.0f * scale_log2;
        const float bias = scale_log2 < 0.f ? neg2c * (float)D : 0.f;      // keeps max(T) == 1
        // BRUTE_ATTENTION_IMPL = tcgen05 (default) | mma (mma.sync scores) | popc (CUDA-core scores)
        const char* env_impl = std::getenv("BRUTE_ATTENTION_IMPL");     // read per call: tests switch it
        const bool want_popc = env_impl && !std::strcmp(env_impl, "popc");
        const bool want_mma = env_impl && !std::strcmp(env_impl, "mma");
        if (!want_popc && !want_mma) {
            const int rc = D == 128 ? ax_run<128>(Qp, Kp_, V, O, B * H, S, causal, neg2c, bias, st)
                                    : ax_run<64>(Qp, Kp_, V, O, B * H, S, causal, neg2c, bias, st);
            if (rc != BRUTE_ERR_DRIVER) return rc;      // no tensor-map encoder: fall through to mma.sync
        }
        if (want_popc) {
            if (D == 128) k_binary_attention_fwd_table<2><<<grid, AT_THREADS, 0, st>>>(Qp, Kp_, v, o, S, causal, neg2c, bias, q_tiles);
            else          k_binary_attention_fwd_table<1><<<grid, AT_THREADS, 0, st>>>(Qp, Kp_, v, o, S, causal, neg2c, bias, q_tiles);
            return launch_status();
        }
        if (D == 128) {
            if (!kernel_smem_ready<k_binary_attention_fwd_mma<2>>(at_mma_smem<2>())) return BRUTE_ERR_LAUNCH;
            k_binary_attention_fwd_mma<2><<<grid, AT_THREADS, at_mma_smem<2>(), st>>>(Qp, Kp_, v, o, S, causal, neg2c, bias, q_tiles);
        } else {
            if (!kernel_smem_ready<k_binary_attention_fwd_mma<1>>(at_mma_smem<1>())) return BRUTE_ERR_LAUNCH;
            k_binary_attention_fwd_mma<1><<<grid, AT_THREADS, at_mma_smem<1>(), st>>>(Qp, Kp_, v, o, S, causal, neg2c, bias, q_tiles);
        }
        return launch_status();
    }
    if (D == 128) k_binary_attention_fwd<2><<<grid, AT_THREADS, 0, st>>>(Qp, Kp_, v, o, S, causal, scale_log2, q_tiles);
    else          k_binary_attention_fwd<1><<<grid, AT_THREADS, 0, st>>>(Qp, Kp_, v, o, S, causal, scale_log2, q_tiles);
    return launch_status();
}
