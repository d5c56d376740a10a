/*
 * CPU oracle for the brute.bit1 hot path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's CPU implementation
 * (TheoCoombes/Brute, cbrute/cpu). Only tests/, __graft_entry__.smoke() and
 * the cpu_baseline / reference legs of bench.py may load it; the product
 * library never links or calls it.
 *
 * Parity pin: checked in tests/test_oracle.py against the reference's own
 * known-answer vectors and bit-by-bit helpers (tests/helpers/reference_ops.py,
 * tests/unit/test_dtype.py:79-83, tests/unit/test_brute_methods.py:92-116);
 * fixtures generated from those helpers are committed under tests/golden/.
 * Binary attention has no reference implementation: its oracle is the
 * composition written below and its parity is UNPINNED.
 *
 * The reference's kernels use google/highway (un-vendored submodule,
 * third_party/highway, pin unknown). The lane-wise integer operations it takes
 * from Highway (Xor, PopulationCount, Add, ReduceSum, Ne, BitsFromMask) have no
 * rounding or ordering freedom, so this scalar/AVX-512 restatement is
 * bit-identical by construction. Threading mirrors at::parallel_for with OpenMP.
 *
 * Build: see oracle/Makefile (gcc -O3 -fopenmp -shared -fPIC).
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#include <math.h>
#include <stdlib.h>

#if defined(__x86_64__)
#include <immintrin.h>
#define ORACLE_X86 1
#else
#define ORACLE_X86 0
#endif

#ifdef _OPENMP
#include <omp.h>
#endif

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------------------
 * pack_bool: bool bytes [rows, ld] -> packed bytes, LSB first; each row is
 * padded to whole 64-bit words with zero bits.
 * Follows cbrute/cpu/ops_cpu.cpp:39-70 (driver, zero-initialised output, one
 * row per task) and PackBoolBytesToBits, cbrute/cpu/kernels/packing.hpp:79-129
 * (any nonzero byte is a 1 bit).
 * ---------------------------------------------------------------------- */
void oracle_pack_bool(const uint8_t* in, uint64_t* out, int64_t rows, int64_t ld) {
    const int64_t wpr = (ld + 63) / 64;
    if (rows <= 0 || ld <= 0) return;
    memset(out, 0, (size_t)(rows * wpr) * sizeof(uint64_t));
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const uint8_t* src = in + r * ld;
        uint8_t* dst = (uint8_t*)(out + r * wpr);
        const int64_t n_full = ld / 8;
        for (int64_t j = 0; j < n_full; ++j) {
            uint8_t byte = 0;
            for (int b = 0; b < 8; ++b) byte |= (uint8_t)((src[j * 8 + b] != 0) << b);
            dst[j] = byte;
        }
        const int64_t left = ld - n_full * 8;
        if (left) {
            uint8_t byte = 0;
            for (int64_t b = 0; b < left; ++b) if (src[n_full * 8 + b]) byte |= (uint8_t)(1u << b);
            dst[n_full] = byte;
        }
    }
}

/* Float threshold then pack. The reference does this in two steps:
 * `_to_bool` (x > 0), brute/tensor.py:163-169, or `randn(...) >= 0`,
 * brute/functional.py:131-133, followed by pack_bool. mode 0: x > 0, 1: x >= 0. */
void oracle_pack_sign_f32(const float* in, uint64_t* out, int64_t rows, int64_t ld, int mode) {
    const int64_t wpr = (ld + 63) / 64;
    if (rows <= 0 || ld <= 0) return;
    memset(out, 0, (size_t)(rows * wpr) * sizeof(uint64_t));
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const float* src = in + r * ld;
        uint64_t* dst = out + r * wpr;
        for (int64_t i = 0; i < ld; ++i) {
            const int bit = mode ? (src[i] >= 0.0f) : (src[i] > 0.0f);
            if (bit) dst[i >> 6] |= 1ull << (i & 63);
        }
    }
}

/* unpack_bool / unpack_bits(+-1 float).
 * Follows cbrute/cpu/ops_cpu.cpp:73-114 and UnpackBitsToBoolBytes /
 * UnpackBitsToPm1, cbrute/cpu/kernels/packing.hpp:134-171 (bit 1 -> 1 / +1.0f,
 * bit 0 -> 0 / -1.0f). */
void oracle_unpack_bool(const uint64_t* in, uint8_t* out, int64_t rows, int64_t ll) {
    const int64_t wpr = (ll + 63) / 64;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const uint8_t* src = (const uint8_t*)(in + r * wpr);
        uint8_t* dst = out + r * ll;
        for (int64_t i = 0; i < ll; ++i) dst[i] = (src[i >> 3] >> (i & 7)) & 1u;
    }
}

void oracle_unpack_pm1_f32(const uint64_t* in, float* out, int64_t rows, int64_t ll) {
    const int64_t wpr = (ll + 63) / 64;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const uint8_t* src = (const uint8_t*)(in + r * wpr);
        float* dst = out + r * ll;
        for (int64_t i = 0; i < ll; ++i) dst[i] = ((src[i >> 3] >> (i & 7)) & 1u) ? 1.0f : -1.0f;
    }
}

/* ------------------------------------------------------------------------
 * popcount family.
 * Per element: cbrute/cpu/ops_cpu.cpp:216-230 + PopcountPerWord,
 * cbrute/cpu/kernels/popcount.hpp:303-328, on the UNSIGNED bit pattern (the
 * reference's scalar tail sign-extends negative inputs, a bug its CUDA kernels
 * k_popcnt_*, cbrute/cuda/kernels/popcount.cuh:22-41, do not have; the oracle
 * follows the CUDA behaviour).
 * Totals: TotalPopcountBytes / TotalPopcountXor, popcount.hpp:202-300, whole
 * words then 1..7 tail bytes.
 * ---------------------------------------------------------------------- */
void oracle_popcount_elems(const void* in, int32_t* out, int64_t n, int elem_bytes) {
    const uint8_t* p = (const uint8_t*)in;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        uint64_t v = 0;
        memcpy(&v, p + i * elem_bytes, (size_t)elem_bytes);
        out[i] = (int32_t)__builtin_popcountll(v);
    }
}

uint64_t oracle_popcount_total(const void* in, int64_t n_bytes) {
    const uint64_t* w = (const uint64_t*)in;
    const int64_t nw = n_bytes / 8;
    uint64_t total = 0;
#pragma omp parallel for schedule(static) reduction(+ : total)
    for (int64_t i = 0; i < nw; ++i) {
        uint64_t v; memcpy(&v, w + i, 8);
        total += (uint64_t)__builtin_popcountll(v);
    }
    const uint8_t* t = (const uint8_t*)in + nw * 8;
    for (int64_t k = 0; k < n_bytes - nw * 8; ++k) total += (uint64_t)__builtin_popcount(t[k]);
    return total;
}

uint64_t oracle_hamming_total(const void* a, const void* b, int64_t n_bytes) {
    const uint64_t* wa = (const uint64_t*)a;
    const uint64_t* wb = (const uint64_t*)b;
    const int64_t nw = n_bytes / 8;
    uint64_t total = 0;
#pragma omp parallel for schedule(static) reduction(+ : total)
    for (int64_t i = 0; i < nw; ++i) {
        uint64_t x, y; memcpy(&x, wa + i, 8); memcpy(&y, wb + i, 8);
        total += (uint64_t)__builtin_popcountll(x ^ y);
    }
    const uint8_t* ta = (const uint8_t*)a + nw * 8;
    const uint8_t* tb = (const uint8_t*)b + nw * 8;
    for (int64_t k = 0; k < n_bytes - nw * 8; ++k) total += (uint64_t)__builtin_popcount((unsigned)(ta[k] ^ tb[k]));
    return total;
}

/* per-word popcount(a ^ b): hamming_distance, cbrute/cpu/ops_cpu.cpp:241-243 */
void oracle_hamming_words(const uint64_t* a, const uint64_t* b, int32_t* out, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = (int32_t)__builtin_popcountll(a[i] ^ b[i]);
}

/* ------------------------------------------------------------------------
 * bitwise ops on packed rows. and/or/xor are ATen int64 ops in the reference
 * (brute/tensor.py:564-598); NOT is bit1_not_packed_composite,
 * cbrute/ext.cpp:27-39: ~A, then the last word of every row ANDed with
 * (1 << (last_dim_bits % 64)) - 1 when last_dim_bits % 64 != 0.
 * op: 0 and, 1 or, 2 xor, 3 xnor (= NOT of xor, masked), 4 andnot, 5 not(a).
 * ---------------------------------------------------------------------- */
void oracle_bitwise(int op, const uint64_t* a, const uint64_t* b, uint64_t* out,
                    int64_t rows, int64_t wpr, int64_t last_dim_bits) {
    const int vb = (int)(last_dim_bits % 64);
    const uint64_t mask = vb == 0 ? ~0ull : ((1ull << vb) - 1ull);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t w = 0; w < wpr; ++w) {
            const int64_t i = r * wpr + w;
            uint64_t x;
            switch (op) {
                case 0: x = a[i] & b[i]; break;
                case 1: x = a[i] | b[i]; break;
                case 2: x = a[i] ^ b[i]; break;
                case 3: x = ~(a[i] ^ b[i]); break;
                case 4: x = a[i] & ~b[i]; break;
                default: x = ~a[i]; break;
            }
            if ((op == 3 || op == 5) && w == wpr - 1) x &= mask;
            out[i] = x;
        }
    }
}

/* packed where: (a & cond) | (b & ~cond), brute/tensor.py:1863-1883 */
void oracle_select(const uint64_t* c, const uint64_t* a, const uint64_t* b, uint64_t* out, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = (a[i] & c[i]) | (b[i] & ~c[i]);
}

/* any / all over the packed axis, brute/tensor.py:1415-1431:
 * any = some word != 0; all = sum of word popcounts == last_dim_bits. */
void oracle_row_any(const uint64_t* a, uint8_t* out, int64_t rows, int64_t wpr) {
    for (int64_t r = 0; r < rows; ++r) {
        uint64_t acc = 0;
        for (int64_t w = 0; w < wpr; ++w) acc |= a[r * wpr + w];
        out[r] = acc != 0;
    }
}

void oracle_row_all(const uint64_t* a, uint8_t* out, int64_t rows, int64_t wpr, int64_t last_dim_bits) {
    for (int64_t r = 0; r < rows; ++r) {
        int64_t pc = 0;
        for (int64_t w = 0; w < wpr; ++w) pc += __builtin_popcountll(a[r * wpr + w]);
        out[r] = pc == last_dim_bits;
    }
}

/* ------------------------------------------------------------------------
 * xnor_popcount_matmul: C[m,n] = K - 2 * sum_k popcount(A[m,k] ^ B[n,k]).
 * Follows the driver cbrute/cpu/ops_cpu.cpp:119-156 (parallel over M in
 * 4-row grains, N tiled by 64 so a B tile stays in cache) and the register
 * blocked microkernels of cbrute/cpu/kernels/matmul.hpp: 4x8 (:137-271),
 * single cell (:29-46) for the tails. The AVX-512 VPOPCNTDQ variant is picked
 * at run time when the host has it, otherwise the scalar one runs; both give
 * identical integers.
 * ---------------------------------------------------------------------- */
static void tile_scalar(const uint64_t* a, const uint64_t* b, int64_t Kp, int32_t K,
                        int mr, int nr, int32_t* C, int64_t ldc) {
    for (int i = 0; i < mr; ++i)
        for (int j = 0; j < nr; ++j) {
            const uint64_t* ar = a + (int64_t)i * Kp;
            const uint64_t* br = b + (int64_t)j * Kp;
            uint64_t s = 0;
            for (int64_t k = 0; k < Kp; ++k) s += (uint64_t)__builtin_popcountll(ar[k] ^ br[k]);
            C[i * ldc + j] = K - 2 * (int32_t)s;
        }
}

#if ORACLE_X86
__attribute__((target("avx512f,avx512vpopcntdq")))
static void tile_4x8_avx512(const uint64_t* a, const uint64_t* b, int64_t Kp, int32_t K,
                            int32_t* C, int64_t ldc) {
    __m512i acc[4][8];
    for (int i = 0; i < 4; ++i) for (int j = 0; j < 8; ++j) acc[i][j] = _mm512_setzero_si512();
    int64_t k = 0;
    for (; k + 8 <= Kp; k += 8) {
        __m512i va[4], vb[8];
        for (int i = 0; i < 4; ++i) va[i] = _mm512_loadu_si512((const void*)(a + i * Kp + k));
        for (int j = 0; j < 8; ++j) vb[j] = _mm512_loadu_si512((const void*)(b + j * Kp + k));
        for (int i = 0; i < 4; ++i)
            for (int j = 0; j < 8; ++j)
                acc[i][j] = _mm512_add_epi64(acc[i][j], _mm512_popcnt_epi64(_mm512_xor_si512(va[i], vb[j])));
    }
    for (int i = 0; i < 4; ++i)
        for (int j = 0; j < 8; ++j) {
            uint64_t s = (uint64_t)_mm512_reduce_add_epi64(acc[i][j]);
            for (int64_t kk = k; kk < Kp; ++kk) s += (uint64_t)__builtin_popcountll(a[i * Kp + kk] ^ b[j * Kp + kk]);
            C[i * ldc + j] = K - 2 * (int32_t)s;
        }
}
static int have_vpopcnt(void) {
    static int cached = -1;
    if (cached < 0) cached = __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512vpopcntdq");
    return cached;
}
#else
static int have_vpopcnt(void) { return 0; }
#endif

int oracle_has_vpopcntdq(void) { return have_vpopcnt(); }

static void tile_4x8_scalar(const uint64_t* a, const uint64_t* b, int64_t Kp, int32_t K,
                            int32_t* C, int64_t ldc) {
    uint32_t acc[4][8];
    memset(acc, 0, sizeof(acc));
    for (int64_t k = 0; k < Kp; ++k) {
        uint64_t va[4], vb[8];
        for (int i = 0; i < 4; ++i) va[i] = a[i * Kp + k];
        for (int j = 0; j < 8; ++j) vb[j] = b[j * Kp + k];
        for (int i = 0; i < 4; ++i)
            for (int j = 0; j < 8; ++j) acc[i][j] += (uint32_t)__builtin_popcountll(va[i] ^ vb[j]);
    }
    for (int i = 0; i < 4; ++i)
        for (int j = 0; j < 8; ++j) C[i * ldc + j] = K - 2 * (int32_t)acc[i][j];
}

void oracle_xnor_gemm(const uint64_t* A, const uint64_t* B, int32_t* C,
                      int64_t M, int64_t N, int64_t Kp, int64_t K, int64_t ldc) {
    const int64_t N_TILE = 64;
    const int64_t mblocks = (M + 3) / 4;
    const int vp = have_vpopcnt();
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t mb = 0; mb < mblocks; ++mb) {
        const int64_t m = mb * 4;
        const int mr = (int)(M - m < 4 ? M - m : 4);
        for (int64_t ns = 0; ns < N; ns += N_TILE) {
            const int64_t ne = ns + N_TILE < N ? ns + N_TILE : N;
            int64_t n = ns;
            if (mr == 4) {
                for (; n + 8 <= ne; n += 8) {
#if ORACLE_X86
                    if (vp) { tile_4x8_avx512(A + m * Kp, B + n * Kp, Kp, (int32_t)K, C + m * ldc + n, ldc); continue; }
#endif
                    tile_4x8_scalar(A + m * Kp, B + n * Kp, Kp, (int32_t)K, C + m * ldc + n, ldc);
                }
            }
            if (n < ne) tile_scalar(A + m * Kp, B + n * Kp, Kp, (int32_t)K, mr, (int)(ne - n), C + m * ldc + n, ldc);
        }
    }
    (void)vp;
}

/* Binarised-MLP layer (BASELINE config 4) as the reference would compose it:
 * xnor_popcount_matmul -> c.float() * scale[n] -> threshold -> pack_bool. */
void oracle_xnor_gemm_scale_sign_pack(const uint64_t* A, const uint64_t* B, const float* scale,
                                      uint64_t* out, int64_t M, int64_t N, int64_t Kp, int64_t K, int mode) {
    const int64_t wpr = (N + 63) / 64;
    int32_t* C = (int32_t*)malloc((size_t)(M * N) * sizeof(int32_t) + 16);
    oracle_xnor_gemm(A, B, C, M, N, Kp, K, N);
    memset(out, 0, (size_t)(M * wpr) * sizeof(uint64_t));
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            const float y = scale[n] * (float)C[m * N + n];
            if (mode ? (y >= 0.0f) : (y > 0.0f)) out[m * wpr + (n >> 6)] |= 1ull << (n & 63);
        }
    free(C);
}

/* ------------------------------------------------------------------------
 * signed_bundle: out[b,m,d] = sign(sum_n W[b,m,n] * pm1(V[b,n,d])), sign(0) = +1 (bit set), pad
 * bits 0. Follows cbrute/cpu/ops_cpu.cpp:164-213 (int32 accumulator per (b,m), V read from its
 * packed words, zero weights skipped).
 * ---------------------------------------------------------------------- */
void oracle_signed_bundle(const int8_t* W, const uint64_t* V, uint64_t* out,
                          int64_t B, int64_t M, int64_t N, int64_t Dp, int64_t D) {
#pragma omp parallel for schedule(static)
    for (int64_t bm = 0; bm < B * M; ++bm) {
        const int64_t b = bm / M;
        int32_t* acc = (int32_t*)calloc((size_t)(Dp * 64 + 1), sizeof(int32_t));
        const int8_t* wrow = W + bm * N;
        for (int64_t n = 0; n < N; ++n) {
            const int32_t w = wrow[n];
            if (w == 0) continue;
            const uint64_t* vrow = V + (b * N + n) * Dp;
            for (int64_t dp = 0; dp < Dp; ++dp)
                for (int bit = 0; bit < 64; ++bit)
                    acc[dp * 64 + bit] += ((vrow[dp] >> bit) & 1ull) ? w : -w;
        }
        for (int64_t dp = 0; dp < Dp; ++dp) {
            uint64_t word = 0;
            for (int bit = 0; bit < 64; ++bit)
                if (dp * 64 + bit < D && acc[dp * 64 + bit] >= 0) word |= 1ull << bit;
            out[bm * Dp + dp] = word;
        }
        free(acc);
    }
}

/* ------------------------------------------------------------------------
 * Binary attention: NO reference implementation exists (one docstring mention,
 * brute/fast.py:122-124); parity UNPINNED. Composition of reference semantics:
 * per (b,h): S = xnor_popcount_matmul(Q, K, D) (cbrute/cpu/ops_cpu.cpp:119-156)
 * -> * scale -> causal mask -> softmax in fp32 (max-subtracted) -> @ V (fp32
 * accumulate) -> float output (the caller rounds to bf16).
 * V and O are fp32 here: the caller converts bf16 <-> fp32 exactly.
 * ---------------------------------------------------------------------- */
void oracle_binary_attention(const uint64_t* Qp, const uint64_t* Kp_, const float* V, float* O,
                             int64_t BH, int64_t S, int64_t D, int causal, float scale) {
    const int64_t W = D / 64;
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (int64_t bh = 0; bh < BH; ++bh)
        for (int64_t i = 0; i < S; ++i) {
            float* p = (float*)malloc((size_t)S * sizeof(float));
            const uint64_t* q = Qp + (bh * S + i) * W;
            const int64_t jend = causal ? i + 1 : S;
            float mx = -INFINITY;
            for (int64_t j = 0; j < jend; ++j) {
                const uint64_t* k = Kp_ + (bh * S + j) * W;
                int h = 0;
                for (int64_t w = 0; w < W; ++w) h += __builtin_popcountll(q[w] ^ k[w]);
                p[j] = (float)((int)D - 2 * h) * scale;
                if (p[j] > mx) mx = p[j];
            }
            float sum = 0.f;
            for (int64_t j = 0; j < jend; ++j) { p[j] = expf(p[j] - mx); sum += p[j]; }
            float* o = O + (bh * S + i) * D;
            for (int64_t d = 0; d < D; ++d) o[d] = 0.f;
            for (int64_t j = 0; j < jend; ++j) {
                const float pj = p[j] / sum;
                const float* v = V + (bh * S + j) * D;
                for (int64_t d = 0; d < D; ++d) o[d] += pj * v[d];
            }
            free(p);
        }
}


/* Bit-matrix transpose of packed rows. The reference has no packed transpose: a transpose that
 * moves the packed axis unpacks, transposes the bools and packs again (brute/tensor.py:699-775,
 * 1112-1121); this is that composition bit by bit. in [batch, R, ceil(C/64)] -> out [batch, C, ceil(R/64)]. */
void oracle_transpose_bits(const uint64_t* in, uint64_t* out, int64_t batch, int64_t R, int64_t C) {
    const int64_t wi = (C + 63) / 64, wo = (R + 63) / 64;
    memset(out, 0, (size_t)(batch * C * wo) * 8);
    for (int64_t b = 0; b < batch; ++b)
        for (int64_t r = 0; r < R; ++r)
            for (int64_t c = 0; c < C; ++c)
                if ((in[(b * R + r) * wi + (c >> 6)] >> (c & 63)) & 1ull)
                    out[(b * C + c) * wo + (r >> 6)] |= 1ull << (r & 63);
}

/* any / all over a non-packed axis: OR / AND of the packed words (brute/tensor.py:1440-1457 does
 * it by halving). op: 1 = OR, 0 = AND (the BRUTE_OP_* codes). in [outer, R, inner] -> out [outer, inner]. */
void oracle_reduce_rows(int op, const uint64_t* in, uint64_t* out, int64_t outer, int64_t R, int64_t inner) {
    for (int64_t o = 0; o < outer; ++o)
        for (int64_t i = 0; i < inner; ++i) {
            uint64_t acc = op == 1 ? 0ull : ~0ull;
            for (int64_t r = 0; r < R; ++r) {
                const uint64_t v = in[(o * R + r) * inner + i];
                acc = op == 1 ? (acc | v) : (acc & v);
            }
            out[o * inner + i] = acc;
        }
}


/* Moves along the packed axis, bit by bit. The reference unpacks, applies torch.flip / torch.roll /
 * index_select on the bools and packs again (brute/tensor.py:699-775, 795-801); these restate that
 * composition. mode 0: flip, 1: roll by `shift` (torch.roll), 2: gather through idx[n_out]. */
void oracle_move_bits(int mode, const uint64_t* in, const int64_t* idx, uint64_t* out,
                      int64_t rows, int64_t n_in, int64_t n_out, int64_t shift) {
    const int64_t wi = (n_in + 63) / 64, wo = (n_out + 63) / 64;
    memset(out, 0, (size_t)(rows * wo) * 8);
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t j = 0; j < n_out; ++j) {
            int64_t s;
            if (mode == 0) s = n_in - 1 - j;
            else if (mode == 1) { s = (j - shift) % n_in; if (s < 0) s += n_in; }
            else s = idx[j];
            if (s < 0 || s >= n_in) continue;
            if ((in[r * wi + (s >> 6)] >> (s & 63)) & 1ull) out[r * wo + (j >> 6)] |= 1ull << (j & 63);
        }
}


/* Scatter along the packed axis, in place. The reference has no packed form: a write through a tensor
 * index on the last axis (x[..., idx] = v, index_copy_, index_fill_) falls to the bool path, i.e.
 * unpack -> torch index op on the bools -> pack (brute/tensor.py:846-853, 1979-1982); this is that
 * composition bit by bit, in index order (the last writer of a repeated position wins).
 * src == NULL: every indexed position takes `value`. */
void oracle_scatter_bits(uint64_t* packed, const int64_t* idx, const uint64_t* src, int value,
                         int64_t rows, int64_t n, int64_t n_idx) {
    const int64_t wp = (n + 63) / 64, ws = (n_idx + 63) / 64;
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t j = 0; j < n_idx; ++j) {
            const int64_t s = idx[j];
            if (s < 0 || s >= n) continue;
            const int on = src ? (int)((src[r * ws + (j >> 6)] >> (j & 63)) & 1ull) : (value != 0);
            if (on) packed[r * wp + (s >> 6)] |= 1ull << (s & 63);
            else    packed[r * wp + (s >> 6)] &= ~(1ull << (s & 63));
        }
}
