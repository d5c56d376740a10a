// Word-wise ops on packed buffers: and / or / xor / xnor / andnot, pad-safe NOT,
// select (packed `where`) and the row reductions any / all. One pass over HBM
// each; ops that complement bits re-zero the pad bits of every row's last word
// inside the same pass.
#include "common.cuh"

namespace bb {

template <int OP> __device__ __forceinline__ uint64_t apply(uint64_t a, uint64_t b) {
    switch (OP) {
        case BRUTE_OP_AND:    return a & b;
        case BRUTE_OP_OR:     return a | b;
        case BRUTE_OP_XOR:    return a ^ b;
        case BRUTE_OP_XNOR:   return ~(a ^ b);
        case BRUTE_OP_ANDNOT: return a & ~b;
        default:              return ~a;        // OP == -1: unary NOT
    }
}

// Vector path: two words per thread and trip. MASK = the op can set pad bits
// and rows have a partial last word; then the word's column decides the mask.
template <int OP, bool MASK, bool UNARY>
__global__ void __launch_bounds__(256)
k_bitwise_vec(const ulonglong2* __restrict__ a, const ulonglong2* __restrict__ b,
              ulonglong2* __restrict__ out, int64_t nvec, uint32_t wpr, uint64_t tail_mask) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const uint4 ra = ldg_stream(a + i);
        uint64_t x = (uint64_t)ra.x | ((uint64_t)ra.y << 32);
        uint64_t y = (uint64_t)ra.z | ((uint64_t)ra.w << 32);
        if (!UNARY) {
            const uint4 rb = ldg_stream(b + i);
            x = apply<OP>(x, (uint64_t)rb.x | ((uint64_t)rb.y << 32));
            y = apply<OP>(y, (uint64_t)rb.z | ((uint64_t)rb.w << 32));
        } else {
            x = ~x; y = ~y;
        }
        if (MASK) {
            const uint64_t w0 = (uint64_t)i * 2;
            // the column of a word within its row; 32-bit modulo when it fits
            const uint32_t c0 = (w0 >> 32) ? (uint32_t)(w0 % wpr) : ((uint32_t)w0 % wpr);
            if (c0 == wpr - 1) x &= tail_mask;
            const uint32_t c1 = (c0 + 1 == wpr) ? 0u : c0 + 1;
            if (c1 == wpr - 1) y &= tail_mask;
        }
        stg_stream(out + i, make_uint4((uint32_t)x, (uint32_t)(x >> 32), (uint32_t)y, (uint32_t)(y >> 32)));
    }
}

// Word path for unaligned buffers and the odd last word.
template <int OP, bool UNARY>
__global__ void __launch_bounds__(256)
k_bitwise_word(const uint64_t* __restrict__ a, const uint64_t* __restrict__ b,
               uint64_t* __restrict__ out, int64_t first, int64_t n, uint64_t wpr, uint64_t tail_mask,
               bool mask) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = first + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        uint64_t x = UNARY ? ~a[i] : apply<OP>(a[i], b[i]);
        if (mask && ((uint64_t)i % wpr) == wpr - 1) x &= tail_mask;
        out[i] = x;
    }
}

__global__ void __launch_bounds__(256)
k_select(const ulonglong2* __restrict__ c, const ulonglong2* __restrict__ a,
         const ulonglong2* __restrict__ b, ulonglong2* __restrict__ out, int64_t nvec) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const uint4 vc = ldg_stream(c + i), va = ldg_stream(a + i), vb = ldg_stream(b + i);
        uint4 r;
        r.x = (va.x & vc.x) | (vb.x & ~vc.x); r.y = (va.y & vc.y) | (vb.y & ~vc.y);
        r.z = (va.z & vc.z) | (vb.z & ~vc.z); r.w = (va.w & vc.w) | (vb.w & ~vc.w);
        stg_stream(out + i, r);
    }
}

__global__ void __launch_bounds__(256)
k_select_word(const uint64_t* __restrict__ c, const uint64_t* __restrict__ a,
              const uint64_t* __restrict__ b, uint64_t* __restrict__ out, int64_t first, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = first + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = (a[i] & c[i]) | (b[i] & ~c[i]);
}

// Row reductions over the packed axis. One warp per row (rows are short in the
// front end's use: `any(dim=-1)` / `all(dim=-1)`); lanes stride over the words.
// ALL = false: out[r] = any bit set. ALL = true: out[r] = every valid bit set.
template <bool ALL>
__global__ void __launch_bounds__(256)
k_row_reduce(const uint64_t* __restrict__ a, uint8_t* __restrict__ out, int64_t rows, int64_t wpr,
             uint64_t tail_mask) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = warp; r < rows; r += nwarps) {
        const uint64_t* rowp = a + r * wpr;
        uint64_t acc = ALL ? ~0ull : 0ull;
        for (int64_t w = lane; w < wpr; w += 32) {
            uint64_t x = __ldcs(rowp + w);
            if (ALL) { if (w == wpr - 1) x |= ~tail_mask; acc &= x; }
            else acc |= x;
        }
        const bool mine = ALL ? (acc == ~0ull) : (acc != 0ull);
        const uint32_t votes = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) out[r] = ALL ? (votes == 0xffffffffu) : (votes != 0u);
    }
}

static inline uint64_t tail_mask_of(int64_t last_dim_bits) {
    const int vb = (int)(last_dim_bits & 63);
    return vb == 0 ? ~0ull : ((1ull << vb) - 1ull);
}

template <int OP, bool UNARY>
static int launch_bitwise(const uint64_t* a, const uint64_t* b, uint64_t* out, int64_t rows,
                          int64_t wpr, int64_t last_dim_bits, bool complements, cudaStream_t st) {
    const int64_t n = rows * wpr;
    const bool mask = complements && (last_dim_bits & 63) != 0;
    const uint64_t tm = tail_mask_of(last_dim_bits);
    const bool vec_ok = aligned16(a) && aligned16(out) && (UNARY || aligned16(b)) &&
                        (!mask || wpr <= 0xFFFFFFFFll);
    int64_t nvec = vec_ok ? n / 2 : 0;
    if (nvec > 0) {
        const int grid = stream_grid(nvec, 256, 8);
        auto* va = reinterpret_cast<const ulonglong2*>(a);
        auto* vb = reinterpret_cast<const ulonglong2*>(b);
        auto* vo = reinterpret_cast<ulonglong2*>(out);
        if (mask) k_bitwise_vec<OP, true, UNARY><<<grid, 256, 0, st>>>(va, vb, vo, nvec, (uint32_t)wpr, tm);
        else      k_bitwise_vec<OP, false, UNARY><<<grid, 256, 0, st>>>(va, vb, vo, nvec, 1u, tm);
        if (int rc = launch_status()) return rc;
    }
    if (nvec * 2 < n) {
        const int64_t rest = n - nvec * 2;
        k_bitwise_word<OP, UNARY><<<stream_grid(rest, 256, 8), 256, 0, st>>>(
            a, b, out, nvec * 2, n, (uint64_t)wpr, tm, mask);
    }
    return launch_status();
}

}  // namespace bb

using namespace bb;

extern "C" int brute_b200_bitwise(int op, const uint64_t* a, const uint64_t* b, uint64_t* out,
                                  int64_t rows, int64_t wpr, int64_t last_dim_bits, void* stream) {
    BB_REQUIRE(rows >= 0 && wpr >= 0 && last_dim_bits >= 0, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(op >= BRUTE_OP_AND && op <= BRUTE_OP_ANDNOT, BRUTE_ERR_INVALID_ARG);
    if (rows == 0 || wpr == 0) return BRUTE_OK;
    BB_REQUIRE(a && b && out, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(a) && aligned8(b) && aligned8(out), BRUTE_ERR_MISALIGNED);
    cudaStream_t st = as_stream(stream);
    switch (op) {
        case BRUTE_OP_AND:    return launch_bitwise<BRUTE_OP_AND, false>(a, b, out, rows, wpr, last_dim_bits, false, st);
        case BRUTE_OP_OR:     return launch_bitwise<BRUTE_OP_OR, false>(a, b, out, rows, wpr, last_dim_bits, false, st);
        case BRUTE_OP_XOR:    return launch_bitwise<BRUTE_OP_XOR, false>(a, b, out, rows, wpr, last_dim_bits, false, st);
        case BRUTE_OP_XNOR:   return launch_bitwise<BRUTE_OP_XNOR, false>(a, b, out, rows, wpr, last_dim_bits, true, st);
        default:              return launch_bitwise<BRUTE_OP_ANDNOT, false>(a, b, out, rows, wpr, last_dim_bits, false, st);
    }
}

extern "C" int brute_b200_not_masked(const uint64_t* a, uint64_t* out, int64_t rows, int64_t wpr,
                                     int64_t last_dim_bits, void* stream) {
    BB_REQUIRE(rows >= 0 && wpr >= 0 && last_dim_bits >= 0, BRUTE_ERR_INVALID_ARG);
    if (rows == 0 || wpr == 0) return BRUTE_OK;
    BB_REQUIRE(a && out, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(a) && aligned8(out), BRUTE_ERR_MISALIGNED);
    return launch_bitwise<-1, true>(a, nullptr, out, rows, wpr, last_dim_bits, true, as_stream(stream));
}

extern "C" int brute_b200_select(const uint64_t* cond, const uint64_t* a, const uint64_t* b,
                                 uint64_t* out, int64_t n_words, void* stream) {
    BB_REQUIRE(n_words >= 0, BRUTE_ERR_INVALID_ARG);
    if (n_words == 0) return BRUTE_OK;
    BB_REQUIRE(cond && a && b && out, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(cond) && aligned8(a) && aligned8(b) && aligned8(out), BRUTE_ERR_MISALIGNED);
    cudaStream_t st = as_stream(stream);
    const bool vec_ok = aligned16(cond) && aligned16(a) && aligned16(b) && aligned16(out);
    const int64_t nvec = vec_ok ? n_words / 2 : 0;
    if (nvec > 0) {
        k_select<<<stream_grid(nvec, 256, 8), 256, 0, st>>>(
            reinterpret_cast<const ulonglong2*>(cond), reinterpret_cast<const ulonglong2*>(a),
            reinterpret_cast<const ulonglong2*>(b), reinterpret_cast<ulonglong2*>(out), nvec);
        if (int rc = launch_status()) return rc;
    }
    if (nvec * 2 < n_words)
        k_select_word<<<stream_grid(n_words - nvec * 2, 256, 8), 256, 0, st>>>(cond, a, b, out, nvec * 2, n_words);
    return launch_status();
}

extern "C" int brute_b200_row_any(const uint64_t* a, uint8_t* out, int64_t rows, int64_t wpr, void* stream) {
    BB_REQUIRE(rows >= 0 && wpr >= 0, BRUTE_ERR_INVALID_ARG);
    if (rows == 0) return BRUTE_OK;
    BB_REQUIRE(out != nullptr && (a != nullptr || wpr == 0), BRUTE_ERR_INVALID_ARG);
    k_row_reduce<false><<<stream_grid(rows, 8, 8), 256, 0, as_stream(stream)>>>(a, out, rows, wpr, ~0ull);
    return launch_status();
}

extern "C" int brute_b200_row_all(const uint64_t* a, uint8_t* out, int64_t rows, int64_t wpr,
                                  int64_t last_dim_bits, void* stream) {
    BB_REQUIRE(rows >= 0 && wpr >= 0 && last_dim_bits >= 0, BRUTE_ERR_INVALID_ARG);
    if (rows == 0) return BRUTE_OK;
    BB_REQUIRE(out != nullptr && (a != nullptr || wpr == 0), BRUTE_ERR_INVALID_ARG);
    k_row_reduce<true><<<stream_grid(rows, 8, 8), 256, 0, as_stream(stream)>>>(
        a, out, rows, wpr, tail_mask_of(last_dim_bits));
    return launch_status();
}
