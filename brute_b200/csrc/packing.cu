// pack / unpack between 1-byte (or float) elements and 64-bit packed words.
//
// All four kernels are HBM-bound streaming kernels. Work is cut into warp
// tasks "(row, chunk of the row)" so that a warp always reads or writes one
// contiguous span with 128-bit accesses; rows whose byte address is not a
// multiple of 16 (e.g. 4097 bools per row) keep 128-bit ALIGNED accesses and
// shift the bits instead. Shapes whose last dimension is a multiple of 64 are
// flattened to a single row by the launchers, since their packed rows are
// contiguous too.
#include "common.cuh"

namespace bb {

// ===========================================================================
// pack_bool
// ===========================================================================

// Load the 16 bytes at the 16-byte-aligned address p, reading only bytes
// inside [lo, hi); bytes outside read as 0.
__device__ __forceinline__ uint4 load16_guarded(uintptr_t p, uintptr_t lo, uintptr_t hi) {
    if (p >= lo && p + 16 <= hi) return ldg_stream(reinterpret_cast<const void*>(p));
    uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        uintptr_t q = p + i;
        if (q >= lo && q < hi)
            w[i >> 2] |= (uint32_t)(*reinterpret_cast<const uint8_t*>(q)) << (8 * (i & 3));
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// task -> (row, chunk of the row). FLAT: a single row, no division at all.
// Otherwise a 32-bit division when the task count allows it (the usual case).
struct TaskMap {
    int64_t cpr;        // chunks (warp tasks) per row
    uint32_t cpr32;
    int small;          // tasks < 2^32
};

template <bool FLAT>
__device__ __forceinline__ void split_task(int64_t task, const TaskMap& tm, int64_t& r, int64_t& c) {
    if (FLAT) { r = 0; c = task; }
    else if (tm.small) {
        const uint32_t t = (uint32_t)task, q = t / tm.cpr32;
        r = q; c = t - q * tm.cpr32;
    } else { r = task / tm.cpr; c = task - r * tm.cpr; }
}

// 16 bool bytes -> 16 bits. Bytes that are already 0/1 (what torch writes) skip
// the normalisation; any other nonzero byte still counts as 1.
__device__ __forceinline__ uint32_t bools16_to_bits(uint4 v) {
    if ((v.x | v.y | v.z | v.w) & 0xFEFEFEFEu) {
        v.x = ((((v.x & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | v.x) >> 7) & 0x01010101u;
        v.y = ((((v.y & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | v.y) >> 7) & 0x01010101u;
        v.z = ((((v.z & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | v.z) >> 7) & 0x01010101u;
        v.w = ((((v.w & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | v.w) >> 7) & 0x01010101u;
    }
    // bits 0,8,16,24 -> 28..31 with one multiply (no two partial products share a bit)
    constexpr uint32_t G = 0x10204080u;
    return ((v.x * G) >> 28) | (((v.y * G) >> 24) & 0xF0u) | (((v.z * G) >> 20) & 0xF00u) |
           (((v.w * G) >> 16) & 0xF000u);
}

struct PackLoad {
    uint4 lo, hi;      // aligned group of this lane; lane 31 also holds the next one
    int64_t r, g;      // row, 16-byte group index within the row
    uint32_t m;        // misalignment of the row start (bytes, 0..15)
};

// ALIGNED: every row starts on a 16-byte boundary, so a lane's group is one
// aligned vector and no bits move between lanes.
template <bool FLAT, bool ALIGNED>
__device__ __forceinline__ PackLoad pack_bool_load(const uint8_t* in, int64_t ld, const TaskMap& tm,
                                                   int64_t task, uintptr_t buf_lo, uintptr_t buf_hi,
                                                   int lane) {
    PackLoad t;
    int64_t c;
    split_task<FLAT>(task, tm, t.r, c);
    t.g = c * 32 + lane;
    const uintptr_t rowp = reinterpret_cast<uintptr_t>(in) + (uintptr_t)(t.r * ld);
    const uintptr_t row_end = rowp + (uintptr_t)ld;
    t.lo = make_uint4(0u, 0u, 0u, 0u);
    t.hi = make_uint4(0u, 0u, 0u, 0u);
    if (ALIGNED) {
        t.m = 0;
        const uintptr_t a = rowp + (uintptr_t)(t.g * 16);
        if (a + 16 <= row_end) t.lo = ldg_stream(reinterpret_cast<const void*>(a));
        else if (a < row_end) t.lo = load16_guarded(a, buf_lo, buf_hi);
    } else {
        t.m = (uint32_t)(rowp & 15u);
        const uintptr_t ab = rowp + (uintptr_t)(t.g * 16) - t.m;
        if (ab < row_end) t.lo = load16_guarded(ab, buf_lo, buf_hi);
        if (t.m != 0 && lane == 31 && ab + 16 < row_end) t.hi = load16_guarded(ab + 16, buf_lo, buf_hi);
    }
    return t;
}

template <bool ALIGNED>
__device__ __forceinline__ void pack_bool_finish(const PackLoad& t, uint64_t* out, int64_t ld,
                                                 int64_t wpr, int lane) {
    uint32_t bits = bools16_to_bits(t.lo);
    if (!ALIGNED) {
        uint32_t hib = __shfl_down_sync(0xffffffffu, bits, 1);
        if (lane == 31) hib = bools16_to_bits(t.hi);
        bits = ((bits | (hib << 16)) >> t.m) & 0xFFFFu;
    }
    const int64_t valid = ld - t.g * 16;
    if (valid < 16) bits = valid <= 0 ? 0u : (bits & ((1u << (int)valid) - 1u));
    // 4 neighbouring lanes hold the four 16-bit quarters of one word
    uint32_t half = bits << (16 * (lane & 1));
    half |= __shfl_xor_sync(0xffffffffu, half, 1);
    const uint32_t other = __shfl_xor_sync(0xffffffffu, half, 2);
    if ((lane & 3) == 0) {
        const int64_t w = t.g >> 2;
        if (w < wpr) out[t.r * wpr + w] = (uint64_t)half | ((uint64_t)other << 32);
    }
}

template <bool FLAT, bool ALIGNED>
__global__ void __launch_bounds__(256, 4)
k_pack_bool(const uint8_t* __restrict__ in, uint64_t* __restrict__ out,
            int64_t rows, int64_t ld, int64_t wpr, TaskMap tm, int64_t tasks) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const uintptr_t buf_lo = reinterpret_cast<uintptr_t>(in);
    const uintptr_t buf_hi = buf_lo + (uintptr_t)(rows * ld);
    int64_t task = warp;
    // four tasks per trip: all loads are in flight before any is consumed
    for (; task + 3 * nwarps < tasks; task += 4 * nwarps) {
        PackLoad t[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
            t[k] = pack_bool_load<FLAT, ALIGNED>(in, ld, tm, task + k * nwarps, buf_lo, buf_hi, lane);
#pragma unroll
        for (int k = 0; k < 4; ++k) pack_bool_finish<ALIGNED>(t[k], out, ld, wpr, lane);
    }
    for (; task < tasks; task += nwarps) {
        PackLoad a = pack_bool_load<FLAT, ALIGNED>(in, ld, tm, task, buf_lo, buf_hi, lane);
        pack_bool_finish<ALIGNED>(a, out, ld, wpr, lane);
    }
}

// Ragged rows whose start is not 16-byte aligned (e.g. 4097 bools per row): one OUTPUT WORD per lane.
// The word's 64 bools start at an arbitrary byte; the lane loads the up to five aligned 16-byte
// vectors that cover them (default caching: its neighbours' vectors share sectors with it), turns
// each into 16 bits and shifts the 80-bit window down by the misalignment. No bits move between
// lanes, there is no per-row task grid (a row of 4097 bools is 65 words, not 9 warp tasks of which
// the last holds one byte), and a lane amortises its index arithmetic over 64 bytes instead of 16:
// a third of the instructions of the warp-task form on bool [4096, 4097].
template <typename IDX>
__global__ void __launch_bounds__(256, 4)
k_pack_bool_words(const uint8_t* __restrict__ in, uint64_t* __restrict__ out,
                  int64_t rows, IDX ld, IDX wpr, int64_t nwords) {
    const uintptr_t buf_lo = reinterpret_cast<uintptr_t>(in);
    const uintptr_t buf_hi = buf_lo + (uintptr_t)rows * (uintptr_t)ld;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < nwords; t += stride) {
        const IDX r = (IDX)t / wpr, w = (IDX)t - r * wpr;
        const uint64_t col0 = (uint64_t)w * 64u;
        const uintptr_t src = buf_lo + (uintptr_t)r * (uintptr_t)ld + (uintptr_t)col0;
        const uint32_t m = (uint32_t)(src & 15u);
        const uintptr_t base = src - m;
        uint64_t valid = (uint64_t)ld - col0;
        if (valid > 64u) valid = 64u;
        const uint32_t nv = (m + (uint32_t)valid + 15u) >> 4;      // 1..5 vectors hold the word's bools
        uint4 v[5];
#pragma unroll
        for (int k = 0; k < 5; ++k) {
            v[k] = make_uint4(0u, 0u, 0u, 0u);
            if ((uint32_t)k < nv) {
                const uintptr_t a = base + 16u * k;
                if (a >= buf_lo && a + 16 <= buf_hi) v[k] = __ldg(reinterpret_cast<const uint4*>(a));
                else v[k] = load16_guarded(a, buf_lo, buf_hi);
            }
        }
        const uint64_t lo = (uint64_t)bools16_to_bits(v[0]) | ((uint64_t)bools16_to_bits(v[1]) << 16) |
                            ((uint64_t)bools16_to_bits(v[2]) << 32) | ((uint64_t)bools16_to_bits(v[3]) << 48);
        uint64_t word = lo;
        if (m) word = (lo >> m) | ((uint64_t)bools16_to_bits(v[4]) << (64u - m));
        if (valid < 64u) word &= (1ull << valid) - 1ull;
        out[t] = word;
    }
}

// ===========================================================================
// pack_sign: float / bf16 / f16 -> bits in one pass
// ===========================================================================

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <int MODE> __device__ __forceinline__ bool sign_bit(float x) {
    return MODE == BRUTE_SIGN_GE0 ? (x >= 0.0f) : (x > 0.0f);   // NaN -> false
}

// One element per lane and load: fully coalesced scalar loads, one ballot per
// 32 elements. Warp task = 256 elements of one row = 4 output words.
template <typename T, bool FLAT, int MODE>
__global__ void __launch_bounds__(256)
k_pack_sign_ballot(const T* __restrict__ in, uint64_t* __restrict__ out,
                   int64_t ld, int64_t wpr, TaskMap tm, int64_t tasks) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t task = warp; task < tasks; task += nwarps) {
        int64_t r, c;
        split_task<FLAT>(task, tm, r, c);
        const int64_t e0 = c * 256;
        const T* p = in + r * ld + e0 + lane;
        float x[8];
        if (e0 + 256 <= ld) {
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = to_f32<T>(__ldcs(p + 32 * j));
        } else {
            const int left = (int)(ld - e0) - lane;      // elements from this lane's first one to the row end
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = (32 * j < left) ? to_f32<T>(__ldcs(p + 32 * j)) : -1.0f;
        }
        uint32_t b[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) b[j] = __ballot_sync(0xffffffffu, sign_bit<MODE>(x[j]));
        if (lane < 4) {
            const uint32_t lo = lane == 0 ? b[0] : lane == 1 ? b[2] : lane == 2 ? b[4] : b[6];
            const uint32_t hi = lane == 0 ? b[1] : lane == 1 ? b[3] : lane == 2 ? b[5] : b[7];
            const int64_t w = c * 4 + lane;
            if (w < wpr) out[r * wpr + w] = (uint64_t)lo | ((uint64_t)hi << 32);
        }
    }
}

// 16-bit source types, two elements per 32-bit load (row starts 4-byte
// aligned): each lane yields 2 bits, a warp-wide OR-reduction builds the word.
// Warp task = 512 elements = 8 output words.
template <typename T, bool FLAT, int MODE>
__global__ void __launch_bounds__(256)
k_pack_sign_pair16(const T* __restrict__ in, uint64_t* __restrict__ out,
                   int64_t ld, int64_t wpr, TaskMap tm, int64_t tasks) {
    static_assert(sizeof(T) == 2, "pair kernel is for 16-bit element types");
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t task = warp; task < tasks; task += nwarps) {
        int64_t r, c;
        split_task<FLAT>(task, tm, r, c);
        const T* rowp = in + r * ld;
        const int64_t base = c * 512 + 2 * lane;
        uint32_t raw[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int64_t i = base + 64 * j;
            raw[j] = 0xBF80BF80u;   // two negative values (-1.0 in bf16; negative in f16)
            if (i + 1 < ld)  raw[j] = __ldcs(reinterpret_cast<const uint32_t*>(rowp + i));
            else if (i < ld) raw[j] = (raw[j] & 0xFFFF0000u) |
                                      (uint32_t)__ldcs(reinterpret_cast<const uint16_t*>(rowp + i));
        }
        uint64_t mine = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            T e0, e1;
            const uint16_t u0 = (uint16_t)(raw[j] & 0xFFFFu), u1 = (uint16_t)(raw[j] >> 16);
            e0 = *reinterpret_cast<const T*>(&u0);
            e1 = *reinterpret_cast<const T*>(&u1);
            const uint32_t two = (sign_bit<MODE>(to_f32<T>(e0)) ? 1u : 0u) |
                                 (sign_bit<MODE>(to_f32<T>(e1)) ? 2u : 0u);
            const uint32_t v = two << (2 * (lane & 15));
            const uint32_t lo = __reduce_or_sync(0xffffffffu, lane < 16 ? v : 0u);
            const uint32_t hi = __reduce_or_sync(0xffffffffu, lane >= 16 ? v : 0u);
            if (lane == j) mine = (uint64_t)lo | ((uint64_t)hi << 32);
        }
        if (lane < 8) {
            const int64_t w = c * 8 + lane;
            if (w < wpr) out[r * wpr + w] = mine;
        }
    }
}

// ===========================================================================
// unpack (bool bytes and +-1 floats)
// ===========================================================================

// 16 consecutive bits of row `rowp` starting at bit `col` (col >= 0 and the 16
// bits lie inside the row's words).
__device__ __forceinline__ uint32_t row_bits16(const uint64_t* rowp, int64_t col, int64_t wpr) {
    const int64_t w = col >> 6;
    const int sh = (int)(col & 63);
    uint64_t x = __ldg(rowp + w) >> sh;
    if (sh > 48 && w + 1 < wpr) x |= __ldg(rowp + w + 1) << (64 - sh);
    return (uint32_t)x & 0xFFFFu;
}

// 4 consecutive bits starting at bit `col` (inside the row's words)
__device__ __forceinline__ uint32_t row_bits16_short(const uint64_t* rowp, int64_t col, int64_t wpr) {
    const int64_t w = col >> 6;
    const int sh = (int)(col & 63);
    uint64_t x = __ldg(rowp + w) >> sh;
    if (sh > 60 && w + 1 < wpr) x |= __ldg(rowp + w + 1) << (64 - sh);
    return (uint32_t)x & 0xFu;
}

// ELEM = bytes per output element (1: bool byte, 4: float +-1). A lane owns one
// 16-byte ALIGNED group of the output, i.e. EPG = 16/ELEM elements.
template <int ELEM, bool FLAT>
// 8 blocks per SM (32 registers): this kernel mostly writes, and measured 17 % faster at full
// occupancy than with the deeper unrolling the compiler picks when given more registers
__global__ void __launch_bounds__(256, 8)
k_unpack(const uint64_t* __restrict__ in, uint8_t* __restrict__ out,
         int64_t ll, int64_t wpr, TaskMap tm, int64_t tasks) {
    constexpr int EPG = 16 / ELEM;
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t task = warp; task < tasks; task += nwarps) {
        int64_t r, c;
        split_task<FLAT>(task, tm, r, c);
        const int64_t g = c * 32 + lane;
        const uint64_t* rowp = in + r * wpr;
        uint8_t* orow = out + r * ll * ELEM;
        const int m = (int)(reinterpret_cast<uintptr_t>(orow) & 15u) / ELEM;   // elements
        const int64_t col0 = g * EPG - m;            // first element of this lane's group
        if (col0 >= ll || col0 + EPG <= 0) continue;
        if (col0 >= 0 && col0 + EPG <= ll) {
            uint32_t bits;
            if (ELEM == 1) {
                bits = row_bits16(rowp, col0, wpr);
            } else {
                bits = row_bits16_short(rowp, col0, wpr);
            }
            uint4 v;
            if (ELEM == 1) {
                v.x = bits4_to_bytes01(bits);       v.y = bits4_to_bytes01(bits >> 4);
                v.z = bits4_to_bytes01(bits >> 8);  v.w = bits4_to_bytes01(bits >> 12);
            } else {
                // +1.0f = 0x3F800000, -1.0f = 0xBF800000: only the sign bit differs
                v.x = 0xBF800000u ^ ((bits & 1u) << 31);        v.y = 0xBF800000u ^ ((bits & 2u) << 30);
                v.z = 0xBF800000u ^ ((bits & 4u) << 29);        v.w = 0xBF800000u ^ ((bits & 8u) << 28);
            }
            stg_stream(orow + col0 * ELEM, v);
        } else {
            // ragged edge of a row: element-wise
#pragma unroll
            for (int i = 0; i < EPG; ++i) {
                const int64_t col = col0 + i;
                if (col < 0 || col >= ll) continue;
                const uint32_t bit = (uint32_t)(__ldg(rowp + (col >> 6)) >> (col & 63)) & 1u;
                if (ELEM == 1) orow[col] = (uint8_t)bit;
                else reinterpret_cast<float*>(orow)[col] = bit ? 1.0f : -1.0f;
            }
        }
    }
}

// The flat, 32-byte aligned case of the two unpacks with 256-bit stores (sm_100): a lane turns 32 bits
// into 32 bool bytes, or 8 bits into 8 floats, and a warp store covers 1 KB of contiguous output,
// half the store instructions of the 16-byte form for this write-bound kernel. n32 = number of
// 32-byte output groups.
__device__ __forceinline__ void stg_stream_256(void* p, const uint32_t (&r)[8]) {
    asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" :: "l"(p),
                 "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}

template <int ELEM>
__global__ void __launch_bounds__(256, 8)
k_unpack_flat256(const uint32_t* __restrict__ in32, uint8_t* __restrict__ out, int64_t n32) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < n32; g += stride) {
        uint32_t r[8];
        if (ELEM == 1) {
            const uint32_t bits = __ldg(in32 + g);
#pragma unroll
            for (int i = 0; i < 8; ++i) r[i] = bits4_to_bytes01(bits >> (4 * i));
        } else {
            // 8 bits of the packed stream per lane: byte g of it
            const uint32_t bits = __ldg(reinterpret_cast<const uint8_t*>(in32) + g);
#pragma unroll
            for (int i = 0; i < 8; ++i) r[i] = 0xBF800000u ^ (((bits >> i) & 1u) << 31);
        }
        stg_stream_256(out + g * 32, r);
    }
}

// Ragged rows (ll not a multiple of 64) with 256-bit stores: the OUTPUT is one dense byte stream
// (row r starts at element r * ll), so a lane owns a 32-byte aligned group of it wherever that falls.
// A group lies in one row, or - once per row - straddles the end of row r and the start of row
// r + 1; both cases take the same path: up to NB = 32 / ELEM bits from row r, and the remainder from
// the first word of row r + 1. No per-row task quantisation (4097-byte rows cost 8.002 warp stores
// instead of 9) and half the store instructions of the 16-byte form. Needs ll >= NB (at most two
// rows per group) and a 32-byte aligned output; the last, partial group is written element by element.
template <int NB>
__device__ __forceinline__ uint32_t row_bits_n(const uint64_t* __restrict__ rowp, uint32_t col, int64_t wpr) {
    const uint32_t w = col >> 6, sh = col & 63u;
    uint64_t x = __ldg(rowp + w) >> sh;
    if (sh + NB > 64u && (int64_t)w + 1 < wpr) x |= __ldg(rowp + w + 1) << (64u - sh);
    return NB == 32 ? (uint32_t)x : ((uint32_t)x & ((1u << NB) - 1u));
}

template <int ELEM, typename IDX>
__global__ void __launch_bounds__(256, 8)
k_unpack_ragged256(const uint64_t* __restrict__ in, uint8_t* __restrict__ out,
                   int64_t rows, IDX ll, int64_t wpr, int64_t total /* rows * ll elements */, int64_t n32) {
    constexpr int NB = 32 / ELEM;                  // elements (= bits) per 32-byte group
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < n32; g += stride) {
        const IDX e0 = (IDX)(g * NB);              // first element of the group
        const IDX r = e0 / ll;
        const uint32_t col0 = (uint32_t)(e0 - r * ll);      // ll < 2^32 on this path
        const uint64_t* rowp = in + (int64_t)r * wpr;
        uint32_t bits = row_bits_n<NB>(rowp, col0, wpr);
        const uint64_t n1 = (uint64_t)ll - col0;           // elements left in row r
        if (n1 < (uint64_t)NB) {                           // the group runs on into row r + 1
            bits &= (1u << (uint32_t)n1) - 1u;
            if ((int64_t)r + 1 < rows) bits |= (uint32_t)__ldg(rowp + wpr) << (uint32_t)n1;
        }
        uint32_t v[8];
        if (ELEM == 1) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = bits4_to_bytes01(bits >> (4 * i));
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0xBF800000u ^ (((bits >> i) & 1u) << 31);
        }
        if ((int64_t)e0 + NB <= total) {
            stg_stream_256(out + g * 32, v);
        } else {                                           // the stream's last, partial group
            for (int i = 0; (int64_t)e0 + i < total; ++i) {
                if (ELEM == 1) out[g * 32 + i] = (uint8_t)((bits >> i) & 1u);
                else reinterpret_cast<float*>(out)[g * 8 + i] = ((bits >> i) & 1u) ? 1.0f : -1.0f;
            }
        }
    }
}

// ---------------------------------------------------------------------------
static inline void flatten_rows(int64_t& rows, int64_t& len) {
    // rows of a multiple of 64 bits pack back to back: treat as one long row
    if (len % 64 == 0 || rows == 1) { len *= rows; rows = 1; }
}

}  // namespace bb

using namespace bb;

static inline TaskMap make_task_map(int64_t cpr, int64_t tasks) {
    TaskMap tm;
    tm.cpr = cpr;
    tm.cpr32 = (uint32_t)(cpr < 0xFFFFFFFFll ? cpr : 0xFFFFFFFFll);
    tm.small = (tasks < 0xFFFFFFFFll && cpr < 0xFFFFFFFFll) ? 1 : 0;
    return tm;
}

extern "C" int brute_b200_pack_bool(const uint8_t* in, uint64_t* out,
                                    int64_t rows, int64_t ld, void* stream) {
    BB_REQUIRE(rows >= 0 && ld >= 0, BRUTE_ERR_INVALID_ARG);
    if (rows == 0 || ld == 0) return BRUTE_OK;
    BB_REQUIRE(in != nullptr && out != nullptr, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(out), BRUTE_ERR_MISALIGNED);
    flatten_rows(rows, ld);
    const int64_t wpr = (ld + 63) / 64;
    const int64_t cpr = (wpr + 7) / 8;      // 32 groups of 16 bytes = 8 words per warp task
    const int64_t tasks = rows * cpr;
    const TaskMap tm = make_task_map(cpr, tasks);
    const int grid = stream_grid(tasks, 8, 8);
    const bool flat = rows == 1;
    const bool aligned = aligned16(in) && (flat || (ld & 15) == 0);
    cudaStream_t st = as_stream(stream);
    if (flat && aligned)  k_pack_bool<true, true><<<grid, 256, 0, st>>>(in, out, rows, ld, wpr, tm, tasks);
    else if (flat)        k_pack_bool<true, false><<<grid, 256, 0, st>>>(in, out, rows, ld, wpr, tm, tasks);
    else if (aligned)     k_pack_bool<false, true><<<grid, 256, 0, st>>>(in, out, rows, ld, wpr, tm, tasks);
    else {
        const int64_t nwords = rows * wpr;
        const int wgrid = stream_grid(nwords, 256, 4);
        if (nwords < (1ll << 32) && ld < (1ll << 32))
            k_pack_bool_words<uint32_t><<<wgrid, 256, 0, st>>>(in, out, rows, (uint32_t)ld, (uint32_t)wpr, nwords);
        else
            k_pack_bool_words<uint64_t><<<wgrid, 256, 0, st>>>(in, out, rows, (uint64_t)ld, (uint64_t)wpr, nwords);
    }
    return launch_status();
}

template <typename T, bool FLAT, int MODE>
static void launch_pack_sign_one(const T* in, uint64_t* out, int64_t rows, int64_t ld, cudaStream_t st) {
    const int64_t wpr = (ld + 63) / 64;
    const bool pair_ok = sizeof(T) == 2 && (reinterpret_cast<uintptr_t>(in) & 3u) == 0 &&
                         (rows == 1 || (ld & 1) == 0);
    if (pair_ok) {
        const int64_t cpr = (wpr + 7) / 8, tasks = rows * cpr;
        if constexpr (sizeof(T) == 2)
            k_pack_sign_pair16<T, FLAT, MODE><<<stream_grid(tasks, 8, 8), 256, 0, st>>>(
                in, out, ld, wpr, make_task_map(cpr, tasks), tasks);
    } else {
        const int64_t cpr = (wpr + 3) / 4, tasks = rows * cpr;
        k_pack_sign_ballot<T, FLAT, MODE><<<stream_grid(tasks, 8, 8), 256, 0, st>>>(
            in, out, ld, wpr, make_task_map(cpr, tasks), tasks);
    }
}

template <typename T>
static int launch_pack_sign(const T* in, uint64_t* out, int64_t rows, int64_t ld, int mode,
                            cudaStream_t st) {
    const bool flat = rows == 1;
    if (mode == BRUTE_SIGN_GE0) {
        if (flat) launch_pack_sign_one<T, true, BRUTE_SIGN_GE0>(in, out, rows, ld, st);
        else      launch_pack_sign_one<T, false, BRUTE_SIGN_GE0>(in, out, rows, ld, st);
    } else {
        if (flat) launch_pack_sign_one<T, true, BRUTE_SIGN_GT0>(in, out, rows, ld, st);
        else      launch_pack_sign_one<T, false, BRUTE_SIGN_GT0>(in, out, rows, ld, st);
    }
    return launch_status();
}

extern "C" int brute_b200_pack_sign(const void* in, int dtype, uint64_t* out,
                                    int64_t rows, int64_t ld, int mode, void* stream) {
    BB_REQUIRE(rows >= 0 && ld >= 0, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(mode == BRUTE_SIGN_GT0 || mode == BRUTE_SIGN_GE0, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(dtype == BRUTE_DT_F32 || dtype == BRUTE_DT_BF16 || dtype == BRUTE_DT_F16,
               BRUTE_ERR_UNSUPPORTED);
    if (rows == 0 || ld == 0) return BRUTE_OK;
    BB_REQUIRE(in != nullptr && out != nullptr, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(out), BRUTE_ERR_MISALIGNED);
    const uintptr_t esz = dtype == BRUTE_DT_F32 ? 4 : 2;
    BB_REQUIRE((reinterpret_cast<uintptr_t>(in) & (esz - 1)) == 0, BRUTE_ERR_MISALIGNED);
    flatten_rows(rows, ld);
    cudaStream_t st = as_stream(stream);
    switch (dtype) {
        case BRUTE_DT_F32:  return launch_pack_sign(static_cast<const float*>(in), out, rows, ld, mode, st);
        case BRUTE_DT_BF16: return launch_pack_sign(static_cast<const __nv_bfloat16*>(in), out, rows, ld, mode, st);
        default:            return launch_pack_sign(static_cast<const __half*>(in), out, rows, ld, mode, st);
    }
}

template <int ELEM>
static int launch_unpack(const uint64_t* in, void* out, int64_t rows, int64_t ll, cudaStream_t st) {
    const int64_t wpr = (ll + 63) / 64;     // words per packed row, from the UNflattened length
    int64_t frows = rows, fll = ll;
    int64_t fwpr = wpr;
    if (ll % 64 == 0 || rows == 1) { fll = ll * rows; frows = 1; fwpr = wpr * rows; }
    if (frows == 1 && (reinterpret_cast<uintptr_t>(out) & 31u) == 0 && (fll * ELEM) % 32 == 0) {
        const int64_t n32 = fll * ELEM / 32;
        k_unpack_flat256<ELEM><<<stream_grid(n32, 256, 8), 256, 0, st>>>(reinterpret_cast<const uint32_t*>(in),
                                                                      static_cast<uint8_t*>(out), n32);
        return launch_status();
    }
    if (frows > 1 && fll >= 32 / ELEM && fll < (1ll << 32) && (reinterpret_cast<uintptr_t>(out) & 31u) == 0) {
        const int64_t total = frows * fll, n32 = (total * ELEM + 31) / 32;
        const int grid = stream_grid(n32, 256, 8);
        if (total < (1ll << 32))
            k_unpack_ragged256<ELEM, uint32_t><<<grid, 256, 0, st>>>(in, static_cast<uint8_t*>(out), frows, (uint32_t)fll, fwpr, total, n32);
        else
            k_unpack_ragged256<ELEM, uint64_t><<<grid, 256, 0, st>>>(in, static_cast<uint8_t*>(out), frows, (uint64_t)fll, fwpr, total, n32);
        return launch_status();
    }
    constexpr int EPG = 16 / ELEM;
    // groups per row: the row may start up to EPG-1 elements into its first group
    const int64_t gpr = (fll + 2 * EPG - 2) / EPG;
    const int64_t cpr = (gpr + 31) / 32;
    const int64_t tasks = frows * cpr;
    const TaskMap tm = make_task_map(cpr, tasks);
    const int grid = stream_grid(tasks, 8, 8);
    if (frows == 1) k_unpack<ELEM, true><<<grid, 256, 0, st>>>(in, static_cast<uint8_t*>(out), fll, fwpr, tm, tasks);
    else            k_unpack<ELEM, false><<<grid, 256, 0, st>>>(in, static_cast<uint8_t*>(out), fll, fwpr, tm, tasks);
    return launch_status();
}

extern "C" int brute_b200_unpack_bool(const uint64_t* in, uint8_t* out,
                                      int64_t rows, int64_t ll, void* stream) {
    BB_REQUIRE(rows >= 0 && ll >= 0, BRUTE_ERR_INVALID_ARG);
    if (rows == 0 || ll == 0) return BRUTE_OK;
    BB_REQUIRE(in != nullptr && out != nullptr, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(in), BRUTE_ERR_MISALIGNED);
    return launch_unpack<1>(in, out, rows, ll, as_stream(stream));
}

extern "C" int brute_b200_unpack_pm1_f32(const uint64_t* in, float* out,
                                         int64_t rows, int64_t ll, void* stream) {
    BB_REQUIRE(rows >= 0 && ll >= 0, BRUTE_ERR_INVALID_ARG);
    if (rows == 0 || ll == 0) return BRUTE_OK;
    BB_REQUIRE(in != nullptr && out != nullptr, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(in) && (reinterpret_cast<uintptr_t>(out) & 3u) == 0, BRUTE_ERR_MISALIGNED);
    return launch_unpack<4>(in, out, rows, ll, as_stream(stream));
}
