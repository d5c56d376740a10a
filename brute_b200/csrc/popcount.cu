// popcount family: per-element, whole-buffer total, fused xor totals.
// All are HBM-bound: 128-bit loads, grid sized in whole waves over the SMs,
// one 64-bit atomic per block for the totals.
#include <atomic>
#include "common.cuh"
#include <algorithm>

namespace bb {

// ---------------------------------------------------------------------------
// per-element popcount -> int32. A thread takes one 16-byte vector of the
// input (16/EB elements) per trip.
// ---------------------------------------------------------------------------
template <int EB> __device__ __forceinline__ void popc_vec(uint4 v, int32_t* o);
template <> __device__ __forceinline__ void popc_vec<8>(uint4 v, int32_t* o) {
    o[0] = __popc(v.x) + __popc(v.y);
    o[1] = __popc(v.z) + __popc(v.w);
}
template <> __device__ __forceinline__ void popc_vec<4>(uint4 v, int32_t* o) {
    o[0] = __popc(v.x); o[1] = __popc(v.y); o[2] = __popc(v.z); o[3] = __popc(v.w);
}
template <> __device__ __forceinline__ void popc_vec<2>(uint4 v, int32_t* o) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { o[2 * i] = __popc(w[i] & 0xFFFFu); o[2 * i + 1] = __popc(w[i] >> 16); }
}
template <> __device__ __forceinline__ void popc_vec<1>(uint4 v, int32_t* o) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int b = 0; b < 4; ++b) o[4 * i + b] = __popc((w[i] >> (8 * b)) & 0xFFu);
    }
}

template <int EB>
__global__ void __launch_bounds__(256)
k_popcount_elems_vec(const uint8_t* __restrict__ in, int32_t* __restrict__ out, int64_t nvec) {
    constexpr int EPV = 16 / EB;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const uint4 v = ldg_stream(in + i * 16);
        int32_t o[EPV];
        popc_vec<EB>(v, o);
        int32_t* dst = out + i * EPV;
        if (EPV == 2) {
            *reinterpret_cast<int2*>(dst) = make_int2(o[0], o[1]);
        } else {
#pragma unroll
            for (int k = 0; k < EPV; k += 4)
                stg_stream(dst + k, make_uint4((uint32_t)o[k], (uint32_t)o[k + 1],
                                               (uint32_t)o[k + 2], (uint32_t)o[k + 3]));
        }
    }
}

// element-wise path for unaligned buffers and the tail after the last vector
template <typename U>
__global__ void __launch_bounds__(256)
k_popcount_elems_scalar(const U* __restrict__ in, int32_t* __restrict__ out, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = sizeof(U) == 8 ? __popcll((unsigned long long)in[i]) : __popc((uint32_t)in[i]);
}

// per-word popcount(a ^ b)
__global__ void __launch_bounds__(256)
k_hamming_words(const uint64_t* __restrict__ a, const uint64_t* __restrict__ b,
                int32_t* __restrict__ out, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = __popcll(__ldcs(a + i) ^ __ldcs(b + i));
}

// ---------------------------------------------------------------------------
// A total in ONE launch, with no memset of the result before it: the blocks add their partial sums
// into an accumulator that is zero at rest, take a ticket, and the block that draws the last ticket
// moves the sum to the caller's word and leaves accumulator and ticket zero again. The accumulators
// are static device memory (the library allocates nothing); the host hands the slots out round
// robin, so two totals collide only if kTotalSlots launches separate them and the first is still
// running (or if two captured graphs that hold the same slot are replayed at the same time).
// ---------------------------------------------------------------------------
constexpr int kTotalSlots = 256;
struct TotalSlot { unsigned long long acc; unsigned int ticket; unsigned int pad; };
__device__ TotalSlot g_total_slots[kTotalSlots];

__device__ __forceinline__ void total_finish(uint64_t block_sum, int slot, unsigned long long* out) {
    TotalSlot* s = &g_total_slots[slot];
    if (block_sum) atomicAdd(&s->acc, (unsigned long long)block_sum);
    __threadfence();
    if (atomicAdd(&s->ticket, 1u) == gridDim.x - 1) {      // every other block's sum is in
        __threadfence();
        *out = atomicExch(&s->acc, 0ull);
        s->ticket = 0;
    }
}

static inline int next_total_slot() {
    static std::atomic<unsigned> seq{0};
    return (int)(seq.fetch_add(1, std::memory_order_relaxed) % kTotalSlots);
}

// ---------------------------------------------------------------------------
// totals. TWO = false: sum popcount(a); TWO = true: sum popcount(a ^ b).
// `a` (and `b`) point at the first 16-byte aligned vector; head and tail bytes
// outside the vector range are added by thread 0 of block 0.
// ---------------------------------------------------------------------------
template <bool TWO>
__global__ void __launch_bounds__(256)
k_popcount_total(const uint8_t* __restrict__ a, const uint8_t* __restrict__ b,
                 int64_t head, int64_t nvec, int64_t tail, unsigned long long* __restrict__ out, int slot) {
    __shared__ uint64_t red[32];
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const uint8_t* av = a + head;
    const uint8_t* bv = TWO ? b + head : nullptr;
    uint64_t acc = 0;
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    // four independent 128-bit loads in flight per thread
    for (; i + 3 * stride < nvec; i += 4 * stride) {
        uint4 v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = ldg_stream(av + (i + k * stride) * 16);
        if (TWO) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint4 w = ldg_stream(bv + (i + k * stride) * 16);
                v[k].x ^= w.x; v[k].y ^= w.y; v[k].z ^= w.z; v[k].w ^= w.w;
            }
        }
        uint32_t s = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) s += __popc(v[k].x) + __popc(v[k].y) + __popc(v[k].z) + __popc(v[k].w);
        acc += s;
    }
    for (; i < nvec; i += stride) {
        uint4 v = ldg_stream(av + i * 16);
        if (TWO) {
            const uint4 w = ldg_stream(bv + i * 16);
            v.x ^= w.x; v.y ^= w.y; v.z ^= w.z; v.w ^= w.w;
        }
        acc += __popc(v.x) + __popc(v.y) + __popc(v.z) + __popc(v.w);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        for (int64_t k = 0; k < head; ++k) acc += __popc((uint32_t)(a[k] ^ (TWO ? b[k] : (uint8_t)0)));
        const int64_t t0 = head + nvec * 16;
        for (int64_t k = 0; k < tail; ++k) acc += __popc((uint32_t)(a[t0 + k] ^ (TWO ? b[t0 + k] : (uint8_t)0)));
    }
    acc = block_sum_u64(acc, red);
    if (threadIdx.x == 0) total_finish(acc, slot, out);
}

// a and b are misaligned differently: byte-granular scalar path (rare)
__global__ void __launch_bounds__(512)
k_hamming_total_bytes(const uint8_t* __restrict__ a, const uint8_t* __restrict__ b, int64_t n,
                      unsigned long long* __restrict__ out, int slot) {
    __shared__ uint64_t red[32];
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    uint64_t acc = 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        acc += __popc((uint32_t)(a[i] ^ b[i]));
    acc = block_sum_u64(acc, red);
    if (threadIdx.x == 0) total_finish(acc, slot, out);
}

static inline void split_aligned(const void* p, int64_t n_bytes, int64_t& head, int64_t& nvec, int64_t& tail) {
    head = (int64_t)((16 - (reinterpret_cast<uintptr_t>(p) & 15u)) & 15u);
    if (head > n_bytes) head = n_bytes;
    nvec = (n_bytes - head) / 16;
    tail = n_bytes - head - nvec * 16;
}

}  // namespace bb

using namespace bb;

extern "C" int brute_b200_popcount_elems(const void* in, int32_t* out, int64_t n,
                                         int elem_bytes, void* stream) {
    BB_REQUIRE(n >= 0, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(elem_bytes == 1 || elem_bytes == 2 || elem_bytes == 4 || elem_bytes == 8,
               BRUTE_ERR_UNSUPPORTED);
    if (n == 0) return BRUTE_OK;
    BB_REQUIRE(in != nullptr && out != nullptr, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE((reinterpret_cast<uintptr_t>(in) & (uintptr_t)(elem_bytes - 1)) == 0 &&
               (reinterpret_cast<uintptr_t>(out) & 3u) == 0, BRUTE_ERR_MISALIGNED);
    cudaStream_t st = as_stream(stream);
    const int epv = 16 / elem_bytes;
    int64_t nvec = (aligned16(in) && aligned16(out)) ? n / epv : 0;
    if (nvec > 0) {
        const int grid = stream_grid(nvec, 256, 8);
        const uint8_t* p = static_cast<const uint8_t*>(in);
        switch (elem_bytes) {
            case 8: k_popcount_elems_vec<8><<<grid, 256, 0, st>>>(p, out, nvec); break;
            case 4: k_popcount_elems_vec<4><<<grid, 256, 0, st>>>(p, out, nvec); break;
            case 2: k_popcount_elems_vec<2><<<grid, 256, 0, st>>>(p, out, nvec); break;
            default: k_popcount_elems_vec<1><<<grid, 256, 0, st>>>(p, out, nvec); break;
        }
        if (int rc = launch_status()) return rc;
    }
    const int64_t done = nvec * epv, rest = n - done;
    if (rest > 0) {
        const int grid = stream_grid(rest, 256, 8);
        const uint8_t* p = static_cast<const uint8_t*>(in) + done * elem_bytes;
        int32_t* o = out + done;
        switch (elem_bytes) {
            case 8: k_popcount_elems_scalar<<<grid, 256, 0, st>>>(reinterpret_cast<const uint64_t*>(p), o, rest); break;
            case 4: k_popcount_elems_scalar<<<grid, 256, 0, st>>>(reinterpret_cast<const uint32_t*>(p), o, rest); break;
            case 2: k_popcount_elems_scalar<<<grid, 256, 0, st>>>(reinterpret_cast<const uint16_t*>(p), o, rest); break;
            default: k_popcount_elems_scalar<<<grid, 256, 0, st>>>(p, o, rest); break;
        }
    }
    return launch_status();
}

extern "C" int brute_b200_hamming_words(const uint64_t* a, const uint64_t* b, int32_t* out,
                                        int64_t n_words, void* stream) {
    BB_REQUIRE(n_words >= 0, BRUTE_ERR_INVALID_ARG);
    if (n_words == 0) return BRUTE_OK;
    BB_REQUIRE(a && b && out, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(a) && aligned8(b), BRUTE_ERR_MISALIGNED);
    k_hamming_words<<<stream_grid(n_words, 256, 8), 256, 0, as_stream(stream)>>>(a, b, out, n_words);
    return launch_status();
}

extern "C" int brute_b200_popcount_total(const void* in, int64_t n_bytes, uint64_t* out, void* stream) {
    BB_REQUIRE(n_bytes >= 0 && out != nullptr, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(out), BRUTE_ERR_MISALIGNED);
    cudaStream_t st = as_stream(stream);
    if (n_bytes == 0) return cudaMemsetAsync(out, 0, sizeof(uint64_t), st) == cudaSuccess ? BRUTE_OK : BRUTE_ERR_LAUNCH;
    BB_REQUIRE(in != nullptr, BRUTE_ERR_INVALID_ARG);
    int64_t head, nvec, tail;
    split_aligned(in, n_bytes, head, nvec, tail);
    static const int per_launch = resident_grid(k_popcount_total<false>, 256, 1 << 30);
    const int grid = (int)std::min<int64_t>(per_launch, std::max<int64_t>(1, (nvec + 256 * 4 - 1) / (256 * 4)));
    k_popcount_total<false><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(in), nullptr, head, nvec, tail,
                                                  reinterpret_cast<unsigned long long*>(out), next_total_slot());
    return launch_status();
}

extern "C" int brute_b200_hamming_total(const void* a, const void* b, int64_t n_bytes,
                                        uint64_t* out, void* stream) {
    BB_REQUIRE(n_bytes >= 0 && out != nullptr, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(out), BRUTE_ERR_MISALIGNED);
    cudaStream_t st = as_stream(stream);
    if (n_bytes == 0) return cudaMemsetAsync(out, 0, sizeof(uint64_t), st) == cudaSuccess ? BRUTE_OK : BRUTE_ERR_LAUNCH;
    BB_REQUIRE(a != nullptr && b != nullptr, BRUTE_ERR_INVALID_ARG);
    auto* o = reinterpret_cast<unsigned long long*>(out);
    if ((reinterpret_cast<uintptr_t>(a) & 15u) != (reinterpret_cast<uintptr_t>(b) & 15u)) {
        k_hamming_total_bytes<<<stream_grid(n_bytes, 512 * 16, 4), 512, 0, st>>>(
            static_cast<const uint8_t*>(a), static_cast<const uint8_t*>(b), n_bytes, o, next_total_slot());
        return launch_status();
    }
    int64_t head, nvec, tail;
    split_aligned(a, n_bytes, head, nvec, tail);
    static const int per_launch = resident_grid(k_popcount_total<true>, 256, 1 << 30);
    const int grid = (int)std::min<int64_t>(per_launch, std::max<int64_t>(1, (nvec + 256 * 4 - 1) / (256 * 4)));
    k_popcount_total<true><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(a), static_cast<const uint8_t*>(b),
                                                 head, nvec, tail, o, next_total_slot());
    return launch_status();
}
