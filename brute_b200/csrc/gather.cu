// Transport form of the GEMM result for the all-gather of a column-sharded GEMM.
//
// C = K - 2H lies in [-K, K]: for K <= 32767 an int16 carries it exactly, so the ranks exchange
// int16 blocks (half the NVLink bytes of the int32 result) and every rank widens what it received
// straight into its replicated int32 matrix. The widening pass also does the layout change that the
// gather leaves behind: NCCL delivers the rank blocks stacked, [world, rows, n_loc], and the result
// is row major [rows, world * n_loc].
// Both kernels are HBM bound; 128-bit loads and stores, grid sized to the SMs.
#include <cstdlib>
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


// ---------------------------------------------------------------------------
// The same exchange over PEER MEMORY, gather and widening in one pass.
//
// Every rank narrows its blocks of C into a buffer that its peers can read (symmetric memory,
// mapped by the host side), raises a flag per row block, and a rank's result is assembled by ONE
// kernel per row block: for each peer it waits for that peer's flag, reads the peer's int16 block
// with plain peer loads over NVLink and stores the widened int32 values where they belong in the
// row-major result. Against all-gather + unstack this drops a pass over HBM (the staged copy of
// everybody's blocks: 0.5 GiB written and read again, and a 0.3 ms kernel at 16384^2 on 8 GPUs) and
// the collective's launch. No multicast, no library kernel touches peer memory.
//
// Flags are 32-bit words in the owner's buffer, written by the owner only (st.release.sys after a
// system fence, from a one-thread kernel queued behind the narrowing pass) and read by the peers
// (ld.acquire.sys). Values are call numbers, so nothing is ever reset. Every wait is bounded: a
// flag that does not arrive within the limit makes the block record the fact and return.
// ---------------------------------------------------------------------------
constexpr int kMaxPeers = 16;
struct PeerBlocks {
    const int16_t* send[kMaxPeers];      // rank p's narrowed blocks, [M, n_loc] int16
    const uint32_t* flags[kMaxPeers];    // rank p's flag words
};

__device__ int g_peer_wait_status;      // 0, or 1 + the rank whose flag did not arrive

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t peer_globaltimer() {
    uint64_t t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t;
}
// true once *flag >= want (call numbers only grow; wrap-around after 2^31 calls is handled by the
// signed difference); false after limit_ns
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t want, uint64_t limit_ns) {
    if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
    const uint64_t t0 = peer_globaltimer();
    while (true) {
        if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
        if (peer_globaltimer() - t0 > limit_ns) return false;
        __nanosleep(200);
    }
}

__global__ void k_peer_set_flag(uint32_t* flag, uint32_t value) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(flag), "r"(value) : "memory");
}

// one thread per peer: every peer's word `index` has reached `want` (used before a send buffer is
// written again: the peers have finished reading what it held two calls ago)
__global__ void k_peer_wait_flags(PeerBlocks t, int world, int self, int index, uint32_t want, uint64_t limit_ns) {
    const int p = threadIdx.x;
    if (p >= world || p == self) return;
    if (!wait_flag(t.flags[p] + index, want, limit_ns)) atomicCAS(&g_peer_wait_status, 0, 1 + p);
}

// grid = (chunks, world): blockIdx.y picks the peer (rotated, so that the ranks do not all read the
// same peer at the same moment), blockIdx.x a share of the rows [m0, m1). n_loc is a multiple of 8.
__global__ void __launch_bounds__(256)
k_gather_peer_widen(PeerBlocks t, int32_t* __restrict__ out, int64_t ldc, int64_t n_loc,
                    int64_t m0, int64_t m1, int world, int self, int flag_index, uint32_t want, uint64_t limit_ns) {
    const int p = (self + 1 + (int)blockIdx.y) % world;      // the own block comes last: it needs no link
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        s_ok = 1;
        if (p != self && !wait_flag(t.flags[p] + flag_index, want, limit_ns)) {
            s_ok = 0;
            atomicCAS(&g_peer_wait_status, 0, 1 + p);
        }
    }
    __syncthreads();
    if (!s_ok) return;
    const int64_t v_per_row = n_loc / 8;
    const int64_t total = (m1 - m0) * v_per_row;
    const int16_t* src0 = t.send[p] + m0 * n_loc;
    int32_t* dst0 = out + m0 * ldc + (int64_t)p * n_loc;
    // Peer loads have a latency of microseconds: eight independent 16-byte loads per thread are in
    // flight before the first store (one per thread and trip moved 2 GB/s per CTA; this moves ~20).
    constexpr int UNROLL = 8;
    const bool small = total < (1ll << 32);
    const int64_t chunk = (int64_t)blockDim.x * UNROLL;
    for (int64_t base_i = (int64_t)blockIdx.x * chunk; base_i < total; base_i += (int64_t)gridDim.x * chunk) {
        uint4 a[UNROLL];
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {
            const int64_t i = base_i + (int64_t)k * blockDim.x + threadIdx.x;
            a[k] = make_uint4(0u, 0u, 0u, 0u);
            if (i < total) {
                int64_t m, v;
                if (small) { const uint32_t mm = (uint32_t)i / (uint32_t)v_per_row; m = mm; v = (uint32_t)i - mm * (uint32_t)v_per_row; }
                else { m = i / v_per_row; v = i - m * v_per_row; }
                const int16_t* src = src0 + m * n_loc + v * 8;
                asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a[k].x), "=r"(a[k].y), "=r"(a[k].z), "=r"(a[k].w) : "l"(src));
            }
        }
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {
            const int64_t i = base_i + (int64_t)k * blockDim.x + threadIdx.x;
            if (i < total) {
                int64_t m, v;
                if (small) { const uint32_t mm = (uint32_t)i / (uint32_t)v_per_row; m = mm; v = (uint32_t)i - mm * (uint32_t)v_per_row; }
                else { m = i / v_per_row; v = i - m * v_per_row; }
                int32_t* dst = dst0 + m * ldc + v * 8;
                stg_stream(dst,     make_uint4((uint32_t)sx16(a[k].x), (uint32_t)sx16(a[k].x >> 16), (uint32_t)sx16(a[k].y), (uint32_t)sx16(a[k].y >> 16)));
                stg_stream(dst + 4, make_uint4((uint32_t)sx16(a[k].z), (uint32_t)sx16(a[k].z >> 16), (uint32_t)sx16(a[k].w), (uint32_t)sx16(a[k].w >> 16)));
            }
        }
    }
}


// The same kernel with bulk copies (TMA, no multicast) instead of per-thread loads. Peer loads take
// microseconds, so the rate of a puller is the bytes it keeps in flight: registers hold 32 KB per CTA
// (measured 10 GB/s per CTA), shared memory a ring of GP_STAGES x 16 KB. One thread issues
// cp.async.bulk from the peer's block (contiguous: [m0, m1) x n_loc int16) into the ring; all threads
// widen a landed stage into the result and the stage is refilled.
constexpr int GP_STAGE_BYTES = 16384, GP_STAGES = 6, GP_THREADS = 256;
constexpr int GP_SMEM = GP_STAGES * GP_STAGE_BYTES + 128;

__device__ __forceinline__ bool gp_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// EB = bytes per element of the peers' blocks: 2 (int16, widened on the way) or 4 (int32, for K > 32767)
template <int EB>
__global__ void __launch_bounds__(GP_THREADS)
k_gather_peer_widen_bulk(PeerBlocks t, int32_t* __restrict__ out, int64_t ldc, int64_t n_loc,
                         int64_t m0, int64_t m1, int world, int self, int flag_index, uint32_t want, uint64_t limit_ns) {
    extern __shared__ __align__(128) uint8_t gp_smem[];
    const int p = (self + 1 + (int)blockIdx.y) % world;
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(gp_smem);
    const uint32_t bars = ring + GP_STAGES * GP_STAGE_BYTES;                 // GP_STAGES mbarriers
    __shared__ int s_ok;
    const int64_t block_bytes = (m1 - m0) * n_loc * EB;
    const int64_t n_tiles = (block_bytes + GP_STAGE_BYTES - 1) / GP_STAGE_BYTES;
    const uint8_t* src0 = reinterpret_cast<const uint8_t*>(t.send[p]) + m0 * n_loc * EB;
    auto tile_bytes = [&](int64_t tile) -> uint32_t {
        const int64_t left = block_bytes - tile * GP_STAGE_BYTES;
        return (uint32_t)(left < GP_STAGE_BYTES ? left : GP_STAGE_BYTES);
    };
    auto issue = [&](int s, int64_t tile) {                                   // thread 0 only
        const uint32_t bytes = tile_bytes(tile);
        const uint32_t bar = bars + 8u * s;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     :: "r"(ring + (uint32_t)s * GP_STAGE_BYTES), "l"(src0 + tile * GP_STAGE_BYTES), "r"(bytes), "r"(bar) : "memory");
    };
    if (threadIdx.x == 0) {
        for (int s = 0; s < GP_STAGES; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bars + 8u * s), "r"(1u) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_ok = 1;
        if (p != self && !wait_flag(t.flags[p] + flag_index, want, limit_ns)) {
            s_ok = 0;
            atomicCAS(&g_peer_wait_status, 0, 1 + p);
        }
        if (s_ok)
            for (int s = 0; s < GP_STAGES; ++s) {
                const int64_t tile = (int64_t)blockIdx.x + (int64_t)s * gridDim.x;
                if (tile < n_tiles) issue(s, tile);
            }
    }
    __syncthreads();
    if (!s_ok) return;
    int32_t* dst0 = out + m0 * ldc + (int64_t)p * n_loc;
    const bool small = (m1 - m0) * n_loc < (1ll << 32);
    int64_t k = 0;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++k) {
        const int s = (int)(k % GP_STAGES);
        const uint32_t parity = (uint32_t)(k / GP_STAGES) & 1u;
        const uint32_t bar = bars + 8u * s;
        // bounded: a copy that does not land within the limit is recorded and the CTA stops issuing
        // (copies already in flight are waited for below before the CTA leaves)
        if (!gp_try(bar, parity)) {
            const uint64_t t0 = peer_globaltimer();
            bool landed = false;
            while (peer_globaltimer() - t0 <= limit_ns) {
                if (gp_try(bar, parity)) { landed = true; break; }
            }
            if (!landed) { atomicCAS(&g_peer_wait_status, 0, 1 + p); s_ok = 0; }
        }
        __syncthreads();                        // also publishes s_ok
        if (!s_ok) break;
        const uint32_t nvec = tile_bytes(tile) / 16;
        constexpr int EPV = 16 / EB;                                          // elements per 16-byte vector
        const int64_t e0 = tile * (GP_STAGE_BYTES / EB);                      // first element of the tile inside the block
        for (uint32_t v = threadIdx.x; v < nvec; v += GP_THREADS) {
            const uint4 a = *reinterpret_cast<const uint4*>(gp_smem + (size_t)s * GP_STAGE_BYTES + 16u * v);
            const int64_t e = e0 + (int64_t)EPV * v;
            int64_t m, j;
            if (small) {                        // a 64-bit division per vector costs more than the vector's copy
                const uint32_t mm = (uint32_t)e / (uint32_t)n_loc;
                m = mm; j = (uint32_t)e - mm * (uint32_t)n_loc;
            } else { m = e / n_loc; j = e - m * n_loc; }
            int32_t* dst = dst0 + m * ldc + j;
            if (EB == 2) {
                stg_stream(dst,     make_uint4((uint32_t)sx16(a.x), (uint32_t)sx16(a.x >> 16), (uint32_t)sx16(a.y), (uint32_t)sx16(a.y >> 16)));
                stg_stream(dst + 4, make_uint4((uint32_t)sx16(a.z), (uint32_t)sx16(a.z >> 16), (uint32_t)sx16(a.w), (uint32_t)sx16(a.w >> 16)));
            } else {
                stg_stream(dst, a);
            }
        }
        __syncthreads();                        // the stage has been read by everyone
        if (threadIdx.x == 0) {
            const int64_t next = tile + (int64_t)GP_STAGES * gridDim.x;
            if (next < n_tiles) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic reads before the async write
                issue(s, next);
            }
        }
    }
    if (!s_ok && threadIdx.x == 0) {
        // gave up: the copies still in flight must land (or their limit pass) before the shared memory goes
        for (int d = 0; d < GP_STAGES; ++d) {      // iterations k .. k + 5 are the ones whose copies were issued
            const int64_t kk = k + d;
            if ((int64_t)blockIdx.x + kk * gridDim.x >= n_tiles) break;
            const uint32_t bar = bars + 8u * (uint32_t)(kk % GP_STAGES), parity = (uint32_t)(kk / GP_STAGES) & 1u;
            const uint64_t t0 = peer_globaltimer();
            while (!gp_try(bar, parity) && peer_globaltimer() - t0 <= limit_ns) {}
        }
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


// ---- peer-memory exchange -------------------------------------------------------------------
static bool peer_table(bb::PeerBlocks& t, const void* const* send_ptrs, const void* const* flag_ptrs, int world) {
    if (world < 1 || world > bb::kMaxPeers || !send_ptrs || !flag_ptrs) return false;
    for (int p = 0; p < bb::kMaxPeers; ++p) {
        t.send[p] = p < world ? static_cast<const int16_t*>(send_ptrs[p]) : nullptr;
        t.flags[p] = p < world ? static_cast<const uint32_t*>(flag_ptrs[p]) : nullptr;
        if (p < world && (!t.send[p] || !t.flags[p])) return false;
    }
    return true;
}

extern "C" int brute_b200_peer_set_flag(uint32_t* flag, uint32_t value, void* stream) {
    BB_REQUIRE(flag != nullptr && (reinterpret_cast<uintptr_t>(flag) & 3u) == 0, BRUTE_ERR_INVALID_ARG);
    bb::k_peer_set_flag<<<1, 1, 0, as_stream(stream)>>>(flag, value);
    return launch_status();
}

extern "C" int brute_b200_peer_wait_flags(const void* const* send_ptrs, const void* const* flag_ptrs, int world, int self,
                                          int index, uint32_t want, int64_t limit_us, void* stream) {
    bb::PeerBlocks t;
    BB_REQUIRE(peer_table(t, send_ptrs, flag_ptrs, world) && self >= 0 && self < world && index >= 0 && limit_us > 0, BRUTE_ERR_INVALID_ARG);
    bb::k_peer_wait_flags<<<1, 32, 0, as_stream(stream)>>>(t, world, self, index, want, (uint64_t)limit_us * 1000ull);
    return launch_status();
}

extern "C" int brute_b200_gather_peer_widen(const void* const* send_ptrs, const void* const* flag_ptrs, int32_t* out,
                                            int64_t M, int64_t n_loc, int elem_bytes, int64_t m0, int64_t m1, int world, int self,
                                            int flag_index, uint32_t want, int ctas_per_peer, int64_t limit_us, void* stream) {
    bb::PeerBlocks t;
    BB_REQUIRE(peer_table(t, send_ptrs, flag_ptrs, world) && self >= 0 && self < world, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(out != nullptr && M >= 0 && 0 <= m0 && m0 <= m1 && m1 <= M && n_loc >= 0 && flag_index >= 0 && limit_us > 0, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(elem_bytes == 2 || elem_bytes == 4, BRUTE_ERR_UNSUPPORTED);
    BB_REQUIRE(n_loc % (16 / elem_bytes) == 0 && aligned16(out), BRUTE_ERR_MISALIGNED);
    for (int p = 0; p < world; ++p) BB_REQUIRE(aligned16(t.send[p]), BRUTE_ERR_MISALIGNED);
    if (m1 == m0 || n_loc == 0) return BRUTE_OK;
    if (ctas_per_peer < 1) ctas_per_peer = 8;
    const dim3 grid((unsigned)ctas_per_peer, (unsigned)world);
    static const bool use_loads = std::getenv("BRUTE_B200_PEER_LOADS") != nullptr;       // the per-thread-load form, for comparison
    if (use_loads && elem_bytes == 2) {
        bb::k_gather_peer_widen<<<grid, 256, 0, as_stream(stream)>>>(t, out, (int64_t)world * n_loc, n_loc, m0, m1, world, self,
                                                                   flag_index, want, (uint64_t)limit_us * 1000ull);
        return launch_status();
    }
    if (elem_bytes == 2) {
        if (!kernel_smem_ready<bb::k_gather_peer_widen_bulk<2>>(bb::GP_SMEM)) return BRUTE_ERR_LAUNCH;
        bb::k_gather_peer_widen_bulk<2><<<grid, bb::GP_THREADS, bb::GP_SMEM, as_stream(stream)>>>(
            t, out, (int64_t)world * n_loc, n_loc, m0, m1, world, self, flag_index, want, (uint64_t)limit_us * 1000ull);
    } else {
        if (!kernel_smem_ready<bb::k_gather_peer_widen_bulk<4>>(bb::GP_SMEM)) return BRUTE_ERR_LAUNCH;
        bb::k_gather_peer_widen_bulk<4><<<grid, bb::GP_THREADS, bb::GP_SMEM, as_stream(stream)>>>(
            t, out, (int64_t)world * n_loc, n_loc, m0, m1, world, self, flag_index, want, (uint64_t)limit_us * 1000ull);
    }
    return launch_status();
}

// 0, or 1 + the rank whose flag a bounded wait of the peer kernels gave up on; reading clears it.
// Synchronises the device (for tests and for the host side's error report after a call).
extern "C" int brute_b200_peer_wait_status(void) {
    int v = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&v, bb::g_peer_wait_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) { const int zero = 0; cudaMemcpyToSymbol(bb::g_peer_wait_status, &zero, sizeof(int)); }
    return v;
}
