// xnor-popcount GEMM on tcgen05.mma kind::i8 with cta_group::2: two CTAs of a cluster (two SMs)
// share one 256 x 256 tile of C.
//
// Same arithmetic as the one-CTA kernel in gemm_tcgen05.cuh (AND-form expansion, weights 2^j and
// 2^(7-j), C = K - 2*pa - 2*pb + 4*(acc >> 7)); what changes is who expands what. The pair issues
// ONE M=256 N=256 K=32 instruction per 32 bytes of K from the leader CTA (cluster rank 0). Each
// CTA owns 128 rows of A (its 128 TMEM lanes of the accumulator) and supplies HALF of B:
// rank r expands rows [128 r, 128 r + 128) of the B tile into its own shared memory and the
// tensor cores of both SMs read both halves. Per 128-bit k-block a CTA therefore expands
// 128 + 128 rows instead of 128 + 256: a third less ALU work, half the B stores and half
// the B operand reads on each SM's shared-memory pipe, which is what bounds the one-CTA kernel.
//
// Per CTA (576 threads, as in the one-CTA kernel):
//   warp 16      TMA producer (own A rows, own half of B; no multicast), 3-deep packed ring.
//   warps 0..15  expanders, two groups alternating k-blocks; A -> own TMEM lanes (tcgen05.st),
//                B half -> own shared memory (SWIZZLE_128B), then ONE arrive per warp on the
//                LEADER's "expanded" barrier (remote mbarrier arrive, release at cluster scope).
//   warp 17      rank 0: MMA issuer; its tcgen05.commit is issued twice, once per CTA, so both
//                CTAs' expanders see the ring slot free. Both ranks: TMEM allocation (cta_group::2).
//   warps 0..15  epilogue of the CTA's own 128 x 256 accumulator half. The row popcounts of the
//                other half of B come from the peer through distributed shared memory.
// Every wait on an mbarrier is bounded (about a second) exactly as in the one-CTA kernel; the only
// unbounded waits are the cluster barriers at entry and exit, which every thread of both CTAs
// reaches on every path.
#pragma once
#include "gemm_tcgen05.cuh"

namespace bb {

constexpr int TP_BM = 128;                               // rows of C per CTA (256 per pair)
constexpr int TP_BN = 256;                               // columns of C per pair
constexpr int TP_BNH = TP_BN / 2;                        // rows of B expanded by one CTA
constexpr int TP_PSTAGES = 3, TP_ESTAGES = 6;          // 12 k-blocks of packed prefetch, 6 expanded k-blocks in flight
constexpr int TP_P_A = TP_BM * TC_PK, TP_P_B = TP_BNH * TC_PK;
constexpr int TP_P_STAGE = TP_P_A + TP_P_B;              // 16 KB
constexpr int TP_E_STAGE = TP_BNH * 128;                 // expanded half of B of one k-block: 16 KB
constexpr int TP_ROWPOP_BYTES = (TP_BM + TP_BN) * 4;
constexpr int TP_SMEM = TP_ESTAGES * TP_E_STAGE + TP_PSTAGES * TP_P_STAGE + 256 + TP_ROWPOP_BYTES + 1024;
static_assert(12 % (2 * TP_ESTAGES) == 0 && TP_PSTAGES * TC_KB_PER_STAGE == 12, "ring parities must be constants of the 12-step unroll");
static_assert(TC_ACC_COLS + TP_ESTAGES * TC_A_COLS <= TC_TMEM_COLS, "A ring must fit beside the accumulator");

// kind::i8, D = s32, A = B = unsigned int8, K-major, M = 256 (128 per CTA), N = 256
constexpr uint32_t TP_IDESC = (2u << 4) | ((uint32_t)(TP_BN >> 3) << 17) | ((uint32_t)((2 * TP_BM) >> 4) << 24);

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r;
}
// shared::cta address of this CTA -> shared::cluster address of the same offset in CTA `rank`
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank)); return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(cluster_addr) : "memory");
}
// The per-k-block signal. A release at cluster scope costs the arriving warp several hundred
// cycles per k-block; what the leader's MMA reads was written by st.shared + fence.proxy.async
// (this SM's shared memory) and tcgen05.st + wait::st (this SM's tensor memory), both complete
// before the arrive leaves the SM, so the CTA-scope default is what the loop uses.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" :: "r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_cl(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait whose acquire reaches the peer CTA's writes
__device__ __forceinline__ bool mbar_wait_cl(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    if (mbar_try_cl(bar, parity)) return true;
    const uint64_t t0 = tc_globaltimer();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_cl(bar, parity)) return true;
        if (((++spins) & 0xFFu) == 0) {
            if (*abort_flag) return false;
            if (tc_globaltimer() - t0 > TC_WAIT_NS) {
                *abort_flag = 1;
                atomicCAS(&g_tc_status, 0, code);
                return false;
            }
        }
    }
}
// completion of every tcgen05 op this thread issued so far -> one arrival on a barrier of either CTA
__device__ __forceinline__ void tp_commit(uint32_t cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tp_mma_i8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
                 :: "r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

struct PairExpanderCtx {
    uint32_t bars, p_ring, e_full_leader;   // e_full_leader: shared::cluster address of the leader's e_full[0]
    uint32_t lds_off[4], sts_addr[4], a_lds_off[4], a_taddr;
    int pc_a, pc_b;
    volatile int* abort_flag;
    int lane;
};

// One k-block of one group; U = k-block index modulo 12, so every ring index is a constant.
template <int G, int U>
__device__ __forceinline__ bool tp_expander_step(PairExpanderCtx& cx, uint32_t p_parity) {
    constexpr int S = U / TC_KB_PER_STAGE, KB = U % TC_KB_PER_STAGE, R = U % TP_ESTAGES;
    constexpr uint32_t E_PARITY = ((U / TP_ESTAGES) & 1) ^ 1;
    const uint32_t p_full = cx.bars + 8u * S, p_empty = cx.bars + 8u * (TP_PSTAGES + S);
    const uint32_t e_empty = cx.bars + 8u * (2 * TP_PSTAGES + TP_ESTAGES + R);
    if (KB == G) {
        if (!__all_sync(0xffffffffu, mbar_wait(p_full, p_parity, cx.abort_flag, 3))) return false;
    }
    const uint2 a = lds64<S * TP_P_STAGE>(cx.p_ring + cx.a_lds_off[KB]);
    const uint2 b = lds64<S * TP_P_STAGE + TP_P_A>(cx.p_ring + cx.lds_off[KB]);
    if (KB == G + 2) {
        // as in the one-CTA kernel: an arrival that a ragged last stage skips is never waited for
        __syncwarp();
        if (cx.lane == 0) mbar_arrive(p_empty);
    }
    cx.pc_a += __popc(a.x) + __popc(a.y);
    cx.pc_b += __popc(b.x) + __popc(b.y);
    if (!__all_sync(0xffffffffu, mbar_wait(e_empty, E_PARITY, cx.abort_flag, 4))) return false;
    tc_fence_after();
    tc_expand_a_half(a, cx.a_taddr + (uint32_t)(R * TC_A_COLS));
    tc_expand_b_half<R * TP_E_STAGE>(b, cx.sts_addr);
    tc_wait_st();
    tc_fence_before();
    fence_proxy_async_smem();
    __syncwarp();
    if (cx.lane == 0) mbar_arrive_remote(cx.e_full_leader + 8u * R);
    return true;
}

template <int G, int U>
__device__ __forceinline__ bool tp_expander_steps(PairExpanderCtx& cx, int32_t i0, int32_t nkb, uint32_t p_parity) {
    if constexpr (U < 12) {
        if (i0 + U >= nkb) return true;
        if constexpr ((U & 1) == G) {
            if (!tp_expander_step<G, U>(cx, p_parity)) return false;
        }
        return tp_expander_steps<G, U + 1>(cx, i0, nkb, p_parity);
    } else {
        return true;
    }
}

template <bool PACK>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
k_xnor_gemm_tcgen05_pair(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         int64_t M, int64_t N, int32_t nkb /* 128-bit k-blocks */, int32_t klogical /* K */,
                         int32_t* __restrict__ C, int64_t ldc,
                         const float* __restrict__ scale, uint32_t* __restrict__ out32, int64_t halves_per_row, int mode) {
    extern __shared__ uint8_t tc_smem_raw[];
    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(tc_smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gbase = tc_smem_raw + (base - raw);
    const uint32_t e_ring = base;                                    // TP_ESTAGES x 16 KB (expanded half of B)
    const uint32_t p_ring = base + TP_ESTAGES * TP_E_STAGE;          // TP_PSTAGES x 16 KB
    const uint32_t bars = p_ring + TP_PSTAGES * TP_P_STAGE;
    uint8_t* gbars = gbase + TP_ESTAGES * TP_E_STAGE + TP_PSTAGES * TP_P_STAGE;
    auto p_full  = [&](int s) { return bars + 8u * s; };
    auto p_empty = [&](int s) { return bars + 8u * (TP_PSTAGES + s); };
    auto e_full  = [&](int s) { return bars + 8u * (2 * TP_PSTAGES + s); };
    auto e_empty = [&](int s) { return bars + 8u * (2 * TP_PSTAGES + TP_ESTAGES + s); };
    constexpr int NB = 2 * TP_PSTAGES + 2 * TP_ESTAGES;
    const uint32_t acc_full = bars + 8u * NB;
    const uint32_t drain_bar = acc_full + 8u;
    const uint32_t pb_bar = acc_full + 16u;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbars + 8 * (NB + 3));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbars + 8 * (NB + 3) + 4);
    volatile int* skip_slot = reinterpret_cast<volatile int*>(gbars + 8 * (NB + 3) + 8);
    const uint32_t skip_addr = bars + 8u * (NB + 3) + 8u;

    int* pa_s = reinterpret_cast<int*>(gbars + 256);      // set bits per A row of this CTA's 128 rows
    int* pb_s = pa_s + TP_BM;                             // set bits per B row of the pair's 256 rows
    const uint32_t pb_addr = bars + 256u + 4u * TP_BM;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t rank = cluster_ctarank(), peer = rank ^ 1u;
    const int64_t m0 = (int64_t)blockIdx.x * TP_BM, n0 = (int64_t)blockIdx.y * TP_BN;
    const int32_t nstages = (nkb + TC_KB_PER_STAGE - 1) / TC_KB_PER_STAGE;

    if (tid < TP_BM + TP_BN) pa_s[tid] = 0;
    if (tid == 0) {
        for (int s = 0; s < TP_PSTAGES; ++s) { mbar_init(p_full(s), 1); mbar_init(p_empty(s), TC_EXP_WARPS); }
        // "expanded" counts the warps of one group in BOTH CTAs (only the leader's copy is used)
        for (int s = 0; s < TP_ESTAGES; ++s) { mbar_init(e_full(s), 2 * TC_GROUP_WARPS); mbar_init(e_empty(s), 1); }
        mbar_init(acc_full, 1);
        mbar_init(drain_bar, 1);
        mbar_init(pb_bar, 1);
        *abort_flag = 0;
        *skip_slot = *(volatile int*)&g_tc_status;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async_smem();
    }
    // Both CTAs' barriers exist before anything arrives on them from the other side, and both
    // take the leader's view of the status word, so the pair skips or runs together.
    cluster_sync_all();
    {
        uint32_t skip;
        asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(skip) : "r"(mapa_shared(skip_addr, 0)) : "memory");
        if (skip != 0) {              // an earlier CTA gave up: do not queue behind it
            cluster_sync_all();       // the leader's shared memory outlives the peer's read
            return;
        }
    }
    if (warp == TC_EXP_WARPS + 1) {      // TMEM allocation: the same warp of both CTAs
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"((uint32_t)__cvta_generic_to_shared((const void*)tmem_slot)), "r"((uint32_t)TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == TC_EXP_WARPS) {
        // ================= TMA producer (per CTA) =================
        if (lane == 0) {
            bool ok = true;
            int32_t issued = 0;
            for (int32_t st = 0; st < nstages && ok; ++st) {
                const int s = st % TP_PSTAGES;
                ok = mbar_wait(p_empty(s), ((st / TP_PSTAGES) & 1) ^ 1, abort_flag, 1);
                if (!ok) break;
                mbar_expect_tx(p_full(s), TP_P_STAGE);
                tma_load_2d(p_ring + s * TP_P_STAGE, &tmA, st * TC_PK, (int32_t)m0, p_full(s));
                tma_load_2d(p_ring + s * TP_P_STAGE + TP_P_A, &tmB, st * TC_PK, (int32_t)(n0 + rank * TP_BNH), p_full(s));
                issued = st + 1;
            }
            if (!ok) {
                const int32_t first = issued > TP_PSTAGES ? issued - TP_PSTAGES : 0;
                for (int32_t st = first; st < issued; ++st) {
                    const uint64_t t0 = tc_globaltimer();
                    while (!mbar_try(p_full(st % TP_PSTAGES), (st / TP_PSTAGES) & 1) &&
                           tc_globaltimer() - t0 < TC_WAIT_NS) {}
                }
            }
        }
    } else if (warp == TC_EXP_WARPS + 1) {
        // ================= MMA issuer (leader CTA only) =================
        if (lane == 0 && rank == 0) {
            bool ok = true;
            for (int32_t i = 0; i < nkb && ok; ++i) {
                const int r = i % TP_ESTAGES;
                ok = mbar_wait(e_full(r), (i / TP_ESTAGES) & 1, abort_flag, 2);
                if (!ok) break;
                tc_fence_after();
                const uint64_t bdesc = tc_smem_desc(e_ring + r * TP_E_STAGE);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    tp_mma_i8_ts(tmem, tmem + (uint32_t)(TC_ACC_COLS + r * TC_A_COLS + 8 * k), bdesc + 2u * k, TP_IDESC,
                                 (i > 0 || k > 0) ? 1u : 0u);
                tp_commit(e_empty(r));
                tp_commit(mapa_shared(e_empty(r), 1));
            }
            if (ok) { tp_commit(acc_full); tp_commit(mapa_shared(acc_full, 1)); }
            tp_commit(drain_bar);
            const uint64_t t0 = tc_globaltimer();
            while (!mbar_try(drain_bar, 0) && tc_globaltimer() - t0 < TC_WAIT_NS) {}
        }
    } else {
        // ================= expanders, then epilogue =================
        const int group = warp / TC_GROUP_WARPS, gwarp = warp % TC_GROUP_WARPS, gtid = tid % (TC_GROUP_WARPS * 32);
        const int erow = gtid >> 1, half = gtid & 1;     // B row erow of this CTA's half, 64-bit half of the k-block
        PairExpanderCtx cx;
        cx.bars = bars; cx.p_ring = p_ring; cx.abort_flag = abort_flag; cx.lane = lane;
        cx.e_full_leader = mapa_shared(e_full(0), 0);
        cx.pc_a = cx.pc_b = 0;
#pragma unroll
        for (int kb = 0; kb < 4; ++kb)       // packed 8 bytes of (row, k-block, half) under SWIZZLE_64B
            cx.lds_off[kb] = (uint32_t)(erow * TC_PK + (((kb ^ (erow >> 1)) & 3) << 4) + half * 8);
#pragma unroll
        for (int c = 0; c < 4; ++c)          // chunk 4*half + c of the 128-byte operand row under SWIZZLE_128B
            cx.sts_addr[c] = e_ring + (uint32_t)(erow * 128 + (((4 * half + c) ^ (erow & 7)) << 4));
        const int arow = (gwarp & 3) * 32 + lane, ahalf = gwarp >> 2;      // own TMEM lane
#pragma unroll
        for (int kb = 0; kb < 4; ++kb)
            cx.a_lds_off[kb] = (uint32_t)(arow * TC_PK + (((kb ^ (arow >> 1)) & 3) << 4) + ahalf * 8);
        cx.a_taddr = tmem + ((uint32_t)((gwarp & 3) * 32) << 16) + (uint32_t)(TC_ACC_COLS + ahalf * 16);
        bool ok = true;
        for (int32_t i0 = 0; i0 < nkb && ok; i0 += 12)
            ok = group == 0 ? tp_expander_steps<0, 0>(cx, i0, nkb, (uint32_t)((i0 / 12) & 1))
                            : tp_expander_steps<1, 0>(cx, i0, nkb, (uint32_t)((i0 / 12) & 1));
        atomicAdd(pa_s + arow, cx.pc_a);
        atomicAdd(pb_s + rank * TP_BNH + erow, cx.pc_b);
        asm volatile("bar.sync 1, %0;" :: "n"(TC_EXP_WARPS * 32) : "memory");
        // hand this CTA's half of pb to the peer: plain remote stores, then one release-arrive
        if (tid < TP_BNH) {
            const uint32_t off = 4u * (rank * TP_BNH + tid);
            asm volatile("st.shared::cluster.u32 [%0], %1;" :: "r"(mapa_shared(pb_addr + off, peer)), "r"(pb_s[rank * TP_BNH + tid]) : "memory");
        }
        asm volatile("bar.sync 1, %0;" :: "n"(TC_EXP_WARPS * 32) : "memory");
        if (tid == 0) mbar_arrive_cluster(mapa_shared(pb_bar, peer));
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait_cl(pb_bar, 0, abort_flag, 6));
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(acc_full, 0, abort_flag, 5));
        if (ok) {
            tc_fence_after();
            const int quarter = warp & 3, cblock = warp >> 2;     // 4 lane quarters x 4 blocks of 64 columns
            const int64_t m = m0 + quarter * 32 + lane;
            const int32_t row_term = klogical - 2 * pa_s[quarter * 32 + lane];
#pragma unroll 1
            for (int cc = 0; cc < 2; ++cc) {
                const int col = cblock * 64 + cc * 32;
                uint32_t v[32];
                tc_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)col, v);
                tc_wait_ld();
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    v[j] = (uint32_t)(row_term - 2 * pb_s[col + j] + 4 * (int32_t)(v[j] >> 7));
                const int64_t n = n0 + col;
                if (!PACK) {
                    if (m < M) {
                        int32_t* dst = C + m * ldc + n;
                        if (n + 32 <= N && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                *reinterpret_cast<int4*>(dst + j) = make_int4((int32_t)v[j], (int32_t)v[j + 1], (int32_t)v[j + 2], (int32_t)v[j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) if (n + j < N) dst[j] = (int32_t)v[j];
                        }
                    }
                } else {
                    uint32_t bits = 0;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (n + j < N) {
                            const float y = __ldg(scale + n + j) * (float)(int32_t)v[j];
                            const bool b = mode == BRUTE_SIGN_GE0 ? (y >= 0.0f) : (y > 0.0f);
                            bits |= (b ? 1u : 0u) << j;
                        }
                    }
                    const int64_t hidx = n >> 5;
                    if (m < M && hidx < halves_per_row) out32[m * halves_per_row + hidx] = bits;
                }
            }
        }
    }
    // Neither CTA may free the pair's tensor memory, or leave while the peer can still write into
    // its shared memory, before both are done.
    tc_fence_before();
    __syncwarp();
    cluster_sync_all();
    if (warp == TC_EXP_WARPS + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"((uint32_t)TC_TMEM_COLS) : "memory");
    }
}

// The pair kernel pays off once there is more than one 128-row block of A to share a B tile.
static bool tc5_pair_accepts(int64_t M, int64_t N) {
    return M > TP_BM && (N + TP_BN - 1) / TP_BN <= 65535 && 2 * ((M + 2 * TP_BM - 1) / (2 * TP_BM)) <= 0x7fffffffll;
}

static int tc5_pair_run(const uint64_t* A, const uint64_t* B, int64_t M, int64_t N, int64_t Kp, int64_t K,
                        int32_t* C, int64_t ldc, const float* scale, uint64_t* out, int mode, bool pack,
                        cudaStream_t st) {
    BB_REQUIRE(tc5_accepts(A, B, M, N, Kp) && tc5_pair_accepts(M, N), BRUTE_ERR_UNSUPPORTED);
    CUtensorMap tmA, tmB;
    BB_REQUIRE(tc5_make_map(&tmA, A, M, Kp * 8, TP_BM) && tc5_make_map(&tmB, B, N, Kp * 8, TP_BNH), BRUTE_ERR_DRIVER);
    static bool attr_set[2] = {false, false};
    const dim3 grid((unsigned)(2 * ((M + 2 * TP_BM - 1) / (2 * TP_BM))), (unsigned)((N + TP_BN - 1) / TP_BN));
    const int32_t nkb = (int32_t)(Kp / 2);
    const int32_t klogical = (int32_t)K;
    if (!pack) {
        if (!attr_set[0]) {
            if (cudaFuncSetAttribute(k_xnor_gemm_tcgen05_pair<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, TP_SMEM) != cudaSuccess)
                return BRUTE_ERR_LAUNCH;
            attr_set[0] = true;
        }
        k_xnor_gemm_tcgen05_pair<false><<<grid, TC_THREADS, TP_SMEM, st>>>(tmA, tmB, M, N, nkb, klogical, C, ldc, nullptr, nullptr, 0, 0);
    } else {
        if (!attr_set[1]) {
            if (cudaFuncSetAttribute(k_xnor_gemm_tcgen05_pair<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, TP_SMEM) != cudaSuccess)
                return BRUTE_ERR_LAUNCH;
            attr_set[1] = true;
        }
        k_xnor_gemm_tcgen05_pair<true><<<grid, TC_THREADS, TP_SMEM, st>>>(tmA, tmB, M, N, nkb, klogical, nullptr, 0, scale,
                                                                         reinterpret_cast<uint32_t*>(out), 2 * ((N + 63) / 64), mode);
    }
    return launch_status();
}

}  // namespace bb
