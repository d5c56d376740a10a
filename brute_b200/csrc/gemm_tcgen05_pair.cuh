// xnor-popcount GEMM on tcgen05.mma kind::i8 with cta_group::2: two CTAs of a cluster (two SMs)
// share one 256 x 256 tile of C, and every pair walks over many tiles (persistent kernel).
//
// Same arithmetic as the one-CTA kernel in gemm_tcgen05.cuh (AND-form expansion, weights 2^j and
// 2^(7-j), C = K - 2*pa - 2*pb + 4*(acc >> 7)); what changes is who expands what, and when the
// output leaves. The pair issues ONE M=256 N=256 K=32 instruction per 32 bytes of K from the
// leader CTA (cluster rank 0). Each CTA owns 128 rows of A (its 128 TMEM lanes of the accumulator)
// and supplies HALF of B: rank r expands rows [128 r, 128 r + 128) of the B tile into its own
// shared memory and the tensor cores of both SMs read both halves. Per 128-bit k-block a CTA
// expands 128 + 128 rows instead of 128 + 256: a third less ALU work, half the B stores and half
// the B operand reads on each SM's shared-memory pipe.
//
// Per CTA, 576 threads:
//   warp 16      TMA producer (own A rows, own half of B; no multicast). One packed stage is 64
//                bytes of K (four 128-bit k-blocks) of 128 + 128 rows; 4-deep ring. It runs ahead
//                into the next tile while the others finish the current one.
//   warps 0..15  expanders, two groups of 8 warps. The unit of work is a DOUBLE k-block (256 bits
//                of K): group g takes the g-th half of every packed stage, so that the waits and
//                fences of one publication (tcgen05.wait::st, fence.proxy.async, mbarrier arrive)
//                are paid once per 256 bits and overlap the other group's work. A thread expands
//                128 bits of one A row into 32 columns of its own TMEM lane (tcgen05.st) and 128
//                bits of one B row into one 128-byte row of a K-major SWIZZLE_128B operand tile
//                (8 x st.shared.v4), then arrives on the LEADER's "expanded" barrier (remote
//                mbarrier arrive). 4-deep ring of expanded slots (2 x 16 KB each).
//   warp 17      rank 0: MMA issuer, 8 instructions per slot; its tcgen05.commit is issued twice,
//                once per CTA, so both CTAs' expanders see the slot free. Both ranks: TMEM
//                allocation (cta_group::2), once for the whole kernel.
//   warps 0..15  epilogue of the CTA's own 128 x 256 accumulator half, once per tile: the row
//                popcounts of the other half of B come from the peer through distributed shared
//                memory; tcgen05.ld, correction, and the int32 tile goes to global memory as
//                eight [128 x 32] boxes staged in the (now idle) expanded ring and written by
//                cp.async.bulk.tensor stores: full 128-byte lines, tails clipped by the tensor
//                map. Tensor memory is handed back to the MMA issuer as soon as it has been read,
//                so the next tile's first MMAs overlap the stores.
// Every wait on an mbarrier is bounded (about a second) exactly as in the one-CTA kernel; the only
// unbounded waits are the cluster barriers at entry and exit, which every thread of both CTAs
// reaches on every path, and cp.async.bulk.wait_group on the issuing thread's own stores.
#pragma once
#include "gemm_tcgen05.cuh"

namespace bb {

constexpr int TP_BM = 128;                               // rows of C per CTA (256 per pair)
constexpr int TP_BN = 256;                               // columns of C per pair
constexpr int TP_BNH = TP_BN / 2;                        // rows of B expanded by one CTA
constexpr int TP_PSTAGES = 4;                            // packed stages (4 k-blocks each)
constexpr int TP_ESLOTS = 4;                             // expanded slots (2 k-blocks each)
constexpr int TP_P_A = TP_BM * TC_PK, TP_P_B = TP_BNH * TC_PK;
constexpr int TP_P_STAGE = TP_P_A + TP_P_B;              // 16 KB
constexpr int TP_E_TILE = TP_BNH * 128;                  // expanded half of B of one k-block: 16 KB
constexpr int TP_E_SLOT = 2 * TP_E_TILE;                 // 32 KB
constexpr int TP_A_SLOT_COLS = 2 * TC_A_COLS;            // 64 TMEM columns per slot
constexpr int TP_NBARS = 2 * TP_PSTAGES + 2 * TP_ESLOTS + 4;   // + acc_full, acc_empty, pb, drain
constexpr int TP_ROWPOP_INTS = 2 * 4 * TP_BM + 2 * 4 * TP_BNH + 4 * TP_BN;   // pa parts, pb parts, pb of the pair, column signs
constexpr int TP_SMEM = TP_ESLOTS * TP_E_SLOT + TP_PSTAGES * TP_P_STAGE + 256 + 4 * TP_ROWPOP_INTS + 1024;
static_assert(TC_ACC_COLS + TP_ESLOTS * TP_A_SLOT_COLS <= TC_TMEM_COLS, "A ring must fit beside the accumulator");
static_assert(TP_ESLOTS * TP_E_SLOT == TP_BM * TP_BN * 4, "the expanded ring doubles as the staging area of one C tile");
static_assert(8 * TP_NBARS + 16 <= 256, "barrier block");

// kind::i8, D = s32, A = B = unsigned int8, K-major, M = 256 (128 per CTA), N = 256
constexpr uint32_t TP_IDESC = (2u << 4) | ((uint32_t)(TP_BN >> 3) << 17) | ((uint32_t)((2 * TP_BM) >> 4) << 24);

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
    uint32_t r; asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r)); return r;
}
__device__ __forceinline__ uint32_t cluster_count_x() {
    uint32_t r; asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r)); return r;
}
// shared::cta address of this CTA -> shared::cluster address of the same offset in CTA `rank`
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank)); return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// once per tile: hands plain remote stores (the row popcounts) to the peer
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(cluster_addr) : "memory");
}
// The per-slot signals. A release at cluster scope costs the arriving warp several hundred
// cycles; what the leader's MMA reads was written by st.shared + fence.proxy.async (this SM's
// shared memory) and tcgen05.st + wait::st (this SM's tensor memory), both complete before the
// arrive leaves the SM, so the CTA-scope default is what the loop uses.
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
// bounded wait whose acquire reaches the peer CTA's plain stores
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
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, uint32_t src, int32_t c0, int32_t c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 :: "l"(tm), "r"(src), "r"(c0), "r"(c1) : "memory");
}
// barrier 1 over the 16 expander warps with an OR reduction: every thread gets the same answer
__device__ __forceinline__ bool tp_any_of_expanders(bool pred) {
    uint32_t res;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.or.pred q, 1, %2, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(res) : "r"((uint32_t)pred), "n"(TC_EXP_WARPS * 32) : "memory");
    return res != 0;
}
template <int IMM>
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(IMM) : "memory");
    return v;
}

struct PairExpanderCtx {
    uint32_t bars, e_full_leader;        // e_full_leader: shared::cluster address of the leader's e_full[0]
    uint32_t a_src, b_src;               // packed 16 bytes of this thread's A row / B row in stage 0
    uint32_t a_taddr, b_dst;             // TMEM address (slot 0) / operand row in slot 0, chunk 0 (swizzle folded in)
    uint32_t pf_mask, ee_mask;           // parity the next wait on p_full[s] / e_empty[r] expects, one bit per slot
    int pc_a, pc_b;                      // set bits seen in this thread's A row / B row during the tile
    volatile int* abort_flag;
    int lane;
};

// One packed stage S (0..3) for group G: the stage's G-th double k-block goes to expanded slot
// (2 S + G) % 4. Slot and stage indices are constants; only the parities are run-time state.
template <int G, int S>
__device__ __forceinline__ bool tp_expander_step(PairExpanderCtx& cx) {
    constexpr int R = (2 * S + G) % TP_ESLOTS;
    const uint32_t p_full = cx.bars + 8u * S, p_empty = cx.bars + 8u * (TP_PSTAGES + S);
    const uint32_t e_empty = cx.bars + 8u * (2 * TP_PSTAGES + TP_ESLOTS + R);
    if (!__all_sync(0xffffffffu, mbar_wait(p_full, (cx.pf_mask >> S) & 1u, cx.abort_flag, 3))) return false;
    cx.pf_mask ^= 1u << S;
    const uint4 a = lds128<S * TP_P_STAGE>(cx.a_src);
    const uint4 b = lds128<S * TP_P_STAGE + TP_P_A>(cx.b_src);
    cx.pc_a += __popc(a.x) + __popc(a.y) + __popc(a.z) + __popc(a.w);
    cx.pc_b += __popc(b.x) + __popc(b.y) + __popc(b.z) + __popc(b.w);
    // the slot is released after the first USE of the loaded words, never straight after the loads
    // were issued: see the one-CTA kernel
    __syncwarp();
    if (cx.lane == 0) mbar_arrive(p_empty);
    if (!__all_sync(0xffffffffu, mbar_wait(e_empty, (cx.ee_mask >> R) & 1u, cx.abort_flag, 4))) return false;
    cx.ee_mask ^= 1u << R;
    tc_fence_after();
    tc_expand_a_half(make_uint2(a.x, a.y), cx.a_taddr + (uint32_t)(R * TP_A_SLOT_COLS));
    tc_expand_a_half(make_uint2(a.z, a.w), cx.a_taddr + (uint32_t)(R * TP_A_SLOT_COLS + 16));
    {
        const uint32_t h[4] = {tc_brev_bytes(b.x), tc_brev_bytes(b.y), tc_brev_bytes(b.z), tc_brev_bytes(b.w)};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int c = 0; c < 2; ++c)      // chunk 2q + c of the row; the swizzle is an XOR on address bits 4..6
                sts128<R * TP_E_SLOT>(cx.b_dst ^ (uint32_t)((2 * q + c) << 4),
                                      tc_expand4<true>(h[q], 4 * c + 0), tc_expand4<true>(h[q], 4 * c + 1),
                                      tc_expand4<true>(h[q], 4 * c + 2), tc_expand4<true>(h[q], 4 * c + 3));
        }
    }
    tc_wait_st();
    tc_fence_before();
    fence_proxy_async_smem();
    __syncwarp();
    if (cx.lane == 0) mbar_arrive_remote(cx.e_full_leader + 8u * R);
    return true;
}

template <int G>
__device__ __forceinline__ bool tp_expand_tile(PairExpanderCtx& cx, int32_t nst) {
    for (int32_t s0 = 0; s0 < nst; s0 += 4) {
        if (!tp_expander_step<G, 0>(cx)) return false;
        if (s0 + 1 >= nst) break;
        if (!tp_expander_step<G, 1>(cx)) return false;
        if (s0 + 2 >= nst) break;
        if (!tp_expander_step<G, 2>(cx)) return false;
        if (s0 + 3 >= nst) break;
        if (!tp_expander_step<G, 3>(cx)) return false;
    }
    return true;
}

// STORE: 3 = int16 C by plain stores (`C` then points at int16 values, ldc counts them), for the exchange
// of a column-sharded result between GPUs; 0 = int32 C through TMA stores (C 16-byte aligned, ldc a multiple of 4), 1 = int32 C by
// plain stores from registers, 2 = fused scale/sign/pack (binarised MLP layer).
template <int STORE>
__global__ void __launch_bounds__(TC_THREADS, 1)
k_xnor_gemm_tcgen05_pair(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmC,
                         int64_t M, int64_t N, int32_t nkb /* 128-bit k-blocks */, int32_t klogical /* K */,
                         int32_t tiles_m, int32_t ntiles,
                         int32_t* __restrict__ C, int64_t ldc,
                         const float* __restrict__ scale, uint32_t* __restrict__ out32, int64_t halves_per_row, int mode) {
    extern __shared__ uint8_t tc_smem_raw[];
    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(tc_smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gbase = tc_smem_raw + (base - raw);
    const uint32_t e_ring = base;                                    // TP_ESLOTS x 32 KB; staging of the C tile in the epilogue
    const uint32_t p_ring = base + TP_ESLOTS * TP_E_SLOT;            // TP_PSTAGES x 16 KB
    const uint32_t bars = p_ring + TP_PSTAGES * TP_P_STAGE;
    uint8_t* gbars = gbase + TP_ESLOTS * TP_E_SLOT + TP_PSTAGES * TP_P_STAGE;
    auto p_full  = [&](int s) { return bars + 8u * s; };
    auto p_empty = [&](int s) { return bars + 8u * (TP_PSTAGES + s); };
    auto e_full  = [&](int s) { return bars + 8u * (2 * TP_PSTAGES + s); };
    auto e_empty = [&](int s) { return bars + 8u * (2 * TP_PSTAGES + TP_ESLOTS + s); };
    constexpr int NB = 2 * TP_PSTAGES + 2 * TP_ESLOTS;
    const uint32_t acc_full = bars + 8u * NB;          // per CTA: the tile's MMAs are complete
    const uint32_t acc_empty = acc_full + 8u;          // leader's copy: both CTAs have read their accumulator half
    const uint32_t pb_bar = acc_full + 16u;            // per CTA: the peer's half of pb has arrived
    const uint32_t drain_bar = acc_full + 24u;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbars + 8 * TP_NBARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbars + 8 * TP_NBARS + 4);
    volatile int* skip_slot = reinterpret_cast<volatile int*>(gbars + 8 * TP_NBARS + 8);
    const uint32_t skip_addr = bars + 8u * TP_NBARS + 8u;

    // row popcounts, double buffered by tile parity: partial sums of the 4 threads that share a row
    int* pa_part = reinterpret_cast<int*>(gbars + 256);              // [2][4][128]
    int* pb_part = pa_part + 2 * 4 * TP_BM;                          // [2][4][128] (this CTA's half of B)
    int* pb_pair = pb_part + 2 * 4 * TP_BNH;                         // [2][256]
    int* col_s = pb_pair + 2 * TP_BN;                                // [2][256] (fused epilogue only)
    const uint32_t pb_pair_addr = bars + 256u + 4u * (2 * 4 * TP_BM + 2 * 4 * TP_BNH);

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);      // a shuffle result: known to the compiler as the same in all lanes
    const uint32_t rank = cluster_ctarank(), peer = rank ^ 1u;
    const int32_t pair_id = (int32_t)cluster_id_x(), npairs = (int32_t)cluster_count_x();
    const int32_t nst = (nkb + TC_KB_PER_STAGE - 1) / TC_KB_PER_STAGE;     // packed stages per tile; K tails are zero filled
    const int32_t ndbl = 2 * nst;

    if (tid == 0) {
        for (int s = 0; s < TP_PSTAGES; ++s) { mbar_init(p_full(s), 1); mbar_init(p_empty(s), TC_EXP_WARPS); }
        // "expanded" counts the warps of one group in BOTH CTAs (only the leader's copy is used)
        for (int s = 0; s < TP_ESLOTS; ++s) { mbar_init(e_full(s), 2 * TC_GROUP_WARPS); mbar_init(e_empty(s), 1); }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 2 * TC_EXP_WARPS);
        mbar_init(pb_bar, 1);
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        *skip_slot = *(volatile int*)&g_tc_status;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async_smem();
    }
    // Both CTAs' barriers exist before anything arrives on them from the other side, and both
    // take the leader's view of the status word, so the pair skips or runs together.
    __syncwarp();
    cluster_sync_all();
    {
        uint32_t skip;
        asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(skip) : "r"(mapa_shared(skip_addr, 0)) : "memory");
        if (skip != 0) {              // an earlier launch or CTA gave up: do not queue behind it
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
            uint32_t pe_mask = (1u << TP_PSTAGES) - 1u;      // a fresh barrier passes a wait on parity 1
            for (int32_t t = pair_id; t < ntiles && ok; t += npairs) {
                const int32_t m0 = ((t % tiles_m) * 2 + (int32_t)rank) * TP_BM;
                const int32_t nb = (t / tiles_m) * TP_BN + (int32_t)rank * TP_BNH;
                for (int32_t st = 0; st < nst; ++st) {
                    const int s = st % TP_PSTAGES;
                    ok = mbar_wait(p_empty(s), (pe_mask >> s) & 1u, abort_flag, 1);
                    if (!ok) break;
                    pe_mask ^= 1u << s;
                    mbar_expect_tx(p_full(s), TP_P_STAGE);
                    tma_load_2d(p_ring + s * TP_P_STAGE, &tmA, st * TC_PK, m0, p_full(s));
                    tma_load_2d(p_ring + s * TP_P_STAGE + TP_P_A, &tmB, st * TC_PK, nb, p_full(s));
                }
            }
            if (!ok) {
                // a copy may still be in flight: give it time to land before the CTA's shared
                // memory can go away (the exit barrier of the cluster comes after)
                const uint64_t t0 = tc_globaltimer();
                while (tc_globaltimer() - t0 < TC_WAIT_NS / 100) {}
            }
        }
    } else if (warp == TC_EXP_WARPS + 1) {
        // ================= MMA issuer (leader CTA only) =================
        if (lane == 0 && rank == 0) {
            bool ok = true;
            uint32_t ef_mask = 0u, it = 0u;
            for (int32_t t = pair_id; t < ntiles && ok; t += npairs, ++it) {
                if (it > 0) {        // both CTAs have read the previous tile out of tensor memory
                    ok = mbar_wait(acc_empty, (it - 1u) & 1u, abort_flag, 7);
                    if (!ok) break;
                    tc_fence_after();
                }
                for (int32_t d = 0; d < ndbl && ok; ++d) {
                    const int r = d % TP_ESLOTS;
                    ok = mbar_wait(e_full(r), (ef_mask >> r) & 1u, abort_flag, 2);
                    if (!ok) break;
                    ef_mask ^= 1u << r;
                    tc_fence_after();
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint64_t bdesc = tc_smem_desc(e_ring + r * TP_E_SLOT + h * TP_E_TILE);
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            tp_mma_i8_ts(tmem, tmem + (uint32_t)(TC_ACC_COLS + r * TP_A_SLOT_COLS + h * TC_A_COLS + 8 * k),
                                         bdesc + 2u * k, TP_IDESC, (d > 0 || h > 0 || k > 0) ? 1u : 0u);
                    }
                    tp_commit(e_empty(r));
                    tp_commit(mapa_shared(e_empty(r), 1));
                }
                if (ok) { tp_commit(acc_full); tp_commit(mapa_shared(acc_full, 1)); }
            }
            tp_commit(drain_bar);
            const uint64_t t0 = tc_globaltimer();
            while (!mbar_try(drain_bar, 0) && tc_globaltimer() - t0 < TC_WAIT_NS) {}
        }
    } else {
        // ================= expanders, then epilogue, tile after tile =================
        const int group = warp / TC_GROUP_WARPS, gwarp = warp % TC_GROUP_WARPS, gtid = tid % (TC_GROUP_WARPS * 32);
        // A: own TMEM lane; the warp's position in the group picks the k-block of the double
        const int arow = (gwarp & 3) * 32 + lane, at = gwarp >> 2;
        // B: one row per thread, all lanes of a warp in the same k-block (conflict-free stores)
        const int erow = gtid & (TP_BNH - 1), bt = gtid >> 7;
        PairExpanderCtx cx;
        cx.bars = bars; cx.abort_flag = abort_flag; cx.lane = lane;
        cx.e_full_leader = mapa_shared(e_full(0), 0);
        cx.pf_mask = 0u; cx.ee_mask = (1u << TP_ESLOTS) - 1u;
        // packed 16 bytes of (row, k-block 2*group + t) under SWIZZLE_64B
        cx.a_src = p_ring + (uint32_t)(arow * TC_PK + ((((2 * group + at) ^ (arow >> 1)) & 3) << 4));
        cx.b_src = p_ring + (uint32_t)(erow * TC_PK + ((((2 * group + bt) ^ (erow >> 1)) & 3) << 4));
        cx.a_taddr = tmem + ((uint32_t)((gwarp & 3) * 32) << 16) + (uint32_t)(TC_ACC_COLS + at * TC_A_COLS);
        cx.b_dst = e_ring + (uint32_t)(bt * TP_E_TILE + erow * 128 + ((erow & 7) << 4));
        const int quarter = warp & 3, cblock = warp >> 2;     // epilogue: 4 lane quarters x 4 blocks of 64 columns
        const int prow = quarter * 32 + lane;
        const uint32_t acc_empty_leader = mapa_shared(acc_empty, 0);
        bool ok = true;
        uint32_t it = 0u;
        for (int32_t t = pair_id; t < ntiles && ok; t += npairs, ++it) {
            const uint32_t par = it & 1u;
            const int64_t m0 = (int64_t)((t % tiles_m) * 2 + (int32_t)rank) * TP_BM;
            const int64_t n0 = (int64_t)(t / tiles_m) * TP_BN;
            cx.pc_a = cx.pc_b = 0;
            ok = group == 0 ? tp_expand_tile<0>(cx, nst) : tp_expand_tile<1>(cx, nst);
            // ---- row popcounts of the tile: 4 threads share a row (2 groups x 2 k-blocks of the double)
            pa_part[(par * 4 + group * 2 + at) * TP_BM + arow] = cx.pc_a;
            pb_part[(par * 4 + group * 2 + bt) * TP_BNH + erow] = cx.pc_b;
            asm volatile("bar.sync 1, %0;" :: "n"(TC_EXP_WARPS * 32) : "memory");
            if (tid < TP_BNH) {
                const int* pp = pb_part + par * 4 * TP_BNH + tid;
                const uint32_t idx = par * TP_BN + rank * TP_BNH + (uint32_t)tid;
                int v = pp[0] + pp[TP_BNH] + pp[2 * TP_BNH] + pp[3 * TP_BNH];
                if (STORE == 2) {
                    // sign(scale * C) without a float per element: bit = (s * C + off >= 0), with
                    //   finite scale > 0: s = 1,  off = 0 (>= 0) or -1 (> 0);   scale < 0: s = -1, same off
                    //   scale = +-0: the product is +-0: s = 0, off = 0 (>= 0 holds) or -1 (> 0 does not)
                    //   scale = +-inf: 0 * inf is NaN, which compares false: s = +-1, off = -1 in both modes
                    //   NaN, and columns past N: s = 0, off = -1 (bit 0)
                    // The column's popcount goes into the offset: u = off - 2 * s * pb.
                    const int64_t n = n0 + (int64_t)rank * TP_BNH + tid;
                    int sg = 0, off = -1;
                    if (n < N) {
                        const float sc = __ldg(scale + n);
                        const bool ge0 = mode == BRUTE_SIGN_GE0;
                        if (sc == 0.0f) off = ge0 ? 0 : -1;
                        else if (sc > 0.0f || sc < 0.0f) {
                            sg = sc > 0.0f ? 1 : -1;
                            off = (ge0 && fabsf(sc) <= 3.402823466e38f) ? 0 : -1;
                        }
                    }
                    asm volatile("st.shared::cluster.u32 [%0], %1;" :: "r"(mapa_shared(pb_pair_addr + 4u * (2 * TP_BN + idx), peer)), "r"(sg) : "memory");
                    col_s[idx] = sg;
                    v = off - 2 * sg * v;
                }
                pb_pair[idx] = v;
                asm volatile("st.shared::cluster.u32 [%0], %1;" :: "r"(mapa_shared(pb_pair_addr + 4u * idx, peer)), "r"(v) : "memory");
            }
            asm volatile("bar.sync 1, %0;" :: "n"(TC_EXP_WARPS * 32) : "memory");
            if (tid == 0) mbar_arrive_cluster(mapa_shared(pb_bar, peer));
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait_cl(pb_bar, par, abort_flag, 6));
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(acc_full, par, abort_flag, 5));
            // one verdict for all 16 warps: the epilogue has barriers that every one of them must reach
            if (tp_any_of_expanders(!ok || *abort_flag != 0)) { ok = false; break; }
            tc_fence_after();
            const int* pap = pa_part + par * 4 * TP_BM + prow;
            const int32_t row_term = klogical - 2 * (pap[0] + pap[TP_BM] + pap[2 * TP_BM] + pap[3 * TP_BM]);
            const int* pbp = pb_pair + par * TP_BN;
            const int64_t m = m0 + prow;
#pragma unroll 1
            for (int cc = 0; cc < 2; ++cc) {
                const int col = cblock * 64 + cc * 32;
                uint32_t v[32];
                tc_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)col, v);
                tc_wait_ld();
                if (cc == 1) {       // this warp's part of the accumulator is in registers: hand it back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_remote(acc_empty_leader);
                }
                if (STORE != 2) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        v[j] = (uint32_t)(row_term - 2 * pbp[col + j] + 4 * (int32_t)(v[j] >> 7));
                }
                const int64_t n = n0 + col;
                if (STORE == 0) {
                    // box (2*cblock + cc): [128 rows][32 ints], 128-byte rows, 16-byte chunks XOR (row & 7)
                    const uint32_t rowaddr = e_ring + (uint32_t)((2 * cblock + cc) * (TP_BM * 128) + prow * 128);
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        sts128<0>(rowaddr + (uint32_t)((c ^ (prow & 7)) << 4), v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
                } else if (STORE == 1) {
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
                } else if (STORE == 3) {
                    // int16 C (exact for K <= 32767), straight from registers: a row's 32 values are 64 bytes
                    if (m < M) {
                        int16_t* dst = reinterpret_cast<int16_t*>(C) + m * ldc + n;
                        if (n + 32 <= N && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8)
                                *reinterpret_cast<uint4*>(dst + j) =
                                    make_uint4((v[j] & 0xFFFFu) | (v[j + 1] << 16), (v[j + 2] & 0xFFFFu) | (v[j + 3] << 16),
                                               (v[j + 4] & 0xFFFFu) | (v[j + 5] << 16), (v[j + 6] & 0xFFFFu) | (v[j + 7] << 16));
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) if (n + j < N) dst[j] = (int16_t)(int32_t)v[j];
                        }
                    }
                } else {
                    // bit j = (s_j * C + off_j >= 0), C = row_term - 2 pb_j + 4 a: integer only
                    const int* csp = col_s + par * TP_BN + col;
                    uint32_t bits = 0;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int32_t t = csp[j] * (row_term + 4 * (int32_t)(v[j] >> 7)) + pbp[col + j];
                        bits = (bits >> 1) | (~(uint32_t)t & 0x80000000u);
                    }
                    // [128 rows][8 words] of this CTA's 256 columns: a row is one 32-byte sector
                    reinterpret_cast<uint32_t*>(gbase)[prow * 8 + 2 * cblock + cc] = bits;
                }
            }
            if (STORE == 2) {
                asm volatile("bar.sync 1, %0;" :: "n"(TC_EXP_WARPS * 32) : "memory");
                if (tid < 2 * TP_BM) {
                    const int r = tid >> 1, h = tid & 1;
                    const int64_t mr = m0 + r, w0 = (n0 >> 5) + 4 * h;        // first of this thread's 4 words
                    if (mr < M && w0 < halves_per_row) {
                        const uint4 q = reinterpret_cast<const uint4*>(gbase)[tid];
                        uint32_t* dst = out32 + mr * halves_per_row + w0;
                        if (w0 + 4 <= halves_per_row && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
                            *reinterpret_cast<uint4*>(dst) = q;
                        } else {
                            const uint32_t qq[4] = {q.x, q.y, q.z, q.w};
                            for (int i = 0; i < 4 && w0 + i < halves_per_row; ++i) dst[i] = qq[i];
                        }
                    }
                }
                // the staging words are rewritten by the next tile's epilogue, after its own barriers
                asm volatile("bar.sync 1, %0;" :: "n"(TC_EXP_WARPS * 32) : "memory");
            }
            if (STORE == 0) {
                // staged tile -> global: one box per warp 0..7, issued once every warp has written
                fence_proxy_async_smem();
                asm volatile("bar.sync 1, %0;" :: "n"(TC_EXP_WARPS * 32) : "memory");
                if (warp < 8 && lane == 0) {
                    const int64_t nbx = n0 + warp * 32;
                    if (m0 < M && nbx < N) tma_store_2d(&tmC, e_ring + (uint32_t)(warp * (TP_BM * 128)), (int32_t)nbx, (int32_t)m0);
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    // the ring is refilled by the next tile: wait until the stores have read it
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                }
                asm volatile("bar.sync 1, %0;" :: "n"(TC_EXP_WARPS * 32) : "memory");
            }
        }
        if (STORE == 0 && warp < 8 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
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

// ---- host side -----------------------------------------------------------
// int32 C [M, ldc] as a 2-D tensor of [128 x 32] boxes, SWIZZLE_128B (128-byte box rows)
static bool tc5_make_c_map(CUtensorMap* tm, const int32_t* C, int64_t M, int64_t N, int64_t ldc) {
    PFN_tmapEncodeTiled enc = tc5_encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)ldc * 4u};
    const cuuint32_t box[2] = {32u, (cuuint32_t)TP_BM};
    const cuuint32_t estr[2] = {1, 1};
    return enc(tm, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<int32_t*>(C), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The pair kernel pays off once there is more than one 128-row block of A to share a B tile.
static bool tc5_pair_accepts(int64_t M, int64_t N) {
    const int64_t tiles = ((M + 2 * TP_BM - 1) / (2 * TP_BM)) * ((N + TP_BN - 1) / TP_BN);
    return M > TP_BM && tiles < (1ll << 30) && M < (1ll << 31) - 2 * TP_BM && N < (1ll << 31) - TP_BN;
}

// AUTO takes the pair kernel once its 256 x 256 tiles can occupy most of the SM pairs; below
// that the one-CTA kernel's 128 x 256 tiles spread a small problem over twice as many SMs.
static bool tc5_pair_prefers(int64_t M, int64_t N) {
    const int64_t tiles = ((M + 2 * TP_BM - 1) / (2 * TP_BM)) * ((N + TP_BN - 1) / TP_BN);
    return tc5_pair_accepts(M, N) && tiles >= 48;
}

template <int STORE>
static int tc5_pair_launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                           int64_t M, int64_t N, int32_t nkb, int32_t klogical, int32_t tiles_m, int32_t ntiles,
                           int32_t* C, int64_t ldc, const float* scale, uint32_t* out32, int64_t halves_per_row, int mode,
                           cudaStream_t st, int leave_sms = 0) {
    static int max_pairs_dev[64] = {0};     // per device: pairs of SMs that can hold this kernel at once
    auto kern = k_xnor_gemm_tcgen05_pair<STORE>;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BRUTE_ERR_LAUNCH;
    int& max_pairs = max_pairs_dev[dev];
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(TC_THREADS); cfg.dynamicSmemBytes = TP_SMEM; cfg.stream = st; cfg.attrs = attr; cfg.numAttrs = 1;
    if (max_pairs == 0) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TP_SMEM) != cudaSuccess) return BRUTE_ERR_LAUNCH;
        int sms = 0, n = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return BRUTE_ERR_LAUNCH;
        cfg.gridDim = dim3((unsigned)(2 * (sms / 2)));
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = sms / 2; }
        max_pairs = n < sms / 2 ? n : sms / 2;
    }
    // leave_sms: SMs that the caller wants free for kernels of other streams (a collective that runs
    // under this GEMM); the persistent grid walks the same tiles with fewer CTA pairs
    int cap = max_pairs - (leave_sms + 1) / 2;
    if (cap < 1) cap = 1;
    const int pairs = ntiles < cap ? ntiles : cap;
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    if (cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, M, N, nkb, klogical, tiles_m, ntiles, C, ldc, scale, out32,
                           halves_per_row, mode) != cudaSuccess)
        return BRUTE_ERR_LAUNCH;
    return launch_status();
}

static int tc5_pair_run(const uint64_t* A, const uint64_t* B, int64_t M, int64_t N, int64_t Kp, int64_t K,
                        int32_t* C, int64_t ldc, const float* scale, uint64_t* out, int mode, bool pack,
                        cudaStream_t st, int leave_sms = 0) {
    BB_REQUIRE(tc5_accepts(A, B, M, N, Kp) && tc5_pair_accepts(M, N), BRUTE_ERR_UNSUPPORTED);
    CUtensorMap tmA, tmB, tmC;
    BB_REQUIRE(tc5_make_map(&tmA, A, M, Kp * 8, TP_BM) && tc5_make_map(&tmB, B, N, Kp * 8, TP_BNH), BRUTE_ERR_DRIVER);
    const int32_t tiles_m = (int32_t)((M + 2 * TP_BM - 1) / (2 * TP_BM));
    const int32_t ntiles = tiles_m * (int32_t)((N + TP_BN - 1) / TP_BN);
    const int32_t nkb = (int32_t)(Kp / 2);
    if (pack) {
        tmC = tmA;      // not used by this variant
        return tc5_pair_launch<2>(tmA, tmB, tmC, M, N, nkb, (int32_t)K, tiles_m, ntiles, nullptr, 0, scale,
                                  reinterpret_cast<uint32_t*>(out), 2 * ((N + 63) / 64), mode, st);
    }
    if (aligned16(C) && (ldc % 4) == 0 && tc5_make_c_map(&tmC, C, M, N, ldc))
        return tc5_pair_launch<0>(tmA, tmB, tmC, M, N, nkb, (int32_t)K, tiles_m, ntiles, C, ldc, nullptr, nullptr, 0, 0, st, leave_sms);
    tmC = tmA;
    return tc5_pair_launch<1>(tmA, tmB, tmC, M, N, nkb, (int32_t)K, tiles_m, ntiles, C, ldc, nullptr, nullptr, 0, 0, st, leave_sms);
}

// C as int16 [M, ldc]: the transport form of a column-sharded result (|C| <= K <= 32767)
static int tc5_pair_run_i16(const uint64_t* A, const uint64_t* B, int64_t M, int64_t N, int64_t Kp, int64_t K,
                            int16_t* C, int64_t ldc, cudaStream_t st, int leave_sms) {
    BB_REQUIRE(K <= 32767 && tc5_accepts(A, B, M, N, Kp) && tc5_pair_accepts(M, N), BRUTE_ERR_UNSUPPORTED);
    CUtensorMap tmA, tmB;
    BB_REQUIRE(tc5_make_map(&tmA, A, M, Kp * 8, TP_BM) && tc5_make_map(&tmB, B, N, Kp * 8, TP_BNH), BRUTE_ERR_DRIVER);
    const int32_t tiles_m = (int32_t)((M + 2 * TP_BM - 1) / (2 * TP_BM));
    const int32_t ntiles = tiles_m * (int32_t)((N + TP_BN - 1) / TP_BN);
    return tc5_pair_launch<3>(tmA, tmB, tmA /* unused */, M, N, (int32_t)(Kp / 2), (int32_t)K, tiles_m, ntiles,
                              reinterpret_cast<int32_t*>(C), ldc, nullptr, nullptr, 0, 0, st, leave_sms);
}

}  // namespace bb
