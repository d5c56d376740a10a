// xnor-popcount GEMM on the 5th-generation tensor cores (tcgen05.mma kind::i8).
//
// sm_100a has no binary tcgen05 kind, so the bits are expanded to unsigned int8 ON CHIP, with
// weights chosen so that the expansion is ONE logic op per 4 bytes and no shift at all:
//   A byte (b, j) = bit << j        : word_j = h & (0x01010101 << j), bits stay where they are;
//   B byte (b, j) = bit << (7 - j)  : the packed word is first bit-reversed inside each byte
//                                     (brev + prmt, once per 32 bits), then word_j = g' & (0x01010101 << (7-j)).
// Every product of two set bits is 2^j * 2^(7-j) = 128, so the int32 accumulator holds
// 128 * popcount(a & b) and, with the row popcounts pa[m], pb[n] that the expanders count on the
// way (pad bits are 0 and count nothing),
//   popcount(a ^ b) = pa + pb - 2*popcount(a & b),   C = K - 2*pa[m] - 2*pb[n] + 4*(acc >> 7),
// exact in int32 for K < 2^24. Only PACKED operands ever cross HBM/L2 (8x less operand traffic
// than an int8 GEMM); the expansion is paid per CTA on chip. The ALU pipe (16 lanes/clk per SM
// quarter) is the scarce unit of the expansion, which is why the op count per byte matters.
//
// Per CTA (one 128 x 256 tile of C; accumulator = TMEM columns [0,256), A ring = columns [256,352)):
//   warp 16      TMA producer: packed A [128 rows x 64 B] and B [256 rows x 64 B] boxes (512 bits
//                of K) into a 3-deep ring, SWIZZLE_64B, cp.async.bulk.tensor + mbarrier complete_tx.
//   warps 0..15  expanders, two groups of 8 warps that alternate k-blocks so that the latency
//                chain of one group (ld.shared, logic ops, stores, fences, arrive) overlaps the
//                other's. Per 128-bit k-block a thread expands one 64-bit half row of A and two of B.
//                A never touches shared memory: the words go from registers into this thread's own
//                TENSOR MEMORY lane (tcgen05.st) and the MMA reads A from TMEM, which takes a third
//                of the stores and of the tensor core's operand reads off the shared-memory pipe.
//                B goes into the canonical K-major SWIZZLE_128B layout (st.shared.v4, 3-deep ring),
//                then fence.proxy.async + mbarrier arrive.
//   warp 17      MMA issuer: 4 x tcgen05.mma (M128 N256 K32, A from TMEM, B from a shared-memory
//                descriptor) per k-block; tcgen05.commit frees the slot; owns the TMEM allocation.
//   warps 0..15  epilogue: tcgen05.ld 32x32b, popcount correction, 128-bit stores (or the fused
//                scale/sign/pack of the binarised MLP).
// The order of the 128 k-positions inside a k-block is permuted by the expansion (byte 4j+i of a
// 32-byte group holds bit 8i+j); A and B share the permutation, which a dot product cannot see.
//
// Every mbarrier wait is bounded (about one second); a wait that gives up sets
// the device status word and an abort flag, the CTA drains its copies, frees
// its TMEM and returns, and CTAs that start later return at once.
#pragma once
#include "tcgen05_common.cuh"

namespace bb {

constexpr int TC_BM = 128, TC_BN = 256;
constexpr int TC_PSTAGES = 3, TC_ESTAGES = 3;
constexpr int TC_PK = 64;                               // packed bytes of K per TMA stage and row
constexpr int TC_KB_PER_STAGE = 4;                      // 128-bit k-blocks per packed stage
constexpr int TC_P_A = TC_BM * TC_PK, TC_P_B = TC_BN * TC_PK;
constexpr int TC_P_STAGE = TC_P_A + TC_P_B;             // 24 KB
constexpr int TC_E_STAGE = TC_BN * 128;                 // expanded B of one k-block: 32 KB
constexpr int TC_GROUP_WARPS = 8;                       // warps that expand one k-block together
constexpr int TC_GROUPS = 2;                            // groups alternate k-blocks, so their latency chains overlap
constexpr int TC_EXP_WARPS = TC_GROUP_WARPS * TC_GROUPS;
constexpr int TC_THREADS = (TC_EXP_WARPS + 2) * 32;     // 576
constexpr int TC_A_COLS = 32;                           // A of one k-block: 128 int8 of K per row = 32 columns of 32 bits
constexpr int TC_ACC_COLS = 256;
constexpr int TC_TMEM_COLS = 512;                       // power of two >= 256 + 3 * 32
constexpr int TC_ROWPOP_BYTES = (TC_BM + 2 * TC_BN) * 4;  // pa[128], pb[256], column signs[256] of the tile
constexpr int TC_SMEM = TC_ESTAGES * TC_E_STAGE + TC_PSTAGES * TC_P_STAGE + 256 + TC_ROWPOP_BYTES + 1024;
// kind::i8, D = s32, A = B = unsigned int8 (format 0), both K-major, M = 128, N = 256
constexpr uint32_t TC_IDESC = (2u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(TC_BN >> 3) << 17) |
                              ((uint32_t)(TC_BM >> 4) << 24);

// 4 bits of h (bits j, 8+j, 16+j, 24+j) -> 4 bytes. A side: the bit stays at position j of its
// byte. B side (h already bit-reversed inside each byte): original bit j sits at position 7-j.
template <bool IS_B>
__device__ __forceinline__ uint32_t tc_expand4(uint32_t h, int j) {
    return h & (0x01010101u << (IS_B ? 7 - j : j));
}
// reverse the bit order inside each byte of a packed word (B operand, once per 32 bits)
__device__ __forceinline__ uint32_t tc_brev_bytes(uint32_t g) { return __byte_perm(__brev(g), 0u, 0x0123u); }

// 64 bits of a B row (one half of a 128-bit k-block) -> 64 int8 into the 4 chunks (16 bytes each)
// of the 128-byte operand row that this half owns. dst[c] is the shared address of chunk c
// (swizzle applied), IMM a constant offset (ring slot, +128 rows).
template <int IMM>
__device__ __forceinline__ void tc_expand_b_half(uint2 bits, const uint32_t (&dst)[4]) {
    const uint32_t h[2] = {tc_brev_bytes(bits.x), tc_brev_bytes(bits.y)};
#pragma unroll
    for (int q = 0; q < 2; ++q) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
            sts128<IMM>(dst[2 * q + c], tc_expand4<true>(h[q], 4 * c + 0), tc_expand4<true>(h[q], 4 * c + 1),
                        tc_expand4<true>(h[q], 4 * c + 2), tc_expand4<true>(h[q], 4 * c + 3));
    }
}
// 64 bits of an A row -> 16 columns of this thread's TMEM lane
__device__ __forceinline__ void tc_expand_a_half(uint2 bits, uint32_t taddr) {
    uint32_t w[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) { w[j] = tc_expand4<false>(bits.x, j); w[8 + j] = tc_expand4<false>(bits.y, j); }
    tc_st16(taddr, w);
}

// One k-block of the expander loop with every ring index a compile-time
// constant: U = k-block index modulo 12 (3 operand slots x 4 k-blocks per
// packed stage), so the only run-time state is the parity bit of the packed ring.
struct ExpanderCtx {
    uint32_t bars, p_ring, lds_off[4], sts_addr[4];
    uint32_t a_lds_off[4], a_taddr;      // A: packed-bit offsets and TMEM address of this thread's half row
    int pc_a, pc_b0, pc_b1;              // set bits seen so far in this thread's half rows (for pa[m], pb[n])
    volatile int* abort_flag;
    int lane;
};

// Group G (0 or 1) owns the k-blocks with U % 2 == G; inside a packed stage (4 k-blocks) it reads
// k-blocks G and G + 2, so it waits for the stage before the first and releases it after the second.
template <int G, int U>
__device__ __forceinline__ bool tc_expander_step(ExpanderCtx& cx, uint32_t p_parity) {
    constexpr int S = U / TC_KB_PER_STAGE, KB = U % TC_KB_PER_STAGE, R = U % TC_ESTAGES;
    constexpr uint32_t E_PARITY = ((U / TC_ESTAGES) & 1) ^ 1;
    const uint32_t p_full = cx.bars + 8u * S, p_empty = cx.bars + 8u * (TC_PSTAGES + S);
    const uint32_t e_full = cx.bars + 8u * (2 * TC_PSTAGES + R), e_empty = cx.bars + 8u * (2 * TC_PSTAGES + TC_ESTAGES + R);
    if (KB == G) {
        if (!__all_sync(0xffffffffu, mbar_wait(p_full, p_parity, cx.abort_flag, 3))) return false;
    }
    const uint32_t src = cx.p_ring + cx.lds_off[KB];
    const uint2 a  = lds64<S * TC_P_STAGE>(cx.p_ring + cx.a_lds_off[KB]);
    const uint2 b0 = lds64<S * TC_P_STAGE + TC_P_A>(src);
    const uint2 b1 = lds64<S * TC_P_STAGE + TC_P_A + 128 * TC_PK>(src);
    cx.pc_a  += __popc(a.x) + __popc(a.y);
    cx.pc_b0 += __popc(b0.x) + __popc(b0.y);
    cx.pc_b1 += __popc(b1.x) + __popc(b1.y);
    if (KB == G + 2) {
        // Release the packed slot only AFTER the loaded words have been used: the popcounts above
        // cannot issue before the loads have returned, so the arrive that follows them cannot
        // overtake a load that is still queued behind this kernel's heavy shared-memory store
        // traffic. (Arriving straight after issuing the loads let the next TMA write reach the
        // slot first in about one tile of 10^5.)
        // The packed slot is only ever refilled for a LATER stage, and a stage that short of
        // 4 k-blocks is the last one, so an arrival that a tail skips is never waited for.
        __syncwarp();
        if (cx.lane == 0) mbar_arrive(p_empty);
    }
    if (!__all_sync(0xffffffffu, mbar_wait(e_empty, E_PARITY, cx.abort_flag, 4))) return false;
    tc_fence_after();
    tc_expand_a_half(a, cx.a_taddr + (uint32_t)(R * TC_A_COLS));
    tc_expand_b_half<R * TC_E_STAGE>(b0, cx.sts_addr);
    tc_expand_b_half<R * TC_E_STAGE + 128 * 128>(b1, cx.sts_addr);
    tc_wait_st();
    tc_fence_before();
    fence_proxy_async_smem();
    __syncwarp();
    if (cx.lane == 0) mbar_arrive(e_full);
    return true;
}

template <int G, int U>
__device__ __forceinline__ bool tc_expander_steps(ExpanderCtx& cx, int32_t i0, int32_t nkb, uint32_t p_parity) {
    if constexpr (U < 12) {
        if (i0 + U >= nkb) return true;
        if constexpr ((U & 1) == G) {
            if (!tc_expander_step<G, U>(cx, p_parity)) return false;
        }
        return tc_expander_steps<G, U + 1>(cx, i0, nkb, p_parity);
    } else {
        return true;
    }
}

template <bool PACK>
__global__ void __launch_bounds__(TC_THREADS, 1)
k_xnor_gemm_tcgen05(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    int64_t M, int64_t N, int32_t nkb_all /* 128-bit k-blocks */, int32_t klogical /* K */,
                    int32_t* __restrict__ C, int64_t ldc,
                    const float* __restrict__ scale, uint32_t* __restrict__ out32, int64_t halves_per_row, int mode,
                    int32_t nkb_split /* k-blocks per blockIdx.z (a multiple of 4), or nkb_all */) {
    extern __shared__ uint8_t tc_smem_raw[];
    __shared__ int s_skip;
    if (threadIdx.x == 0) s_skip = *(volatile int*)&g_tc_status;
    __syncthreads();
    if (s_skip != 0) return;                            // an earlier CTA gave up: do not queue behind it

    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(tc_smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gbase = tc_smem_raw + (base - raw);
    const uint32_t e_ring = base;                                    // TC_ESTAGES x 32 KB (expanded B)
    const uint32_t p_ring = base + TC_ESTAGES * TC_E_STAGE;          // TC_PSTAGES x 24 KB
    const uint32_t bars = p_ring + TC_PSTAGES * TC_P_STAGE;
    uint8_t* gp_ring = gbase + TC_ESTAGES * TC_E_STAGE;
    uint8_t* gbars = gp_ring + TC_PSTAGES * TC_P_STAGE;
    // barrier slots (8 bytes each)
    auto p_full  = [&](int s) { return bars + 8u * s; };
    auto p_empty = [&](int s) { return bars + 8u * (TC_PSTAGES + s); };
    auto e_full  = [&](int s) { return bars + 8u * (2 * TC_PSTAGES + s); };
    auto e_empty = [&](int s) { return bars + 8u * (2 * TC_PSTAGES + TC_ESTAGES + s); };
    const uint32_t acc_full = bars + 8u * (2 * TC_PSTAGES + 2 * TC_ESTAGES);
    const uint32_t drain_bar = acc_full + 8u;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbars + 8 * (2 * TC_PSTAGES + 2 * TC_ESTAGES + 2));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbars + 8 * (2 * TC_PSTAGES + 2 * TC_ESTAGES + 2) + 4);

    int* pa_s = reinterpret_cast<int*>(gbars + 256);      // set bits per A row of the tile
    int* pb_s = pa_s + TC_BM;                             // set bits per B row of the tile
    int* cs_s = pb_s + TC_BN;                             // fused epilogue: sign of the column's scale

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);      // a shuffle result: known to the compiler as the same in all lanes
    const int64_t m0 = (int64_t)blockIdx.y * TC_BM, n0 = (int64_t)blockIdx.x * TC_BN;
    // split K (gridDim.z > 1, int32 output only): this CTA contracts k-blocks [kb0, kb0 + nkb) and ADDS its
    // part of C to memory that the launcher has zeroed; integer sums do not depend on the order
    const int32_t kb0 = (int32_t)blockIdx.z * nkb_split;
    const int32_t nkb = nkb_all - kb0 < nkb_split ? nkb_all - kb0 : nkb_split;
    const int32_t nstages = (nkb + TC_KB_PER_STAGE - 1) / TC_KB_PER_STAGE;

    if (tid < TC_BM + TC_BN) pa_s[tid] = 0;
    if (tid == 0) {
        for (int s = 0; s < TC_PSTAGES; ++s) { mbar_init(p_full(s), 1); mbar_init(p_empty(s), TC_EXP_WARPS); }
        for (int s = 0; s < TC_ESTAGES; ++s) { mbar_init(e_full(s), TC_GROUP_WARPS); mbar_init(e_empty(s), 1); }
        mbar_init(acc_full, 1);
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async_smem();
    }
    if (warp == TC_EXP_WARPS + 1) {      // TMEM allocation: one full warp
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"((uint32_t)__cvta_generic_to_shared((const void*)tmem_slot)), "r"((uint32_t)TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == TC_EXP_WARPS) {
        // ================= TMA producer =================
        if (lane == 0) {
            bool ok = true;
            int32_t issued = 0;
            for (int32_t st = 0; st < nstages && ok; ++st) {
                const int s = st % TC_PSTAGES;
                ok = mbar_wait(p_empty(s), ((st / TC_PSTAGES) & 1) ^ 1, abort_flag, 1);
                if (!ok) break;
                mbar_expect_tx(p_full(s), TC_P_STAGE);
                tma_load_2d(p_ring + s * TC_P_STAGE, &tmA, kb0 * 16 + st * TC_PK, (int32_t)m0, p_full(s));
                tma_load_2d(p_ring + s * TC_P_STAGE + TC_P_A, &tmB, kb0 * 16 + st * TC_PK, (int32_t)n0, p_full(s));
                issued = st + 1;
            }
            if (!ok) {
                // drain: wait (bounded) for the copies already issued before the CTA may exit
                const int32_t first = issued > TC_PSTAGES ? issued - TC_PSTAGES : 0;
                for (int32_t st = first; st < issued; ++st) {
                    const uint64_t t0 = tc_globaltimer();
                    while (!mbar_try(p_full(st % TC_PSTAGES), (st / TC_PSTAGES) & 1) &&
                           tc_globaltimer() - t0 < TC_WAIT_NS) {}
                }
            }
        }
    } else if (warp == TC_EXP_WARPS + 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            bool ok = true;
            for (int32_t i = 0; i < nkb && ok; ++i) {
                const int r = i % TC_ESTAGES;
                ok = mbar_wait(e_full(r), (i / TC_ESTAGES) & 1, abort_flag, 2);
                if (!ok) break;
                tc_fence_after();
                const uint64_t bdesc = tc_smem_desc(e_ring + r * TC_E_STAGE);
#pragma unroll
                for (int k = 0; k < 4; ++k)      // 32 bytes of K per instruction: +2 in the encoded address, +8 TMEM columns
                    tc_mma_i8_ts(tmem, tmem + (uint32_t)(TC_ACC_COLS + r * TC_A_COLS + 8 * k), bdesc + 2u * k, TC_IDESC,
                                 (i > 0 || k > 0) ? 1u : 0u);
                tc_commit(e_empty(r));
            }
            if (ok) tc_commit(acc_full);
            // all MMAs issued so far are complete once this commit lands
            tc_commit(drain_bar);
            const uint64_t t0 = tc_globaltimer();
            while (!mbar_try(drain_bar, 0) && tc_globaltimer() - t0 < TC_WAIT_NS) {}
        }
    } else {
        // ================= expanders, then epilogue =================
        const int group = warp / TC_GROUP_WARPS, gwarp = warp % TC_GROUP_WARPS, gtid = tid % (TC_GROUP_WARPS * 32);
        const int erow = gtid >> 1, half = gtid & 1;     // B rows erow and erow + 128 of this group's k-blocks
        ExpanderCtx cx;
        cx.bars = bars; cx.p_ring = p_ring; cx.abort_flag = abort_flag; cx.lane = lane;
        cx.pc_a = cx.pc_b0 = cx.pc_b1 = 0;
#pragma unroll
        for (int kb = 0; kb < 4; ++kb)       // packed 8 bytes of (row, k-block, half) under SWIZZLE_64B
            cx.lds_off[kb] = (uint32_t)(erow * TC_PK + (((kb ^ (erow >> 1)) & 3) << 4) + half * 8);
#pragma unroll
        for (int c = 0; c < 4; ++c)          // chunk 4*half + c of the 128-byte operand row under SWIZZLE_128B
            cx.sts_addr[c] = e_ring + (uint32_t)(erow * 128 + (((4 * half + c) ^ (erow & 7)) << 4));
        // A: a thread can only write its own TMEM lane, 32 * (warp % 4) + lane: it expands that
        // row of A, the half of the k-block given by gwarp / 4
        const int arow = (gwarp & 3) * 32 + lane, ahalf = gwarp >> 2;
#pragma unroll
        for (int kb = 0; kb < 4; ++kb)
            cx.a_lds_off[kb] = (uint32_t)(arow * TC_PK + (((kb ^ (arow >> 1)) & 3) << 4) + ahalf * 8);
        cx.a_taddr = tmem + ((uint32_t)((gwarp & 3) * 32) << 16) + (uint32_t)(TC_ACC_COLS + ahalf * 16);
        bool ok = true;
        for (int32_t i0 = 0; i0 < nkb && ok; i0 += 12)
            ok = group == 0 ? tc_expander_steps<0, 0>(cx, i0, nkb, (uint32_t)((i0 / 12) & 1))
                            : tc_expander_steps<1, 0>(cx, i0, nkb, (uint32_t)((i0 / 12) & 1));
        // row popcounts of the tile: every thread adds what it saw (half rows, alternate k-blocks)
        atomicAdd(pa_s + arow, cx.pc_a);
        atomicAdd(pb_s + erow, cx.pc_b0);
        atomicAdd(pb_s + erow + 128, cx.pc_b1);
        asm volatile("bar.sync 1, %0;" :: "n"(TC_EXP_WARPS * 32) : "memory");     // all expander warps, whatever `ok` is
        if (PACK) {
            // sign(scale * C) in integers: bit = (s * C + off >= 0). Finite scale > 0: s = 1, off = 0
            // for ">= 0" or -1 for "> 0"; scale < 0: s = -1; scale = +-0: s = 0, off = 0 / -1 (the
            // product is +-0); +-inf: off = -1 in both modes (0 * inf is NaN, which compares false);
            // NaN and columns past N: s = 0, off = -1. pb_s becomes u = off - 2 * s * pb.
            if (tid < TC_BN) {
                const int64_t n = n0 + tid;
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
                cs_s[tid] = sg;
                pb_s[tid] = off - 2 * sg * pb_s[tid];
            }
            asm volatile("bar.sync 1, %0;" :: "n"(TC_EXP_WARPS * 32) : "memory");
        }
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(acc_full, 0, abort_flag, 5));
        if (ok) {
            tc_fence_after();
            const int quarter = warp & 3, cblock = warp >> 2;     // 16 warps: 4 lane quarters x 4 blocks of 64 columns
            const int64_t m = m0 + quarter * 32 + lane;
            // C = K - 2*(pa + pb) + 4*popcount(a & b), popcount(a & b) = acc >> 7
            const int32_t row_term = (blockIdx.z == 0 ? klogical : 0) - 2 * pa_s[quarter * 32 + lane];
#pragma unroll 1
            for (int cc = 0; cc < 2; ++cc) {
                const int col = cblock * 64 + cc * 32;
                uint32_t v[32];
                tc_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)col, v);
                tc_wait_ld();
                if (!PACK) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        v[j] = (uint32_t)(row_term - 2 * pb_s[col + j] + 4 * (int32_t)(v[j] >> 7));
                }
                const int64_t n = n0 + col;
                if (!PACK) {
                    if (m < M && gridDim.z > 1) {
                        int32_t* dst = C + m * ldc + n;
#pragma unroll
                        for (int j = 0; j < 32; ++j) if (n + j < N) atomicAdd(dst + j, (int32_t)v[j]);
                    } else if (m < M) {
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
                        const int32_t t = cs_s[col + j] * (row_term + 4 * (int32_t)(v[j] >> 7)) + pb_s[col + j];
                        bits = (bits >> 1) | (~(uint32_t)t & 0x80000000u);
                    }
                    const int64_t hidx = n >> 5;
                    if (m < M && hidx < halves_per_row) out32[m * halves_per_row + hidx] = bits;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == TC_EXP_WARPS + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"((uint32_t)TC_TMEM_COLS) : "memory");
    }
}

// ---- host side -----------------------------------------------------------
// Packed operand [rows, kbytes] as a 2-D byte tensor, box = [box_rows, 64 bytes].
static bool tc5_make_map(CUtensorMap* tm, const void* ptr, int64_t rows, int64_t kbytes, int box_rows) {
    PFN_tmapEncodeTiled enc = tc5_encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)kbytes, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)kbytes};
    const cuuint32_t box[2] = {(cuuint32_t)TC_PK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Shapes the tcgen05 path takes: row pitch a multiple of 16 bytes (TMA global
// stride rule), 16-byte aligned bases, tile counts within the grid limits.
static bool tc5_accepts(const uint64_t* A, const uint64_t* B, int64_t M, int64_t N, int64_t Kp) {
    return Kp > 0 && (Kp % 2) == 0 && aligned16(A) && aligned16(B) && M > 0 && N > 0 &&
           (M + TC_BM - 1) / TC_BM <= 65535 && Kp * 64 < (1ll << 24);   // 128 * K must fit int32
}

static int tc5_run(const uint64_t* A, const uint64_t* B, int64_t M, int64_t N, int64_t Kp, int64_t K,
                   int32_t* C, int64_t ldc, const float* scale, uint64_t* out, int mode, bool pack,
                   cudaStream_t st) {
    BB_REQUIRE(tc5_accepts(A, B, M, N, Kp), BRUTE_ERR_UNSUPPORTED);
    CUtensorMap tmA, tmB;
    BB_REQUIRE(tc5_make_map(&tmA, A, M, Kp * 8, TC_BM) && tc5_make_map(&tmB, B, N, Kp * 8, TC_BN), BRUTE_ERR_DRIVER);
    const dim3 grid((unsigned)((N + TC_BN - 1) / TC_BN), (unsigned)((M + TC_BM - 1) / TC_BM));
    const int32_t nkb = (int32_t)(Kp / 2);
    const int32_t klogical = (int32_t)K;
    if (!pack) {
        if (!kernel_smem_ready<k_xnor_gemm_tcgen05<false>>(TC_SMEM)) return BRUTE_ERR_LAUNCH;
        // A handful of tiles with a long K (small batch against a wide layer) would leave most SMs
        // idle behind one serial k loop per tile: split K over blockIdx.z until the CTAs about fill
        // the GPU, at least 16 k-blocks each, and let the parts add up in the zeroed output. The
        // zeroing and the atomic adds cost about as much as a two-way split saves, so only four-way
        // and wider splits are taken (CUDA-graph replays: 128 x 4096 x 16384 50 -> 30 us,
        // 64 x 1024 x 16384 48 -> 20 us; 1024 x 1024 x 4096 would go from 20 to 29 us two-way).
        const int64_t tiles = (int64_t)grid.x * grid.y;
        int64_t splits = tiles > 0 ? kNumSMs / tiles : 1;
        if (splits > nkb / 16) splits = nkb / 16;
        if (splits > 64) splits = 64;
        if (splits >= 4) {
            int32_t per = (int32_t)((nkb + splits - 1) / splits);
            per = (per + TC_KB_PER_STAGE - 1) / TC_KB_PER_STAGE * TC_KB_PER_STAGE;
            const unsigned gz = (unsigned)((nkb + per - 1) / per);
            if (gz >= 2) {
                if (cudaMemset2DAsync(C, (size_t)ldc * 4, 0, (size_t)N * 4, (size_t)M, st) != cudaSuccess) return BRUTE_ERR_LAUNCH;
                k_xnor_gemm_tcgen05<false><<<dim3(grid.x, grid.y, gz), TC_THREADS, TC_SMEM, st>>>(
                    tmA, tmB, M, N, nkb, klogical, C, ldc, nullptr, nullptr, 0, 0, per);
                return launch_status();
            }
        }
        k_xnor_gemm_tcgen05<false><<<grid, TC_THREADS, TC_SMEM, st>>>(tmA, tmB, M, N, nkb, klogical, C, ldc, nullptr, nullptr, 0, 0, nkb);
    } else {
        if (!kernel_smem_ready<k_xnor_gemm_tcgen05<true>>(TC_SMEM)) return BRUTE_ERR_LAUNCH;
        k_xnor_gemm_tcgen05<true><<<grid, TC_THREADS, TC_SMEM, st>>>(tmA, tmB, M, N, nkb, klogical, nullptr, 0, scale,
                                                                    reinterpret_cast<uint32_t*>(out), 2 * ((N + 63) / 64), mode, nkb);
    }
    return launch_status();
}

}  // namespace bb
