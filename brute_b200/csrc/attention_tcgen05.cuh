// Fused binary attention forward on the 5th-generation tensor cores (D = 128 or 64; the text
// below gives the figures for 128).
//
// Both contractions run on tcgen05.mma with accumulators in tensor memory:
//   S = Q.K^T   kind::i8, M128 N64 K32 x 4. Q (+1/-1) is expanded once per CTA and the K tile
//               (64 keys, -2/+2) once per tile from packed bits to int8 in shared memory, both
//               K-major SWIZZLE_128B. The accumulator is 4*h - 2*D for Hamming distance h, i.e.
//               the byte offset of T[h] from the middle of the float table.
//   O += P.V    kind::f16 (bf16), M128 N128 K16 x 4. P is the A operand, read from TMEM; V arrives by
//               TMA as two [64 keys x 64 d] SWIZZLE_128B boxes and is the B operand in MN-major
//               form, so the row-major V of the caller needs no transpose.
// S is double buffered in tensor memory and P is written over the S it came from (a thread's bf16
// weights go into the first half of the columns it just read), so the score MMA of tile j+2 is
// issued right behind the P.V MMA of tile j: the tensor pipe executes in order, which is all the
// buffer reuse needs, and the round trip softmax -> MMA issuer -> tcgen05.commit -> softmax is off
// the softmax threads' critical path.
// Softmax is the table form: P = T[h] (bf16-exact entries, T <= 1), no running maximum, no exp and
// no rescaling of O, so O simply accumulates in TMEM over all key tiles and is divided by the row
// sum at the end. Two threads own one query row = one TMEM lane (32 of the tile's 64 keys each):
// a thread reads its 32 scores with tcgen05.ld, looks them up, adds them to its part of the row
// sum, packs bf16 pairs and writes them back with tcgen05.st. Rounding matches the mma.sync kernels: the row sum adds exactly the bf16 weights that
// enter P.V.
//
// CTA = 128 query rows of one (batch, head); 384 threads; 256 TMEM columns (S/P 2 x 64, O 128),
// so two CTAs share an SM.
//   warp 0      TMA producer for V (4-deep ring).
//   warp 1      MMA issuer (convergent, one elected lane), TMEM owner; waits on p_full only: softmax
//               warps 4 and 5 check v_full / ke_full on its behalf before they arrive.
//   warps 2-3   K expanders (int8 tiles, three in flight; packed words prefetched four tiles ahead).
//   warps 4-11  softmax, then the epilogue (tcgen05.ld of O, 1/l, bf16, 16-byte stores): warps w and
//               w + 4 share a TMEM lane quarter and split the key (then the output) columns.
// Every mbarrier wait is bounded; a wait that gives up raises the CTA's abort flag and the device
// status word, and all roles fall through to the common exit where the TMEM is freed.
#pragma once
#include "tcgen05_common.cuh"

namespace bb {

constexpr int AX_BM = 128, AX_BN = 64, AX_DMAX = 128, AX_THREADS = 384;
constexpr int AX_SOFTMAX_WARPS = 8;
constexpr int AX_NV = 4;                                   // V stages (a power of two)
constexpr int AX_V_HALF = AX_BN * 128;                     // [64 keys][64 d] bf16 = 8 KB
constexpr int AX_V_STAGE = 2 * AX_V_HALF;                  // 16 KB
constexpr int AX_KE_TILE = AX_BN * AX_DMAX;                // int8 [64 keys][128-byte rows] = 8 KB
constexpr int AX_NK = 3;                                   // expanded K tiles in flight
constexpr int AX_COL_S = 0 /* two buffers of 64 */, AX_COL_O = 128, AX_TMEM_COLS = 256;
constexpr int AX_Q_TILE = AX_BM * AX_DMAX;                 // int8 [128 rows][128-byte rows] = 16 KB
constexpr int AX_OFF_KE = AX_NV * AX_V_STAGE;              // 64 KB
constexpr int AX_OFF_Q = AX_OFF_KE + AX_NK * AX_KE_TILE;   // 88 KB
constexpr int AX_OFF_L = AX_OFF_Q + AX_Q_TILE;             // 104 KB: row-sum parts [2][128] floats
constexpr int AX_OFF_BARS = AX_OFF_L + 1024;
constexpr int AX_SMEM = AX_OFF_BARS + 256 + 1024;          // + alignment slack

// kind::i8: D s32, A and B signed int8, K-major both, M 128, N 64
constexpr uint32_t AX_IDESC_QK = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(AX_BN >> 3) << 17) | ((uint32_t)(AX_BM >> 4) << 24);
// kind::f16: D f32, A and B bf16, A K-major (TMEM), B MN-major, M 128, N = head dim
template <int D>
constexpr uint32_t AX_IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(AX_BM >> 4) << 24);

__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 :: "r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// V stage as the B operand of P.V: MN-major SWIZZLE_128B. 64 d (128 bytes) are contiguous; the
// next 64 d are AX_V_HALF bytes further (leading byte offset); 8 keys form a 1024-byte atom and
// the next 8 keys follow it (stride byte offset).
__device__ __forceinline__ uint64_t ax_v_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(AX_V_HALF >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// 4 bits (j, 8+j, 16+j, 24+j of h) -> 4 int8: query side +1 / -1, key side -2 / +2
__device__ __forceinline__ uint32_t ax_enc_q(uint32_t h, int j) { return 0xFFFFFFFFu ^ (((h >> j) & 0x01010101u) * 0xFEu); }
// key side as multiply-ADD (per byte 0x02 + {0, 0xFC}: no carry leaves a byte), one instruction less
// than multiply, then XOR: the expander warps' instruction count is what their tile rate hangs on
__device__ __forceinline__ uint32_t ax_enc_k(uint32_t h, int j) { return ((h >> j) & 0x01010101u) * 0xFCu + 0x02020202u; }

// acc (two packed fp32) += {p0, p1}: one instruction on sm_100
__device__ __forceinline__ void ax_add2(uint64_t& acc, float p0, float p1) {
    asm("{\n\t.reg .b64 t;\n\tmov.b64 t, {%1, %2};\n\tadd.rn.f32x2 %0, %0, t;\n\t}" : "+l"(acc) : "f"(p0), "f"(p1));
}
__device__ __forceinline__ float ax_sum4(uint64_t a, uint64_t b) {
    float a0, a1, b0, b1;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a0), "=f"(a1) : "l"(a));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(b0), "=f"(b1) : "l"(b));
    return (a0 + a1) + (b0 + b1);
}

template <int AX_D>      // head dim, 64 or 128. With 64 every operand row keeps its 128-byte pitch and half of it is used.
__global__ void __launch_bounds__(AX_THREADS, 2)
k_binary_attention_fwd_tcgen05(const __grid_constant__ CUtensorMap tmV,
                               const uint64_t* __restrict__ Qp, const uint64_t* __restrict__ Kp,
                               __nv_bfloat16* __restrict__ O,
                               int64_t S, int causal, float neg2c_log2 /* -2*scale*log2(e) */, float bias_log2,
                               int64_t q_tiles, int qt_major_flag) {
    extern __shared__ uint8_t ax_smem_raw[];
    // A CTA lives for 2 to 64 key tiles (a few microseconds), so its set-up is a real share of it: every
    // global load whose latency would head a role - the status word, the first K words, the Q rows, the
    // tensor map - is issued HERE, before the barrier set-up and the allocation of tensor memory, and
    // consumed after the one __syncthreads that the set-up needs anyway.
    __shared__ int s_skip;
    int skip_reg = 0;
    if (threadIdx.x == 0) skip_reg = *(volatile int*)&g_tc_status;      // an earlier CTA gave up: do not queue behind it

    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(ax_smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gbase = ax_smem_raw + (base - raw);
    const uint32_t v_ring = base, ke_ring = base + AX_OFF_KE, q_tile = base + AX_OFF_Q, bars = base + AX_OFF_BARS;
    uint8_t* gke = gbase + AX_OFF_KE;
    uint8_t* gq = gbase + AX_OFF_Q;
    // static, so that its address is a constant that folds into the lookups' load offsets
    __shared__ __align__(16) float T[AX_DMAX + 4];
    float* l_part = reinterpret_cast<float*>(gbase + AX_OFF_L);
    uint8_t* gbars = gbase + AX_OFF_BARS;
    auto v_full   = [&](int s) { return bars + 8u * s; };
    auto v_empty  = [&](int s) { return bars + 8u * (AX_NV + s); };
    auto ke_full  = [&](int s) { return bars + 8u * (2 * AX_NV + s); };
    auto ke_empty = [&](int s) { return bars + 8u * (2 * AX_NV + AX_NK + s); };
    const uint32_t s_full0 = bars + 8u * (2 * AX_NV + 2 * AX_NK), p_full0 = s_full0 + 16u;      // [2] each, by S/P buffer
    auto s_full = [&](int b) { return s_full0 + 8u * b; };
    auto p_full = [&](int b) { return p_full0 + 8u * b; };
    const uint32_t q_full = s_full0 + 32u, o_full = s_full0 + 40u, drain_bar = s_full0 + 48u;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbars + 8 * (2 * AX_NV + 2 * AX_NK + 7));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbars + 8 * (2 * AX_NV + 2 * AX_NK + 7) + 4);

    const int tid = threadIdx.x, lane = tid & 31;
    // through a shuffle so that the compiler knows the warp index, and with it every role branch
    // below, to be the same for all lanes of a warp
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    // Heavy (late) causal tiles first. grid = (q_tiles, heads): head by head, so that the CTAs in
    // flight share few heads' K and V in L2. grid = (heads, q_tiles) is the launcher's choice when
    // all heads' K and V fit in L2 together: then the heavy tiles of ALL heads go first and the light
    // ones fill the tail (few heads per GPU: 3.5 waves otherwise end half empty).
    const bool head_major = qt_major_flag == 0;
    const int64_t qt = q_tiles - 1 - (int64_t)(head_major ? blockIdx.x : blockIdx.y);
    const int64_t bh = head_major ? blockIdx.y : blockIdx.x;
    const int64_t q0 = qt * AX_BM;
    const int64_t kend = causal ? (q0 + AX_BM < S ? q0 + AX_BM : S) : S;
    const int32_t ntiles = (int32_t)((kend + AX_BN - 1) / AX_BN);  // >= 1 because q0 < S

    // ---- early loads (see above) ----
    constexpr int WPK = AX_D / 32;                        // 32-bit words per key: 4 or 2
    constexpr int AX_KPF = 4;                             // K words are fetched this many tiles ahead (a ring of registers)
    constexpr int QW = AX_D / 64;                         // 32-bit words of a Q row per softmax thread
    const uint32_t* Kw = reinterpret_cast<const uint32_t*>(Kp + bh * S * (AX_D / 64));
    const int khalf = warp - 2;                           // K expanders: keys [32 khalf, 32 khalf + 32) of the tile
    uint32_t kring[AX_KPF][WPK];
    // lane -> (key, word): 32 * WPK words per half tile, WPK per lane, coalesced
    auto load_tile = [&](int32_t j, uint32_t (&w)[WPK]) {
#pragma unroll
        for (int i = 0; i < WPK; ++i) {
            const int idx = lane + 32 * i;                // 0 .. 32 * WPK - 1
            const int64_t key = (int64_t)j * AX_BN + 32 * khalf + idx / WPK;
            w[i] = (j < ntiles && key < S) ? __ldg(Kw + key * WPK + idx % WPK) : 0u;
        }
    };
    uint32_t qh[QW];
    if (warp == 0) {
        if (lane == 0) asm volatile("prefetch.tensormap [%0];" :: "l"(&tmV) : "memory");
    } else if (warp == 2 || warp == 3) {
#pragma unroll
        for (int u = 0; u < AX_KPF - 1; ++u) load_tile(u, kring[u]);
    } else if (warp >= 4) {
        const int grp = (warp - 4) >> 2;
        const int64_t row = q0 + (warp & 3) * 32 + lane;
        const uint32_t* Qw = reinterpret_cast<const uint32_t*>(Qp + bh * S * (AX_D / 64));
#pragma unroll
        for (int w = 0; w < QW; ++w) qh[w] = row < S ? __ldg(Qw + row * (2 * QW) + QW * grp + w) : 0u;
    }

    // weights are bf16-exact, so the fp32 row sum adds exactly what the P.V MMA multiplies
    if (tid <= AX_D) T[tid] = __bfloat162float(__float2bfloat16_rn(exp2f(neg2c_log2 * (float)tid - bias_log2)));
    if (tid == 0) {
        for (int s = 0; s < AX_NV; ++s) { mbar_init(v_full(s), 1); mbar_init(v_empty(s), 1); }
        for (int s = 0; s < AX_NK; ++s) { mbar_init(ke_full(s), 2); mbar_init(ke_empty(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(s_full(b), 1); mbar_init(p_full(b), AX_SOFTMAX_WARPS); }
        mbar_init(q_full, AX_SOFTMAX_WARPS); mbar_init(o_full, 1); mbar_init(drain_bar, 1);
        *abort_flag = 0;
        s_skip = skip_reg;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async_smem();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"((uint32_t)__cvta_generic_to_shared((const void*)tmem_slot)), "r"((uint32_t)AX_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (s_skip != 0) {
        // an earlier CTA of this launch gave up: only hand the tensor memory back
    } else if (warp == 0) {
        // ================= TMA producer: V tiles =================
        if (lane == 0) {
            bool ok = true;
            int32_t issued = 0;
            for (int32_t j = 0; j < ntiles && ok; ++j) {
                const int s = j & (AX_NV - 1);
                ok = mbar_wait_relaxed(v_empty(s), ((j / AX_NV) & 1) ^ 1, abort_flag, 11);
                if (!ok) break;
                mbar_expect_tx(v_full(s), AX_V_HALF * (AX_D / 64));
                tma_load_3d(v_ring + s * AX_V_STAGE, &tmV, 0, j * AX_BN, (int32_t)bh, v_full(s));
                if (AX_D == 128) tma_load_3d(v_ring + s * AX_V_STAGE + AX_V_HALF, &tmV, 64, j * AX_BN, (int32_t)bh, v_full(s));
                issued = j + 1;
            }
            if (!ok) {
                const int32_t first = issued > AX_NV ? issued - AX_NV : 0;
                for (int32_t j = first; j < issued; ++j) {
                    const uint64_t t0 = tc_globaltimer();
                    while (!mbar_try(v_full(j % AX_NV), (j / AX_NV) & 1) && tc_globaltimer() - t0 < TC_WAIT_NS) {}
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        // The whole warp runs this loop convergently and one elected lane issues: descriptors,
        // addresses and loop state are then warp-uniform values, which the tcgen05 instructions take
        // as they are. Issued from inside an `if (lane == 0)` branch every operand first has to be
        // moved out of that one thread's registers, and each MMA took 70-100 clocks to issue - more
        // than the 32-64 clocks it runs.
        bool ok = __all_sync(0xffffffffu, mbar_wait(q_full, 0, abort_flag, 12));
        const uint64_t qdesc = tc_smem_desc(q_tile);
        const uint64_t kdesc0 = tc_smem_desc(ke_ring), vdesc0 = ax_v_desc(v_ring);
        // score MMA of tile j into S buffer j % 2. The buffer's last reader is the P.V MMA of tile
        // j - 2, issued before this one, and the tensor pipe runs in issue order.
        int kq = 0;                                  // K buffer of the next score MMA: tile % AX_NK
        auto issue_qk = [&](int b) {
            if (tc_elect_one()) {
                const uint64_t kdesc = kdesc0 + (uint64_t)(kq * (AX_KE_TILE >> 4));
#pragma unroll
                for (int k = 0; k < AX_D / 32; ++k)      // 32 bytes of d per instruction
                    tc_mma_i8_ss(tmem + (uint32_t)(AX_COL_S + 64 * b), qdesc + 2u * k, kdesc + 2u * k, AX_IDESC_QK, k > 0 ? 1u : 0u);
                tc_commit(s_full(b));
                tc_commit(ke_empty(kq));
            }
            __syncwarp();
            if (++kq == AX_NK) kq = 0;
        };
        // The prologue waits for the first two expanded K tiles itself. In the loop this warp waits
        // for ONE barrier per tile, p_full: two of the softmax warps check that V tile j and K tile
        // j + 2 have landed before they arrive on it (they have the slack; every wait, fence and
        // commit here is on the serial path that feeds the tensor pipe).
        for (int t = 0; t < 2 && t < ntiles && ok; ++t) {
            ok = __all_sync(0xffffffffu, mbar_wait(ke_full(t), 0, abort_flag, 13));
            if (!ok) break;
            tc_fence_after();
            issue_qk(t);
        }
        for (int32_t j0 = 0; j0 < ntiles && ok; j0 += AX_NV) {
#pragma unroll
            for (int u = 0; u < AX_NV; ++u) {            // u = V stage; S/P buffer b = u % 2: both static
                const int32_t j = j0 + u;
                if (j >= ntiles || !ok) break;
                const int b = u & 1;
                ok = __all_sync(0xffffffffu, mbar_wait(p_full(b), (j >> 1) & 1, abort_flag, 16));
                if (!ok) break;
                tc_fence_after();
                if (tc_elect_one()) {
                    const uint64_t vdesc = vdesc0 + (uint64_t)(u * (AX_V_STAGE >> 4));
#pragma unroll
                    for (int k = 0; k < 4; ++k) {    // 16 keys per instruction = two 1024-byte atoms of V
                        // P of keys [16k, 16k+16): 8 columns, inside the S columns of the thread that wrote them
                        const uint32_t pcol = (uint32_t)(AX_COL_S + 64 * b + 32 * (k >> 1) + 8 * (k & 1));
                        tc_mma_f16_ts(tmem + AX_COL_O, tmem + pcol, vdesc + (uint64_t)(128u * k), AX_IDESC_PV<AX_D>, (j > 0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(v_empty(u));
                }
                __syncwarp();
                if (j + 2 < ntiles) issue_qk(b);
            }
        }
        if (lane == 0) {
            if (ok) tc_commit(o_full);
            tc_commit(drain_bar);
            const uint64_t t0 = tc_globaltimer();
            while (!mbar_try(drain_bar, 0) && tc_globaltimer() - t0 < TC_WAIT_NS) {}
        }
        __syncwarp();
    } else if (warp < 4) {
        // ================= K expanders: packed bits -> int8 tile, K-major SWIZZLE_128B =================
        // The packed words are fetched AX_KPF tiles ahead into a ring of registers (the first three tiles'
        // before the CTA's set-up): one tile ahead left the load latency (L2, under load) on the path
        // and made this role the slowest of the CTA.
        const int half = khalf;
        auto& ring = kring;
        bool ok = true;
        int kb = 0;                                       // K buffer of tile j, j % AX_NK, and its phase
        uint32_t kbp = 0;
        for (int32_t j0 = 0; j0 < ntiles && ok; j0 += AX_KPF) {
#pragma unroll
            for (int u = 0; u < AX_KPF; ++u) {            // ring slots are static register names
                const int32_t j = j0 + u;
                if (j >= ntiles || !ok) break;
                load_tile(j + AX_KPF - 1, ring[(u + AX_KPF - 1) % AX_KPF]);
                // K buffer kb is free once the score MMA of tile j - AX_NK has completed. (A barrier of its
                // own: s_full of that tile may already be a phase further, which a parity wait cannot tell.)
                ok = __all_sync(0xffffffffu, mbar_wait_relaxed(ke_empty(kb), kbp ^ 1u, abort_flag, 17));
                if (!ok) break;
                const uint32_t (&cur)[WPK] = ring[u];
#pragma unroll
                for (int i = 0; i < WPK; ++i) {
                    const int idx = lane + 32 * i;
                    const int key = 32 * half + idx / WPK, w = idx % WPK;
                    uint8_t* row = gke + kb * AX_KE_TILE + key * 128;
                    const int sw = key & 7;
                    *reinterpret_cast<uint4*>(row + (((2 * w) ^ sw) << 4)) =
                        make_uint4(ax_enc_k(cur[i], 0), ax_enc_k(cur[i], 1), ax_enc_k(cur[i], 2), ax_enc_k(cur[i], 3));
                    *reinterpret_cast<uint4*>(row + (((2 * w + 1) ^ sw) << 4)) =
                        make_uint4(ax_enc_k(cur[i], 4), ax_enc_k(cur[i], 5), ax_enc_k(cur[i], 6), ax_enc_k(cur[i], 7));
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(ke_full(kb));
                if (++kb == AX_NK) { kb = 0; kbp ^= 1u; }
            }
        }
    } else {
        // ================= softmax (two threads per query row = TMEM lane), then epilogue =================
        const int quarter = warp & 3, grp = (warp - 4) >> 2;       // grp: which 32 of the tile's 64 keys
        const int r = quarter * 32 + lane;
        const int64_t row = q0 + r;
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
        {
            // Q row: this thread's half of the bits -> int8 chunks of the 128-byte operand row
            // (D = 128: 64 bits -> chunks 4 grp .. 4 grp + 3; D = 64: 32 bits -> chunks 2 grp, 2 grp + 1)
            uint8_t* qrow = gq + r * 128;
#pragma unroll
            for (int w = 0; w < QW; ++w) {
                const uint32_t h = qh[w];                 // loaded before the CTA's set-up
                const int ch = 2 * QW * grp + 2 * w;
                *reinterpret_cast<uint4*>(qrow + ((ch ^ (r & 7)) << 4)) =
                    make_uint4(ax_enc_q(h, 0), ax_enc_q(h, 1), ax_enc_q(h, 2), ax_enc_q(h, 3));
                *reinterpret_cast<uint4*>(qrow + (((ch + 1) ^ (r & 7)) << 4)) =
                    make_uint4(ax_enc_q(h, 4), ax_enc_q(h, 5), ax_enc_q(h, 6), ax_enc_q(h, 7));
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(q_full);
        }
        const uint32_t tc_addr = (uint32_t)__cvta_generic_to_shared(T) + 2 * AX_D;      // acc = 4*h - 2*D -> T[h]
        int kx = 2 % AX_NK;                                        // K buffer and phase of tile j + 2
        uint32_t kxp = 2 / AX_NK;
        uint64_t l2a = 0, l2b = 0;                                  // two packed pairs of fp32 partial row sums
        bool ok = true;
        for (int32_t j = 0; j < ntiles && ok; ++j) {
            const int64_t k0 = (int64_t)j * AX_BN + 32 * grp;       // first key of this thread's 32
            const bool need_mask = (causal && k0 + 31 > q0) || (k0 + 32 > S);
            const int b = j & 1;
            const uint32_t my_cols = lane_base + (uint32_t)(AX_COL_S + 64 * b + 32 * grp);
            ok = __all_sync(0xffffffffu, mbar_wait(s_full(b), (j >> 1) & 1, abort_flag, 18));
            if (!ok) break;
            tc_fence_after();
            uint32_t sc[32], pk[16];
            tc_ld32(my_cols, sc);
            tc_wait_ld();
            if (!need_mask) {
                // the common tile: nothing but 2 loads, 1 packed add and 1 byte permute per pair of
                // scores, with no branch between the 32 loads
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float p0, p1;
                    asm("ld.shared.f32 %0, [%1];" : "=f"(p0) : "r"(tc_addr + sc[i]));
                    asm("ld.shared.f32 %0, [%1];" : "=f"(p1) : "r"(tc_addr + sc[i + 1]));
                    ax_add2(i & 2 ? l2b : l2a, p0, p1);
                    // entries are bf16-exact: the pair is the two upper halves
                    pk[i >> 1] = __byte_perm(__float_as_uint(p0), __float_as_uint(p1), 0x7632);
                }
            } else {
                // keys [k0, k0 + lim) of this thread's 32 are inside the sequence and not above the diagonal
                int64_t a = S - k0;
                if (causal && row - k0 + 1 < a) a = row - k0 + 1;
                const int lim = a < 0 ? 0 : (a > 32 ? 32 : (int)a);
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float p0, p1;
                    asm("ld.shared.f32 %0, [%1];" : "=f"(p0) : "r"(tc_addr + sc[i]));
                    asm("ld.shared.f32 %0, [%1];" : "=f"(p1) : "r"(tc_addr + sc[i + 1]));
                    p0 = i < lim ? p0 : 0.f;
                    p1 = i + 1 < lim ? p1 : 0.f;
                    ax_add2(i & 2 ? l2b : l2a, p0, p1);
                    pk[i >> 1] = __byte_perm(__float_as_uint(p0), __float_as_uint(p1), 0x7632);
                }
            }
            // over the first 16 of the 32 columns this thread has just read
            tc_st16(my_cols, pk);
            tc_wait_st();
            tc_fence_before();
            // on behalf of the MMA warp, which waits for p_full alone: V tile j and the expanded K
            // tile j + 2 (the operands of the two MMA groups it issues next) have landed
            if (warp == 4) ok = __all_sync(0xffffffffu, mbar_wait(v_full(j & (AX_NV - 1)), (j / AX_NV) & 1, abort_flag, 15));
            if (warp == 5 && j + 2 < ntiles) ok = __all_sync(0xffffffffu, mbar_wait(ke_full(kx), kxp, abort_flag, 13));
            if (++kx == AX_NK) { kx = 0; kxp ^= 1u; }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(b));
        }
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(o_full, 0, abort_flag, 20));
        // the two halves of a row exchange their sums; one verdict for all softmax warps first
        l_part[grp * AX_BM + r] = ax_sum4(l2a, l2b);
        uint32_t bad;
        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.or.pred q, 1, %2, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                     : "=r"(bad) : "r"((uint32_t)(!ok)), "n"(AX_SOFTMAX_WARPS * 32) : "memory");
        if (!bad) {
            tc_fence_after();
            const float lsum = l_part[r] + l_part[AX_BM + r];
            const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
            __nv_bfloat16* orow = O + (bh * S + row) * AX_D + (AX_D / 2) * grp;      // this thread's half of the columns
#pragma unroll 1
            for (int c = 0; c < AX_D / 64; ++c) {
                uint32_t v[32];
                tc_ld32(lane_base + AX_COL_O + (AX_D / 2) * grp + 32 * c, v);
                tc_wait_ld();
                if (row < S) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 o4;
                        o4.x = pack_bf16x2(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
                        o4.y = pack_bf16x2(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
                        o4.z = pack_bf16x2(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
                        o4.w = pack_bf16x2(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + 32 * c + i) = o4;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"((uint32_t)AX_TMEM_COLS) : "memory");
    }
}

// V [BH, S, D] bf16 as a 3-D tensor, box = [64 d, 64 keys, 1], SWIZZLE_128B: keys past S read as zero
static bool ax_make_v_map(CUtensorMap* tm, const void* V, int64_t BH, int64_t S, int AX_D) {
    PFN_tmapEncodeTiled enc = tc5_encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)AX_D, (cuuint64_t)S, (cuuint64_t)BH};
    const cuuint64_t strides[2] = {(cuuint64_t)AX_D * 2u, (cuuint64_t)S * AX_D * 2u};
    const cuuint32_t box[3] = {64u, (cuuint32_t)AX_BN, 1u};
    const cuuint32_t estr[3] = {1, 1, 1};
    return enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(V), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D>
static int ax_run(const uint64_t* Qp, const uint64_t* Kp, const void* V, void* O, int64_t BH, int64_t S,
                  int causal, float neg2c_log2, float bias_log2, cudaStream_t st) {
    CUtensorMap tmV;
    BB_REQUIRE(S < (1ll << 31) - AX_BM && ax_make_v_map(&tmV, V, BH, S, D), BRUTE_ERR_DRIVER);
    if (!kernel_smem_ready<k_binary_attention_fwd_tcgen05<D>>(AX_SMEM)) return BRUTE_ERR_LAUNCH;
    const int64_t q_tiles = (S + AX_BM - 1) / AX_BM;
    // K + V of all heads against a third of the L2 (126 MB): see the kernel's tile order
    const bool qt_major = causal && q_tiles <= 65535 && BH * S * (int64_t)(2 * D + D / 4) <= (80ll << 20);
    const dim3 grid = qt_major ? dim3((unsigned)BH, (unsigned)q_tiles) : dim3((unsigned)q_tiles, (unsigned)BH);
    k_binary_attention_fwd_tcgen05<D><<<grid, AX_THREADS, AX_SMEM, st>>>(tmV, Qp, Kp, static_cast<__nv_bfloat16*>(O), S, causal,
                                                                       neg2c_log2, bias_log2, q_tiles, qt_major ? 1 : 0);
    return launch_status();
}

}  // namespace bb
