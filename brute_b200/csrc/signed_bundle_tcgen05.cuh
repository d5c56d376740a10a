// signed_bundle on the 5th-generation tensor cores.
//
//   out[b, m, d] = ( sum_n W[b, m, n] * pm1(V[b, n, d]) >= 0 ),   pm1(bit) = 2*bit - 1
// This is a GEMM with M = rows of W, N = d, K = n: W [M, N] int8 is already the K-major A operand and
// goes from global memory straight into SWIZZLE_128B shared memory by TMA; the B operand is V
// TRANSPOSED ([d, n], n contiguous). FUSED: the expander warps read V itself and transpose each
// 128 (n) x 128 (d) bit block in registers, one 64 x 64 butterfly per warp and k-block, so the op is
// ONE launch and needs no workspace. Otherwise (the entry points that take a workspace) the launcher
// first bit-transposes V into it (brute_b200_transpose_bits) and a thread expands 128 bits of a Vt
// row. Either way a bit becomes a byte of +1 / -1 in the K-major SWIZZLE_128B tile, so the
// accumulator IS the signed sum and its sign bit is the output (an earlier version expanded to 0 / 1
// and took the row sums of W from a 129th B row: 144 accumulator columns, which left no room for a
// second accumulator in the CTA's 256 columns of tensor memory).
// kind::i8 with A and B signed; M128 N128 K32, 4 per 128 bytes of n.
//
// The kernel streams W once: B*M*N bytes against B*M*N*D MACs, i.e. it is HBM bound once the
// tensor cores do the MACs (the dp4a kernel in signed_bundle.cu is 30x away from that bound).
//
// Work item = 128 rows of W of one batch x one block of 128 d; persistent CTAs of 320 threads
// (two per SM) walk over the items:
//   warp 0      TMA producer for W tiles (4-deep ring of 16 KB)
//   warp 1      MMA issuer, TMEM owner (256 columns = TWO accumulators; two CTAs per SM)
//   warps 2-9   expand Vt bits into the B tile (2-deep ring of 128 x 128 bytes), item after item: two
//               groups of four warps, one per ring stage, take the k-blocks alternately (measured with
//               one group: the MMA warp spent two thirds of every k-block waiting for the expanded
//               tile, the expanders a tenth of theirs waiting for a free stage)
//   warps 10-13 epilogue: one thread per row reads its TMEM lane and packs the sign bits, while the
//               other accumulator already takes the next item's MMAs (an item is only 8 k-blocks
//               at N = 1024: with one accumulator and the expanders doing the epilogue, every
//               item drained the W ring).
// Every mbarrier wait is bounded; a wait that gives up raises the abort flag and the status word.
#pragma once
#include "tcgen05_common.cuh"

namespace bb {

constexpr int ST_BM = 128;                   // rows of W per CTA
constexpr int ST_DB = 128;                   // d per CTA (two packed output words per row)
constexpr int ST_NMMA = ST_DB;
constexpr int ST_KB = 128;                   // bytes (= n) per k-block
constexpr int ST_ASTAGES = 4, ST_BSTAGES = 2;
constexpr int ST_A_TILE = ST_BM * ST_KB;     // 16 KB
constexpr int ST_B_TILE = ST_NMMA * ST_KB;   // 16 KB
constexpr int ST_THREADS = 448;
constexpr int ST_FIRST_EPI_WARP = 10;      // warps 2-5 and 6-9: two expander groups; 10-13: epilogue
constexpr int ST_TMEM_COLS = 256;
constexpr int ST_OFF_B = ST_ASTAGES * ST_A_TILE;
constexpr int ST_OFF_BARS = ST_OFF_B + ST_BSTAGES * ST_B_TILE;
constexpr int ST_SMEM = ST_OFF_BARS + 256 + 1024;
static_assert(ST_B_TILE % 1024 == 0, "operand tiles are 1024-byte aligned");
static_assert(ST_ASTAGES % ST_BSTAGES == 0, "the B ring position is static inside the unrolled A ring");

// kind::i8: D s32, A and B signed int8, K-major both, M 128, N 128
constexpr uint32_t ST_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(ST_NMMA >> 3) << 17) | ((uint32_t)(ST_BM >> 4) << 24);

// bits p..p+3 of w -> 4 bytes of +1 / -1 in natural order (byte i = bit p + i): 0 / 1 per byte first,
// then 0xFF - 0xFE * that, as one multiply-add (no byte borrows: 0xFF - 0xFE = 0x01)
__device__ __forceinline__ uint32_t st_bits4_to_bytes(uint32_t w, int p) {
    return ((((w >> p) & 0xFu) * 0x00204081u) & 0x01010101u) * 0xFFFFFF02u + 0xFFFFFFFFu;
}

template <bool FUSED>
__global__ void __launch_bounds__(ST_THREADS, 2)
k_signed_bundle_tcgen05(const __grid_constant__ CUtensorMap tmW,
                        const uint64_t* __restrict__ Vt /* FUSED: V itself, [B, N, Dp] words; else [B, D, wpn] words, bit n of row d */,
                        uint64_t* __restrict__ out /* [B, M, Dp] */,
                        int64_t M, int64_t N, int64_t D, int64_t Dp, int64_t wpn,
                        int32_t m_tiles, int32_t d_blocks, int64_t items) {
    extern __shared__ uint8_t st_smem_raw[];
    __shared__ int s_skip;
    if (threadIdx.x == 0) s_skip = *(volatile int*)&g_tc_status;
    __syncthreads();
    if (s_skip != 0) return;

    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(st_smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gbase = st_smem_raw + (base - raw);
    const uint32_t a_ring = base, b_ring = base + ST_OFF_B, bars = base + ST_OFF_BARS;
    uint8_t* gb = gbase + ST_OFF_B;
    uint8_t* gbars = gbase + ST_OFF_BARS;
    auto a_full  = [&](int s) { return bars + 8u * s; };
    auto a_empty = [&](int s) { return bars + 8u * (ST_ASTAGES + s); };
    auto b_full  = [&](int s) { return bars + 8u * (2 * ST_ASTAGES + s); };
    auto b_empty = [&](int s) { return bars + 8u * (2 * ST_ASTAGES + ST_BSTAGES + s); };
    constexpr int NB = 2 * ST_ASTAGES + 2 * ST_BSTAGES;
    auto acc_full  = [&](int s) { return bars + 8u * (NB + s); };          // two accumulators
    auto acc_empty = [&](int s) { return bars + 8u * (NB + 2 + s); };
    const uint32_t drain_bar = bars + 8u * (NB + 4);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbars + 8 * (NB + 5));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbars + 8 * (NB + 5) + 4);

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);      // a shuffle result: known to the compiler as the same in all lanes
    const int32_t nkb = (int32_t)((N + ST_KB - 1) / ST_KB);
    // work item -> (row tile, d block, batch); consecutive items share the batch and the d block
    auto item_coords = [&](int64_t it, int64_t& m0, int64_t& dblk, int64_t& b) {
        m0 = (it % m_tiles) * ST_BM;
        dblk = (it / m_tiles) % d_blocks;
        b = it / ((int64_t)m_tiles * d_blocks);
    };

    if (tid == 0) {
        for (int s = 0; s < ST_ASTAGES; ++s) { mbar_init(a_full(s), 1); mbar_init(a_empty(s), 1); }
        for (int s = 0; s < ST_BSTAGES; ++s) { mbar_init(b_full(s), 4); mbar_init(b_empty(s), 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(acc_full(s), 1); mbar_init(acc_empty(s), 4); }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_proxy_async_smem();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"((uint32_t)__cvta_generic_to_shared((const void*)tmem_slot)), "r"((uint32_t)ST_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // Persistent: the CTA walks over work items, and every role keeps ONE running count of the
    // k-blocks it has handled, so the TMA ring never drains between items (a CTA per item paid its
    // set-up, its first TMA latency and its epilogue once per 128 KB of W).
    if (warp == 0) {
        // ================= TMA producer: W tiles [128 rows x 128 bytes of n] =================
        if (lane == 0) {
            bool ok = true;
            uint32_t g = 0;                                   // k-blocks issued so far
            for (int64_t it = blockIdx.x; it < items && ok; it += gridDim.x) {
                int64_t m0, dblk, b;
                item_coords(it, m0, dblk, b);
                for (int32_t kb = 0; kb < nkb; ++kb, ++g) {
                    const int s = (int)(g % ST_ASTAGES);
                    ok = mbar_wait(a_empty(s), ((g / ST_ASTAGES) & 1u) ^ 1u, abort_flag, 21);
                    if (!ok) break;
                    mbar_expect_tx(a_full(s), ST_A_TILE);
                    tma_load_3d(a_ring + s * ST_A_TILE, &tmW, kb * ST_KB, (int32_t)m0, (int32_t)b, a_full(s));
                }
            }
            if (!ok) {
                // g loads were issued; let the last ring's worth land before the shared memory goes away
                const uint32_t first = g > (uint32_t)ST_ASTAGES ? g - ST_ASTAGES : 0u;
                for (uint32_t k = first; k < g; ++k) {
                    const uint64_t t0 = tc_globaltimer();
                    while (!mbar_try(a_full((int)(k % ST_ASTAGES)), (k / ST_ASTAGES) & 1u) && tc_globaltimer() - t0 < TC_WAIT_NS) {}
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        // The whole warp runs the loop and one elected lane issues: next to busy warps a one-thread
        // role pays 10+ clocks per instruction, and this one sits between the TMA data and the
        // tensor pipe.
        bool ok = true;
        const uint64_t adesc0 = tc_smem_desc(a_ring), bdesc0 = tc_smem_desc(b_ring);
        uint32_t g = 0, n_items = 0;
        for (int64_t it = blockIdx.x; it < items && ok; it += gridDim.x, ++n_items) {
            // this accumulator's previous item (two items back) has been read by the four epilogue warps
            const int ab = (int)(n_items & 1u);
            const uint32_t acc = tmem + (uint32_t)(ST_DB * ab);
            ok = __all_sync(0xffffffffu, mbar_wait(acc_empty(ab), ((n_items >> 1) & 1u) ^ 1u, abort_flag, 26));
            if (!ok) break;
            tc_fence_after();
            for (int32_t kb = 0; kb < nkb && ok; ++kb, ++g) {
                const int sa = (int)(g % ST_ASTAGES), sb = (int)(g % ST_BSTAGES);
                ok = __all_sync(0xffffffffu, mbar_wait(a_full(sa), (g / ST_ASTAGES) & 1u, abort_flag, 22) &&
                                             mbar_wait(b_full(sb), (g / ST_BSTAGES) & 1u, abort_flag, 23));
                if (!ok) break;
                tc_fence_after();
                if (tc_elect_one()) {
                    const uint64_t adesc = adesc0 + (uint64_t)(sa * (ST_A_TILE >> 4));
                    const uint64_t bdesc = bdesc0 + (uint64_t)(sb * (ST_B_TILE >> 4));
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tc_mma_i8_ss(acc, adesc + 2u * k, bdesc + 2u * k, ST_IDESC, (kb > 0 || k > 0) ? 1u : 0u);
                    tc_commit(a_empty(sa));
                    tc_commit(b_empty(sb));
                }
                __syncwarp();
            }
            if (ok && tc_elect_one()) tc_commit(acc_full(ab));
            __syncwarp();
        }
        if (lane == 0) {
            tc_commit(drain_bar);
            const uint64_t t0 = tc_globaltimer();
            while (!mbar_try(drain_bar, 0) && tc_globaltimer() - t0 < TC_WAIT_NS) {}
        }
        __syncwarp();
    } else if (warp < ST_FIRST_EPI_WARP) {
        // ================= B expanders, item after item =================
        // The CTA's k-blocks form one stream over all of its items; the packed words are fetched
        // ST_VPF - 1 k-blocks ahead of the expansion ACROSS item boundaries (a ring of registers), so
        // that no item starts with a global-load latency on its path.
        const int t = (tid - 64) & 127;                      // 0..127: non-fused, the thread's d row
        const int grp = (warp - 2) >> 2;                     // this group takes the k-blocks g with g % 2 == grp, into stage grp
        // FUSED: warp (rb, cb) owns the 64 (n) x 64 (d) bit block rb, cb of the k-block's 128 x 128:
        // lane L loads word cb of rows n0 + 64 rb + L and + 32, the butterfly turns them into the
        // 64 n-bits of d rows 64 cb + L and + 32, and the lane writes those two half rows.
        const int wq = (warp - 2) & 3, rb = wq >> 1, cb = wq & 1;
        const int64_t my_items = blockIdx.x < items ? (items - 1 - blockIdx.x) / gridDim.x + 1 : 0;
        const int64_t total = my_items * nkb;                // k-blocks of this CTA
        // the fetch cursor: item, k-block, and what depends on the item only
        int64_t pit = blockIdx.x;
        int32_t pkb = 0;
        const uint64_t* pvrow = Vt;
        bool plive = false;
        auto fetch_item = [&]() {
            plive = false;
            if (pit >= items) return;
            int64_t m0, dblk, b;
            item_coords(pit, m0, dblk, b);
            if (FUSED) {
                const int64_t vword = 2 * dblk + cb;             // word of a V row
                plive = vword < Dp;
                pvrow = Vt + b * N * Dp + (plive ? vword : 0);
            } else {
                const int64_t d = dblk * ST_DB + t;
                plive = d < D;
                pvrow = Vt + (b * D + (plive ? d : 0)) * wpn;
            }
        };
        auto advance = [&]() {
            if (pit >= items) return;
            if (++pkb == nkb) { pkb = 0; pit += gridDim.x; fetch_item(); }
        };
        auto fetch = [&](uint64_t (&w)[2]) {
            w[0] = w[1] = 0ull;
            if (pit >= items) return;
            if (FUSED) {
                const int64_t n = (int64_t)pkb * ST_KB + 64 * rb + lane;
                if (plive && n < N) w[0] = __ldg(pvrow + n * Dp);
                if (plive && n + 32 < N) w[1] = __ldg(pvrow + (n + 32) * Dp);
            } else {
                const int64_t w0 = 2 * (int64_t)pkb;
                if (plive && w0 < wpn) w[0] = __ldg(pvrow + w0);
                if (plive && w0 + 1 < wpn) w[1] = __ldg(pvrow + w0 + 1);
            }
            advance();
            advance();                                       // the other group takes the k-block in between
        };
        fetch_item();
        if (grp == 1) advance();
        constexpr int ST_VPF = 4;
        uint64_t ring[ST_VPF][2];
#pragma unroll
        for (int u = 0; u < ST_VPF - 1; ++u) fetch(ring[u]);
        bool ok = true;
        static_assert(ST_BSTAGES == 2, "one expander group per stage");
        for (int64_t g0 = grp; g0 < total && ok; g0 += 2 * ST_VPF) {
#pragma unroll
            for (int u = 0; u < ST_VPF; ++u) {                // ring slots are static register names
                const int64_t g = g0 + 2 * u;
                if (g >= total || !ok) break;
                fetch(ring[(u + ST_VPF - 1) % ST_VPF]);
                const int sb = grp;
                ok = __all_sync(0xffffffffu, mbar_wait(b_empty(sb), ((uint32_t)(g / ST_BSTAGES) & 1u) ^ 1u, abort_flag, 24));
                if (!ok) break;
                // rows d >= D expand whatever their (zero) words say: those output bits are masked in the epilogue
                if (FUSED) {
                    uint64_t lo = ring[u][0], hi = ring[u][1];
                    transpose64x64(lo, hi, lane);             // lo: d row 64 cb + lane, hi: + 32; bit j = n0 + 64 rb + j
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int r = 64 * cb + lane + 32 * h;
                        const uint64_t bitsr = h ? hi : lo;
                        uint8_t* row = gb + sb * ST_B_TILE + r * 128;
#pragma unroll
                        for (int c = 0; c < 4; ++c) {         // chunk 4 rb + c of the row: its 16 bits 16 c .. 16 c + 15
                            const uint32_t w32 = (uint32_t)(bitsr >> (16 * c));
                            *reinterpret_cast<uint4*>(row + (((4 * rb + c) ^ (r & 7)) << 4)) =
                                make_uint4(st_bits4_to_bytes(w32, 0), st_bits4_to_bytes(w32, 4), st_bits4_to_bytes(w32, 8), st_bits4_to_bytes(w32, 12));
                        }
                    }
                } else {
                    const uint64_t (&cur)[2] = ring[u];
                    uint8_t* row = gb + sb * ST_B_TILE + t * 128;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {             // chunk c: bytes 16c .. 16c+15 = bits 16c .. 16c+15
                        const uint32_t w32 = (uint32_t)(cur[c >> 2] >> (16 * (c & 3)));
                        *reinterpret_cast<uint4*>(row + ((c ^ (t & 7)) << 4)) =
                            make_uint4(st_bits4_to_bytes(w32, 0), st_bits4_to_bytes(w32, 4), st_bits4_to_bytes(w32, 8), st_bits4_to_bytes(w32, 12));
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(b_full(sb));
            }
        }
    } else {
        // ================= epilogue (thread = one row of W): sign bits of the accumulator =================
        const int quarter = warp & 3;
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
        bool ok = true;
        uint32_t n_items = 0;
        for (int64_t it = blockIdx.x; it < items && ok; it += gridDim.x, ++n_items) {
            int64_t m0, dblk, b;
            item_coords(it, m0, dblk, b);
            const int ab = (int)(n_items & 1u);
            ok = __all_sync(0xffffffffu, mbar_wait(acc_full(ab), (n_items >> 1) & 1u, abort_flag, 25));
            if (!ok) break;
            tc_fence_after();
            const int64_t m = m0 + quarter * 32 + lane;
            uint32_t bits[4];
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tc_ld32(lane_base + (uint32_t)(ST_DB * ab + 32 * c), v);
                tc_wait_ld();
                if (c == 3) {                                 // the accumulator is in registers: hand it back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty(ab));
                }
                uint32_t w = 0;
#pragma unroll
                for (int j = 0; j < 32; ++j) w |= ((int32_t)v[j] >= 0 ? 1u : 0u) << j;
                bits[c] = w;
            }
            if (m < M) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int64_t word = 2 * dblk + h;
                    if (word >= Dp) continue;
                    uint64_t w = (uint64_t)bits[2 * h] | ((uint64_t)bits[2 * h + 1] << 32);
                    const int64_t valid = D - word * 64;                 // pad bits stay 0
                    if (valid < 64) w = valid <= 0 ? 0ull : (w & ((1ull << valid) - 1ull));
                    out[(b * M + m) * Dp + word] = w;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"((uint32_t)ST_TMEM_COLS) : "memory");
    }
}

// W [B, M, N] int8 as a 3-D tensor, box = [128 n, 128 m, 1], SWIZZLE_128B: rows past M and bytes past N read as zero
static bool st_make_w_map(CUtensorMap* tm, const int8_t* W, int64_t B, int64_t M, int64_t N) {
    PFN_tmapEncodeTiled enc = tc5_encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)B};
    const cuuint64_t strides[2] = {(cuuint64_t)N, (cuuint64_t)(M * N)};
    const cuuint32_t box[3] = {(cuuint32_t)ST_KB, (cuuint32_t)ST_BM, 1u};
    const cuuint32_t estr[3] = {1, 1, 1};
    return enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t*>(W), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Shapes the tensor-core path takes: TMA wants a 16-byte aligned base and row pitch; below one
// full tile of rows the dp4a kernel is as good; |S| and |T| stay far inside int32 for N < 2^23.
static bool st_accepts(const int8_t* W, int64_t B, int64_t M, int64_t N, int64_t D) {
    return aligned16(W) && (N % 16) == 0 && N >= 128 && M >= 64 && D >= 1 && N < (1ll << 23) &&
           B <= 65535 && (M + ST_BM - 1) / ST_BM <= 0x7fffffffll && (D + ST_DB - 1) / ST_DB <= 65535;
}

// fused: `Vt` is V itself ([B, N, Dp]) and the kernel transposes on the fly; else the bit-transposed V
static int st_run(const int8_t* W, const uint64_t* Vt, uint64_t* out, int64_t B, int64_t M, int64_t N,
                  int64_t Dp, int64_t D, cudaStream_t st, bool fused) {
    CUtensorMap tmW;
    BB_REQUIRE(st_make_w_map(&tmW, W, B, M, N), BRUTE_ERR_DRIVER);
    if (!(fused ? kernel_smem_ready<k_signed_bundle_tcgen05<true>>(ST_SMEM)
                : kernel_smem_ready<k_signed_bundle_tcgen05<false>>(ST_SMEM))) return BRUTE_ERR_LAUNCH;
    const int64_t m_tiles = (M + ST_BM - 1) / ST_BM, d_blocks = (D + ST_DB - 1) / ST_DB;
    const int64_t items = m_tiles * d_blocks * B;
    const int64_t resident = 2 * (int64_t)kNumSMs;                     // two CTAs per SM (shared memory)
    const unsigned grid = (unsigned)(items < resident ? items : resident);
    if (fused)
        k_signed_bundle_tcgen05<true><<<grid, ST_THREADS, ST_SMEM, st>>>(tmW, Vt, out, M, N, D, Dp, (N + 63) / 64,
                                                                       (int32_t)m_tiles, (int32_t)d_blocks, items);
    else
        k_signed_bundle_tcgen05<false><<<grid, ST_THREADS, ST_SMEM, st>>>(tmW, Vt, out, M, N, D, Dp, (N + 63) / 64,
                                                                        (int32_t)m_tiles, (int32_t)d_blocks, items);
    return launch_status();
}

}  // namespace bb
