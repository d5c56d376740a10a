// signed_bundle on the 5th-generation tensor cores.
//
//   out[b, m, d] = ( sum_n W[b, m, n] * pm1(V[b, n, d]) >= 0 ),   pm1(bit) = 2*bit - 1
//                = ( 2*T[m, d] - S[m] >= 0 ),  T = sum_n W[m, n] * bit(V[n, d]),  S[m] = sum_n W[m, n].
// T is a GEMM with M = rows of W, N = d, K = n: W [M, N] int8 is already the K-major A operand and
// goes from global memory straight into SWIZZLE_128B shared memory by TMA; the B operand is V
// TRANSPOSED ([d, n], n contiguous). FUSED: the expander warps read V itself and transpose each
// 128 (n) x 128 (d) bit block in registers, one 64 x 64 butterfly per warp and k-block, so the op is
// ONE launch and needs no workspace. Otherwise (the entry points that take a workspace) the launcher
// first bit-transposes V into it (brute_b200_transpose_bits) and a thread expands 128 bits of a Vt
// row. Either way a bit becomes a byte of 0/1 in the K-major SWIZZLE_128B tile.
// S comes out of the same MMAs from one extra B row of ones (accumulator column 128).
// kind::i8 with A signed, B unsigned; M128 N144 K32, 4 per 128 bytes of n.
//
// The kernel streams W once: B*M*N bytes against B*M*N*D MACs, i.e. it is HBM bound once the
// tensor cores do the MACs (the dp4a kernel in signed_bundle.cu is 30x away from that bound).
//
// Work item = 128 rows of W of one batch x one block of 128 d; persistent CTAs of 192 threads
// (two per SM) walk over the items:
//   warp 0      TMA producer for W tiles (4-deep ring of 16 KB)
//   warp 1      MMA issuer, TMEM owner (256 columns; two CTAs per SM)
//   warps 2-5   expand Vt bits into the B tile (2-deep ring of 144 x 128 bytes), then the epilogue:
//               one thread per row reads T and S from its TMEM lane and packs the sign bits.
// Every mbarrier wait is bounded; a wait that gives up raises the abort flag and the status word.
#pragma once
#include "tcgen05_common.cuh"

namespace bb {

constexpr int ST_BM = 128;                   // rows of W per CTA
constexpr int ST_DB = 128;                   // d per CTA (two packed output words per row)
constexpr int ST_NMMA = ST_DB + 16;          // + the row of ones (and 15 rows of zeros: N must be a multiple of 16)
constexpr int ST_KB = 128;                   // bytes (= n) per k-block
constexpr int ST_ASTAGES = 4, ST_BSTAGES = 2;
constexpr int ST_A_TILE = ST_BM * ST_KB;     // 16 KB
constexpr int ST_B_TILE = ST_NMMA * ST_KB;   // 18 KB
constexpr int ST_THREADS = 192;
constexpr int ST_TMEM_COLS = 256;
constexpr int ST_OFF_B = ST_ASTAGES * ST_A_TILE;
constexpr int ST_OFF_BARS = ST_OFF_B + ST_BSTAGES * ST_B_TILE;
constexpr int ST_SMEM = ST_OFF_BARS + 256 + 1024;
static_assert(ST_B_TILE % 1024 == 0, "operand tiles are 1024-byte aligned");
static_assert(ST_ASTAGES % ST_BSTAGES == 0, "the B ring position is static inside the unrolled A ring");

// kind::i8: D s32, A signed int8, B unsigned int8, K-major both, M 128, N 144
constexpr uint32_t ST_IDESC = (2u << 4) | (1u << 7) | (0u << 10) | ((uint32_t)(ST_NMMA >> 3) << 17) | ((uint32_t)(ST_BM >> 4) << 24);

__device__ __forceinline__ uint32_t tc_ld1(uint32_t taddr) {
    uint32_t r;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
    return r;
}
// bits p..p+3 of w -> 4 bytes of 0/1 in natural order (byte i = bit p + i)
__device__ __forceinline__ uint32_t st_bits4_to_bytes(uint32_t w, int p) {
    return (((w >> p) & 0xFu) * 0x00204081u) & 0x01010101u;
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
    const uint32_t acc_full = bars + 8u * NB, acc_empty = acc_full + 8u, drain_bar = acc_full + 16u;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbars + 8 * (NB + 3));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbars + 8 * (NB + 3) + 4);

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);      // a shuffle result: known to the compiler as the same in all lanes
    const int32_t nkb = (int32_t)((N + ST_KB - 1) / ST_KB);
    // work item -> (row tile, d block, batch); consecutive items share the batch and the d block
    auto item_coords = [&](int64_t it, int64_t& m0, int64_t& dblk, int64_t& b) {
        m0 = (it % m_tiles) * ST_BM;
        dblk = (it / m_tiles) % d_blocks;
        b = it / ((int64_t)m_tiles * d_blocks);
    };

    // the constant rows of both B tiles: row 128 = ones (gives S), rows 129..143 = zeros
    for (int i = tid; i < ST_BSTAGES * 16 * 8; i += ST_THREADS) {
        const int s = i / (16 * 8), r = ST_DB + (i / 8) % 16, c = i % 8;
        const uint32_t v = r == ST_DB ? 0x01010101u : 0u;
        *reinterpret_cast<uint4*>(gb + s * ST_B_TILE + r * 128 + ((c ^ (r & 7)) << 4)) = make_uint4(v, v, v, v);
    }
    if (tid == 0) {
        for (int s = 0; s < ST_ASTAGES; ++s) { mbar_init(a_full(s), 1); mbar_init(a_empty(s), 1); }
        for (int s = 0; s < ST_BSTAGES; ++s) { mbar_init(b_full(s), 4); mbar_init(b_empty(s), 1); }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 4);
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
            // the accumulator of the previous item has been read by the four epilogue warps
            ok = __all_sync(0xffffffffu, mbar_wait(acc_empty, (n_items & 1u) ^ 1u, abort_flag, 26));
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
                        tc_mma_i8_ss(tmem, adesc + 2u * k, bdesc + 2u * k, ST_IDESC, (kb > 0 || k > 0) ? 1u : 0u);
                    tc_commit(a_empty(sa));
                    tc_commit(b_empty(sb));
                }
                __syncwarp();
            }
            if (ok && tc_elect_one()) tc_commit(acc_full);
            __syncwarp();
        }
        if (lane == 0) {
            tc_commit(drain_bar);
            const uint64_t t0 = tc_globaltimer();
            while (!mbar_try(drain_bar, 0) && tc_globaltimer() - t0 < TC_WAIT_NS) {}
        }
        __syncwarp();
    } else {
        // ================= B expanders (thread = one d row), then the epilogue (thread = one row of W) =================
        const int t = tid - 64;                              // 0..127
        const int quarter = warp & 3;
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
        bool ok = true;
        uint32_t g = 0, n_items = 0;
        for (int64_t it = blockIdx.x; it < items && ok; it += gridDim.x, ++n_items) {
            int64_t m0, dblk, b;
            item_coords(it, m0, dblk, b);
            // FUSED: warp (rb, cb) owns the 64 (n) x 64 (d) bit block rb, cb of the k-block's 128 x 128:
            // lane L loads word cb of rows n0 + 64 rb + L and + 32, the butterfly turns them into the
            // 64 n-bits of d rows 64 cb + L and + 32, and the lane writes those two half rows.
            const int wq = warp - 2, rb = wq >> 1, cb = wq & 1;
            const int64_t d = FUSED ? dblk * ST_DB + 64 * cb + lane : dblk * ST_DB + t;      // FUSED: the first of its two d rows
            const int64_t vword = 2 * dblk + cb;                                             // FUSED: word of a V row
            const uint64_t* vrow = FUSED ? Vt + b * N * Dp : Vt + (b * D + (d < D ? d : 0)) * wpn;
            auto load_bits = [&](int32_t kb, uint64_t (&w)[2]) {
                if (FUSED) {
                    const int64_t n = (int64_t)kb * ST_KB + 64 * rb + lane;
                    const bool live = kb < nkb && vword < Dp;
                    w[0] = (live && n < N) ? __ldg(vrow + n * Dp + vword) : 0ull;
                    w[1] = (live && n + 32 < N) ? __ldg(vrow + (n + 32) * Dp + vword) : 0ull;
                } else {
                    const int64_t w0 = 2 * (int64_t)kb;
                    w[0] = (kb < nkb && d < D && w0 < wpn) ? __ldg(vrow + w0) : 0ull;
                    w[1] = (kb < nkb && d < D && w0 + 1 < wpn) ? __ldg(vrow + w0 + 1) : 0ull;
                }
            };
            // the packed words are fetched ST_VPF k-blocks ahead (a ring of registers): one ahead
            // leaves the load latency on the path of every k-block
            constexpr int ST_VPF = 4;
            uint64_t ring[ST_VPF][2];
#pragma unroll
            for (int u = 0; u < ST_VPF - 1; ++u) load_bits(u, ring[u]);
            for (int32_t kb0 = 0; kb0 < nkb && ok; kb0 += ST_VPF) {
#pragma unroll
                for (int u = 0; u < ST_VPF; ++u) {            // ring slots are static register names
                    const int32_t kb = kb0 + u;
                    if (kb >= nkb || !ok) break;
                    load_bits(kb + ST_VPF - 1, ring[(u + ST_VPF - 1) % ST_VPF]);
                    const int sb = (int)(g % ST_BSTAGES);
                    ok = __all_sync(0xffffffffu, mbar_wait(b_empty(sb), ((g / ST_BSTAGES) & 1u) ^ 1u, abort_flag, 24));
                    if (!ok) break;
                    ++g;
                    if (FUSED) {
                        uint64_t lo = ring[u][0], hi = ring[u][1];
                        transpose64x64(lo, hi, lane);         // lo: d row 64 cb + lane, hi: + 32; bit j = n0 + 64 rb + j
                        if (d >= D) lo = 0ull;
                        if (d + 32 >= D) hi = 0ull;
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int r = 64 * cb + lane + 32 * h;
                            const uint64_t bitsr = h ? hi : lo;
                            uint8_t* row = gb + sb * ST_B_TILE + r * 128;
#pragma unroll
                            for (int c = 0; c < 4; ++c) {     // chunk 4 rb + c of the row: its 16 bits 16 c .. 16 c + 15
                                const uint32_t w32 = (uint32_t)(bitsr >> (16 * c));
                                *reinterpret_cast<uint4*>(row + (((4 * rb + c) ^ (r & 7)) << 4)) =
                                    make_uint4(st_bits4_to_bytes(w32, 0), st_bits4_to_bytes(w32, 4), st_bits4_to_bytes(w32, 8), st_bits4_to_bytes(w32, 12));
                            }
                        }
                    } else {
                        const uint64_t (&cur)[2] = ring[u];
                        uint8_t* row = gb + sb * ST_B_TILE + t * 128;
#pragma unroll
                        for (int c = 0; c < 8; ++c) {         // chunk c: bytes 16c .. 16c+15 = bits 16c .. 16c+15
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
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(acc_full, n_items & 1u, abort_flag, 25));
            if (!ok) break;
            tc_fence_after();
            const int64_t m = m0 + quarter * 32 + lane;
            const int32_t S = (int32_t)tc_ld1(lane_base + ST_DB);
            uint32_t bits[4];
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tc_ld32(lane_base + 32 * c, v);
                tc_wait_ld();
                if (c == 3) {                                 // the accumulator is in registers: hand it back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty);
                }
                uint32_t w = 0;
#pragma unroll
                for (int j = 0; j < 32; ++j) w |= (2 * (int32_t)v[j] - S >= 0 ? 1u : 0u) << j;
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
