// Layout kernels on packed words: bit-matrix transpose and OR/AND over a non-packed axis.
//
// transpose_bits: in [batch, R, ceil(C/64)] -> out [batch, C, ceil(R/64)], out bit (c, r) = in bit
// (r, c). A 64 x 64 bit block is transposed in registers by the butterfly (swap the off-diagonal
// 32 x 32 quadrants, then 16 x 16 inside each, ... down to 1 x 1): lane L holds rows L and L + 32
// of the block, the first round is inside the lane and the other five exchange with lane L ^ j
// through shuffles, about a hundred instructions per 64 x 64 block instead of 4096 single-bit moves. A CTA
// of 8 warps owns a 512 x 512 bit tile; warp w transposes the eight blocks of row-block w, and the
// transposed words go through shared memory so that every input and output row of the tile is one
// contiguous 64-byte run. HBM bound: 2 * R * C / 8 bytes.
//
// reduce_rows: in [outer, R, inner] words -> out [outer, inner] words, OR or AND over R. Rows of
// whole 16-byte vectors: one launch, no preset, no atomics (k_reduce_rows_slab: a CTA owns a
// 512-byte slab of the rows, the rows are split over a thread-block cluster and merged through
// distributed shared memory). Other rows: one thread per inner word, R cut into chunks across
// blockIdx.y, partial results merged with 64-bit atomics into an output that the launcher presets.
#include "tcgen05_common.cuh"

namespace bb {

constexpr int TB_TILE = 512;            // bits per tile side = 8 blocks of 64: 64-byte runs on both sides
constexpr int TB_BLOCKS = TB_TILE / 64;
constexpr int TB_THREADS = 32 * TB_BLOCKS;
constexpr int TB_PITCH = TB_BLOCKS + 1; // words per staged output row (+1 pad: conflict-free 8-byte accesses)

__global__ void __launch_bounds__(TB_THREADS)
k_transpose_bits(const uint64_t* __restrict__ in, uint64_t* __restrict__ out,
                 int64_t R, int64_t C, int64_t wpr_in, int64_t wpr_out, int64_t gx, int64_t gy, int64_t sgx) {
    __shared__ uint64_t stage[TB_TILE * TB_PITCH];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t b = blockIdx.y;
    // Tiles run in 8 x 8 groups: the CTAs that are resident together then read 512-byte runs of
    // the input rows and write 512-byte runs of the output rows between them, instead of one
    // 64-byte run per DRAM page.
    const int64_t grp = (int64_t)blockIdx.x >> 6;
    const int in_grp = (int)(blockIdx.x & 63);
    // sgx = 0: a matrix with fewer than 8 tiles along a side gets one CTA per tile, in row-major order
    const int64_t tx = sgx ? (grp % sgx) * 8 + (in_grp & 7) : (int64_t)blockIdx.x % gx;
    const int64_t ty = sgx ? (grp / sgx) * 8 + (in_grp >> 3) : (int64_t)blockIdx.x / gx;
    if (tx >= gx || ty >= gy) return;
    const int64_t r0 = ty * TB_TILE;                               // first input row of the tile
    const int64_t cw0 = tx * TB_BLOCKS;                            // first input word (column block) of the tile
    const uint64_t* inb = in + b * R * wpr_in;
    uint64_t* outb = out + b * C * wpr_out;

    // warp w: rows [r0 + 64 w, +64) of the tile, all TB_BLOCKS column blocks; lane L: rows L and L + 32
    uint64_t lo[TB_BLOCKS], hi[TB_BLOCKS];
    {
        const int64_t ra = r0 + 64 * warp + lane, rb = ra + 32;
        const uint64_t* pa = inb + ra * wpr_in + cw0;
        const uint64_t* pb = inb + rb * wpr_in + cw0;
        const bool full = cw0 + TB_BLOCKS <= wpr_in && (wpr_in & 1) == 0 && (reinterpret_cast<uintptr_t>(inb) & 15u) == 0;
        if (full && rb < R) {
#pragma unroll
            for (int cb = 0; cb < TB_BLOCKS; cb += 2) {
                const uint4 va = ldg_stream(pa + cb), vb = ldg_stream(pb + cb);
                lo[cb] = (uint64_t)va.x | ((uint64_t)va.y << 32); lo[cb + 1] = (uint64_t)va.z | ((uint64_t)va.w << 32);
                hi[cb] = (uint64_t)vb.x | ((uint64_t)vb.y << 32); hi[cb + 1] = (uint64_t)vb.z | ((uint64_t)vb.w << 32);
            }
        } else {
#pragma unroll
            for (int cb = 0; cb < TB_BLOCKS; ++cb) {
                const bool okw = cw0 + cb < wpr_in;
                lo[cb] = (ra < R && okw) ? __ldg(pa + cb) : 0ull;
                hi[cb] = (rb < R && okw) ? __ldg(pb + cb) : 0ull;
            }
        }
    }
#pragma unroll
    for (int cb = 0; cb < TB_BLOCKS; ++cb) {
        transpose64x64(lo[cb], hi[cb], lane);
        stage[(64 * cb + lane) * TB_PITCH + warp] = lo[cb];
        stage[(64 * cb + 32 + lane) * TB_PITCH + warp] = hi[cb];
    }
    __syncthreads();
    const int64_t ow0 = ty * TB_BLOCKS;                             // first output word of the tile's rows
#pragma unroll
    for (int k = 0; k < TB_TILE / TB_THREADS; ++k) {
        const int orow = tid + TB_THREADS * k;
        const int64_t c = cw0 * 64 + orow;                          // output row = input bit column
        if (c >= C) continue;
        uint64_t* dst = outb + c * wpr_out + ow0;
        const uint64_t* src = stage + orow * TB_PITCH;
        if (ow0 + TB_BLOCKS <= wpr_out && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
            for (int w = 0; w < TB_BLOCKS; w += 2)
                stg_stream(dst + w, make_uint4((uint32_t)src[w], (uint32_t)(src[w] >> 32), (uint32_t)src[w + 1], (uint32_t)(src[w + 1] >> 32)));
        } else {
#pragma unroll
            for (int w = 0; w < TB_BLOCKS; ++w) if (ow0 + w < wpr_out) dst[w] = src[w];
        }
    }
}

// The same tile through TMA: strided 64-byte rows are what the bulk tensor copies are for. With
// plain loads a warp touches 32 different 128-byte lines per instruction and the load/store unit,
// not HBM, sets the pace (about 2 TB/s). Here one thread issues two [256 rows x 64 bytes] box loads,
// the warps read their rows from SWIZZLE_64B shared memory without bank conflicts, and the transposed
// tile leaves as two box stores; rows and words past the edges are zero filled on the way in and
// clipped on the way out, so there is no edge code. Needs 16-byte row pitches on both sides.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* tm, uint32_t src, int32_t c0, int32_t c1, int32_t c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 :: "l"(tm), "r"(src), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

constexpr int TB_TMA_SMEM = TB_TILE * 64 + 64 + 1024;     // ONE tile buffer: the transposed tile is staged over the input

__global__ void __launch_bounds__(TB_THREADS)
k_transpose_bits_tma(const __grid_constant__ CUtensorMap tmIn, const __grid_constant__ CUtensorMap tmOut,
                     int64_t gx, int64_t gy, int64_t sgx) {
    extern __shared__ uint8_t tb_smem_raw[];
    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(tb_smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    // The whole tile is in registers before anything is staged, so the output reuses the input's
    // 32 KB (one barrier in between): half the shared memory, twice the CTAs per SM to overlap the
    // load, butterfly and store phases of different tiles.
    const uint32_t in_s = base, out_s = base, bar = base + TB_TILE * 64;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tb_smem_raw + (base - raw) + TB_TILE * 64 + 8);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t b = blockIdx.y;
    const int64_t grp = (int64_t)blockIdx.x >> 6;
    const int in_grp = (int)(blockIdx.x & 63);
    // sgx = 0: a matrix with fewer than 8 tiles along a side gets one CTA per tile, in row-major order
    const int64_t tx = sgx ? (grp % sgx) * 8 + (in_grp & 7) : (int64_t)blockIdx.x % gx;
    const int64_t ty = sgx ? (grp / sgx) * 8 + (in_grp >> 3) : (int64_t)blockIdx.x / gx;
    if (tx >= gx || ty >= gy) return;

    if (tid == 0) {
        mbar_init(bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async_smem();
        mbar_expect_tx(bar, TB_TILE * 64);
        tma_load_3d(in_s, &tmIn, (int32_t)(tx * TB_BLOCKS), (int32_t)(ty * TB_TILE), (int32_t)b, bar);
        tma_load_3d(in_s + 256 * 64, &tmIn, (int32_t)(tx * TB_BLOCKS), (int32_t)(ty * TB_TILE + 256), (int32_t)b, bar);
    }
    __syncthreads();
    const bool ok = __all_sync(0xffffffffu, mbar_wait(bar, 0, abort_flag, 31));
    // shared-memory row = 64 bytes = 4 chunks of 16; chunk c of row r sits at c ^ ((r >> 1) & 3)
    uint64_t lo[TB_BLOCKS], hi[TB_BLOCKS];
    {
        const int ra = 64 * warp + lane, rb = ra + 32;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint4 va, vb;
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(va.x), "=r"(va.y), "=r"(va.z), "=r"(va.w)
                         : "r"(in_s + (uint32_t)(ra * 64 + ((c ^ ((ra >> 1) & 3)) << 4))) : "memory");
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(vb.x), "=r"(vb.y), "=r"(vb.z), "=r"(vb.w)
                         : "r"(in_s + (uint32_t)(rb * 64 + ((c ^ ((rb >> 1) & 3)) << 4))) : "memory");
            lo[2 * c] = (uint64_t)va.x | ((uint64_t)va.y << 32); lo[2 * c + 1] = (uint64_t)va.z | ((uint64_t)va.w << 32);
            hi[2 * c] = (uint64_t)vb.x | ((uint64_t)vb.y << 32); hi[2 * c + 1] = (uint64_t)vb.z | ((uint64_t)vb.w << 32);
        }
    }
    __syncthreads();                 // every warp has read its rows: the buffer may be overwritten
#pragma unroll
    for (int cb = 0; cb < TB_BLOCKS; ++cb) {
        transpose64x64(lo[cb], hi[cb], lane);
        // output tile row = input bit column; word `warp` of that row
        const int oa = 64 * cb + lane, ob = oa + 32;
        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" :: "r"(out_s + (uint32_t)(oa * 64 + (((warp >> 1) ^ ((oa >> 1) & 3)) << 4) + (warp & 1) * 8)),
                     "r"((uint32_t)lo[cb]), "r"((uint32_t)(lo[cb] >> 32)) : "memory");
        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" :: "r"(out_s + (uint32_t)(ob * 64 + (((warp >> 1) ^ ((ob >> 1) & 3)) << 4) + (warp & 1) * 8)),
                     "r"((uint32_t)hi[cb]), "r"((uint32_t)(hi[cb] >> 32)) : "memory");
    }
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0 && ok) {
        tma_store_3d(&tmOut, out_s, (int32_t)(ty * TB_BLOCKS), (int32_t)(tx * TB_TILE), (int32_t)b);
        tma_store_3d(&tmOut, out_s + 256 * 64, (int32_t)(ty * TB_BLOCKS), (int32_t)(tx * TB_TILE + 256), (int32_t)b);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");      // the tile must outlive the stores' reads
    }
}

// packed words [batch, rows, wpr] as a 3-D tensor of 8-byte elements, box = [8 words, 256 rows, 1], SWIZZLE_64B
static bool tb_make_map(CUtensorMap* tm, const uint64_t* p, int64_t batch, int64_t rows, int64_t wpr) {
    PFN_tmapEncodeTiled enc = tc5_encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)wpr, (cuuint64_t)rows, (cuuint64_t)batch};
    const cuuint64_t strides[2] = {(cuuint64_t)wpr * 8u, (cuuint64_t)(rows * wpr) * 8u};
    const cuuint32_t box[3] = {(cuuint32_t)TB_BLOCKS, 256u, 1u};
    const cuuint32_t estr[3] = {1, 1, 1};
    return enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, const_cast<uint64_t*>(p), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool IS_OR>
__global__ void __launch_bounds__(256)
k_reduce_rows(const uint64_t* __restrict__ in, unsigned long long* __restrict__ out,
              int64_t R, int64_t inner, int64_t rows_per_chunk) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= inner) return;
    const int64_t o = blockIdx.z;
    const int64_t ra = (int64_t)blockIdx.y * rows_per_chunk;
    const int64_t rb = ra + rows_per_chunk < R ? ra + rows_per_chunk : R;
    const uint64_t* p = in + (o * R + ra) * inner + i;
    uint64_t acc = IS_OR ? 0ull : ~0ull;
    int64_t r = ra;
    for (; r + 4 <= rb; r += 4, p += 4 * inner) {         // four independent loads in flight
        const uint64_t a = __ldg(p), b = __ldg(p + inner), c = __ldg(p + 2 * inner), d = __ldg(p + 3 * inner);
        acc = IS_OR ? (acc | a | b | c | d) : (acc & a & b & c & d);
    }
    for (; r < rb; ++r, p += inner) acc = IS_OR ? (acc | __ldg(p)) : (acc & __ldg(p));
    if (IS_OR) { if (acc != 0ull) atomicOr(out + o * inner + i, acc); }
    else       { if (acc != ~0ull) atomicAnd(out + o * inner + i, acc); }
}

// The same reduction without the preset and without atomics, for rows of whole 16-byte vectors. A
// CTA owns a slab of 64 words (512 contiguous bytes of every row) and a share of the rows: its 256
// threads are 32 column threads (one 16-byte vector each) times 8 row lanes, every thread keeps four
// loads in flight, the row lanes meet in shared memory (narrower slabs, 16 column threads times 16
// row lanes, when there are few of them). When the slabs alone do not fill the GPU
// the rows are split over the 2, 4 or 8 CTAs of a thread-block CLUSTER and the CTAs' partial slabs
// meet through distributed shared memory: rank 0 reads its peers' partials and stores the slab.
constexpr int RR_THREADS = 256;

__device__ __forceinline__ uint32_t rr_cluster_rank() {
    uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r;
}
__device__ __forceinline__ uint32_t rr_cluster_size() {
    uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r;
}
__device__ __forceinline__ void rr_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <bool IS_OR, int RR_COLS>
__global__ void __launch_bounds__(RR_THREADS)
k_reduce_rows_slab(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, int64_t R, int64_t inner) {
    constexpr int RR_LANES = RR_THREADS / RR_COLS, RR_SLAB = 2 * RR_COLS;      // row lanes; words per slab
    __shared__ __align__(16) uint64_t part[RR_LANES][RR_SLAB];
    const int col = threadIdx.x % RR_COLS, rl = threadIdx.x / RR_COLS;
    const uint32_t crank = rr_cluster_rank(), csize = rr_cluster_size();      // cluster spans blockIdx.y
    const int64_t o = blockIdx.z;
    const int64_t w = (int64_t)blockIdx.x * RR_SLAB + 2 * col;                // first word of this thread's vector
    const bool live = w < inner;                                              // inner is even: both words or none
    // rows of this CTA: an equal share of R
    const int64_t per = R / csize, extra = R % csize;
    const int64_t ra = crank * per + (crank < extra ? crank : extra);
    const int64_t rb = ra + per + (crank < extra ? 1 : 0);
    const uint64_t ident = IS_OR ? 0ull : ~0ull;
    uint64_t a0 = ident, a1 = ident;
    if (live) {
        const uint64_t* p = in + (o * R + ra + rl) * inner + w;
        const int64_t step = (int64_t)RR_LANES * inner;
        int64_t r = ra + rl;
        for (; r + 7 * RR_LANES < rb; r += 8 * RR_LANES, p += 8 * step) {      // eight independent loads in flight
            uint4 v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = ldg_stream(p + k * step);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint64_t x = ((uint64_t)v[k].y << 32) | v[k].x, y = ((uint64_t)v[k].w << 32) | v[k].z;
                a0 = IS_OR ? (a0 | x) : (a0 & x);
                a1 = IS_OR ? (a1 | y) : (a1 & y);
            }
        }
        for (; r < rb; r += RR_LANES, p += step) {
            const uint4 v = ldg_stream(p);
            const uint64_t x = ((uint64_t)v.y << 32) | v.x, y = ((uint64_t)v.w << 32) | v.z;
            a0 = IS_OR ? (a0 | x) : (a0 & x);
            a1 = IS_OR ? (a1 | y) : (a1 & y);
        }
    }
    part[rl][2 * col] = a0;
    part[rl][2 * col + 1] = a1;
    __syncthreads();
    if (rl == 0) {
#pragma unroll
        for (int k = 1; k < RR_LANES; ++k) {
            a0 = IS_OR ? (a0 | part[k][2 * col]) : (a0 & part[k][2 * col]);
            a1 = IS_OR ? (a1 | part[k][2 * col + 1]) : (a1 & part[k][2 * col + 1]);
        }
        part[0][2 * col] = a0;
        part[0][2 * col + 1] = a1;
    }
    if (csize > 1) {
        rr_cluster_sync();                      // every CTA's part[0] is complete and visible to the cluster
        if (crank == 0 && rl == 0) {
            const uint32_t mine = (uint32_t)__cvta_generic_to_shared(&part[0][2 * col]);
            for (uint32_t k = 1; k < csize; ++k) {
                uint32_t remote;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(mine), "r"(k));
                uint64_t b0, b1;
                asm volatile("ld.shared::cluster.v2.u64 {%0, %1}, [%2];" : "=l"(b0), "=l"(b1) : "r"(remote) : "memory");
                a0 = IS_OR ? (a0 | b0) : (a0 & b0);
                a1 = IS_OR ? (a1 | b1) : (a1 & b1);
            }
        }
        rr_cluster_sync();                      // peers keep their shared memory alive until rank 0 has read it
    }
    if (crank == 0 && rl == 0 && live)
        stg_stream(out + o * inner + w, make_uint4((uint32_t)a0, (uint32_t)(a0 >> 32), (uint32_t)a1, (uint32_t)(a1 >> 32)));
}

// ---------------------------------------------------------------------------
// Moves along the packed axis, in the packed domain.
//
// flip and roll: every output word is a 64-bit WINDOW of the input row at some bit offset (for
// flip the window is then bit-reversed), so one thread makes one output word from at most two
// (roll across the end of the row: three) input words. HBM bound, 2 * n / 8 bytes.
// gather (index_select on the last axis): the source bit of every output bit comes from an index
// vector, so a warp builds 1024 output bits with 32 ballots: lane l looks up the bit for position
// 32 t + l in round t and keeps the ballot of round t == l.

// bits [p, p + 64) of a row of n bits stored in `row` (wpr words); positions outside [0, n) read as 0
__device__ __forceinline__ uint64_t row_window(const uint64_t* __restrict__ row, int64_t wpr, int64_t n, int64_t p) {
    if (p >= n || p <= -64) return 0ull;
    const int64_t w = p >> 6;                  // floor division: p may be negative
    const int sh = (int)(p & 63);
    const uint64_t lo = (w >= 0 && w < wpr) ? __ldg(row + w) : 0ull;
    uint64_t v = lo >> sh;
    if (sh != 0) {
        const uint64_t hi = (w + 1 >= 0 && w + 1 < wpr) ? __ldg(row + w + 1) : 0ull;
        v |= hi << (64 - sh);
    }
    return v;                                  // pad bits of the input are 0, so nothing past n leaks in
}

template <bool FLIP>
__global__ void __launch_bounds__(256)
k_flip_roll_bits(const uint64_t* __restrict__ in, uint64_t* __restrict__ out,
                 int64_t rows, int64_t n, int64_t wpr, int64_t shift /* roll: 0 <= shift < n */) {
    const int64_t total = rows * wpr;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / wpr, w = i - r * wpr;
        const uint64_t* row = in + r * wpr;
        uint64_t v;
        if (FLIP) {
            // out bit j = in bit n - 1 - j: output bits [64 w, 64 w + 64) are the window that ENDS at n - 64 w, reversed
            v = __brevll(row_window(row, wpr, n, n - 64 * (w + 1)));
        } else {
            // out bit j = in bit (j - shift) mod n
            int64_t p = 64 * w - shift;
            if (p < 0) p += n;                                       // -n < 64 w - shift, since shift < n
            v = row_window(row, wpr, n, p);
            if (p + 64 > n) v |= row_window(row, wpr, n, p - n);     // the window runs over the end: wrap to bit 0
        }
        const int64_t valid = n - 64 * w;
        if (valid < 64) v &= (1ull << valid) - 1ull;
        out[i] = v;
    }
}

// bits [s, s + 64) of the 128-bit little-endian value (lo, hi), 0 <= s < 64
__device__ __forceinline__ uint64_t funnel64(uint64_t lo, uint64_t hi, int s) {
    return s ? (lo >> s) | (hi << (64 - s)) : lo;
}

// The same two moves for rows of whole 16-byte vectors (wpr even, 16-byte aligned bases): a warp
// makes 128 consecutive output words of one row per task, a lane four of them (32 bytes). Every lane
// loads TWO aligned 16-byte vectors of the input, takes the first vector of its neighbour through
// shuffles, cuts its eight 32-bit output words out of those twelve input words with 32-bit funnel
// shifts (the word offset is the same for the whole warp) and stores two 16-byte vectors. A task
// whose window runs over an end of the row (the wrap of a roll, the ragged last words) takes the
// word-by-word form. Index arithmetic is 32-bit: the launcher checks that it fits.
template <bool FLIP>
__device__ __forceinline__ void fr_words_slow(const uint64_t* __restrict__ row, uint64_t* __restrict__ orow,
                                              int64_t n, int64_t wpr, int64_t shift, int64_t W) {
    uint64_t v[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int64_t w = W + k;
        if (FLIP) {
            v[k] = __brevll(row_window(row, wpr, n, n - 64 * (w + 1)));
        } else {
            int64_t p = 64 * w - shift;
            if (p < 0) p += n;
            v[k] = row_window(row, wpr, n, p);
            if (p + 64 > n) v[k] |= row_window(row, wpr, n, p - n);
        }
        const int64_t valid = n - 64 * w;
        if (valid < 64) v[k] = valid > 0 ? (v[k] & ((1ull << valid) - 1ull)) : 0ull;
    }
    stg_stream(orow + W, make_uint4((uint32_t)v[0], (uint32_t)(v[0] >> 32), (uint32_t)v[1], (uint32_t)(v[1] >> 32)));
}

// y[j] = bits [32 (K + j) + s, 32 (K + j) + s + 32) of the little-endian word array x, j < 8
template <int K>
__device__ __forceinline__ void fr_cut(const uint32_t (&x)[12], uint32_t s, uint32_t (&y)[8]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = __funnelshift_r(x[K + j], x[K + j + 1], s);
}

template <bool FLIP>
__global__ void __launch_bounds__(256, 6)
k_flip_roll_vec(const uint64_t* __restrict__ in, uint64_t* __restrict__ out,
                uint32_t tasks, uint32_t chunks_per_row, int64_t n, int64_t wpr, int64_t shift) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t nwarps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t t = warp; t < tasks; t += nwarps) {
        const uint32_t r = t / chunks_per_row;
        const int64_t W0 = (int64_t)(t - r * chunks_per_row) * 128;             // first output word of the task
        const int64_t cw = (wpr - W0) < 128 ? (wpr - W0) : 128;                 // output words of the task
        const uint64_t* row = in + (int64_t)r * wpr;
        uint64_t* orow = out + (int64_t)r * wpr;
        const int64_t W = W0 + 4 * lane;                                        // this lane's four output words
        bool fast;
        int64_t start;                                                          // first input bit this lane reads
        if (FLIP) {
            fast = n - 64 * (W0 + cw) >= 0;                                     // the window of the task's last word
            start = n - 64 * (W + 4);
        } else {
            int64_t P = (64 * W0 - shift) % n;
            if (P < 0) P += n;
            fast = P + 64 * cw <= n;
            start = P + 256 * lane;
        }
        if (!fast) {                                                            // warp-uniform
            if (W < wpr) fr_words_slow<FLIP>(row, orow, n, wpr, shift, W);
            if (W + 2 < wpr) fr_words_slow<FLIP>(row, orow, n, wpr, shift, W + 2);
            continue;
        }
        const int64_t q = start >> 6;                                           // word that holds the first bit
        const int64_t qa = q & ~1ll;
        uint32_t x[12];
        {
            uint4 a = make_uint4(0, 0, 0, 0), b = a, c = a;
            if (qa >= 0 && qa < wpr) a = ldg_stream(row + qa);
            if (qa + 2 >= 0 && qa + 2 < wpr) b = ldg_stream(row + qa + 2);
            // the vector after these two is the first vector of a neighbour, except at the end of the warp
            const bool edge = FLIP ? (lane == 0) : (lane == 31);
            if (edge && qa + 4 >= 0 && qa + 4 < wpr) c = ldg_stream(row + qa + 4);
            uint4 nb;
            if (FLIP) {
                nb.x = __shfl_up_sync(0xffffffffu, a.x, 1); nb.y = __shfl_up_sync(0xffffffffu, a.y, 1);
                nb.z = __shfl_up_sync(0xffffffffu, a.z, 1); nb.w = __shfl_up_sync(0xffffffffu, a.w, 1);
            } else {
                nb.x = __shfl_down_sync(0xffffffffu, a.x, 1); nb.y = __shfl_down_sync(0xffffffffu, a.y, 1);
                nb.z = __shfl_down_sync(0xffffffffu, a.z, 1); nb.w = __shfl_down_sync(0xffffffffu, a.w, 1);
            }
            if (!edge) c = nb;
            x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
            x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
            x[8] = c.x; x[9] = c.y; x[10] = c.z; x[11] = c.w;
        }
        if (W >= wpr) continue;
        // bit offset of the window inside x: 64 (q odd) + start mod 64, the same for every lane
        const uint32_t o = (uint32_t)(start & 63) + ((q & 1) ? 64u : 0u);
        const uint32_t s5 = o & 31u;
        uint32_t y[8];
        switch (o >> 5) {
            case 0: fr_cut<0>(x, s5, y); break;
            case 1: fr_cut<1>(x, s5, y); break;
            case 2: fr_cut<2>(x, s5, y); break;
            default: fr_cut<3>(x, s5, y); break;
        }
        uint4 lo4, hi4;                                                         // output words (W, W+1) and (W+2, W+3)
        if (FLIP) {
            lo4 = make_uint4(__brev(y[7]), __brev(y[6]), __brev(y[5]), __brev(y[4]));
            hi4 = make_uint4(__brev(y[3]), __brev(y[2]), __brev(y[1]), __brev(y[0]));
        } else {
            lo4 = make_uint4(y[0], y[1], y[2], y[3]);
            hi4 = make_uint4(y[4], y[5], y[6], y[7]);
        }
        // the last word of a ragged row keeps its pad bits 0 (a roll fills it from anywhere in the ring)
        const int64_t last = wpr - 1 - W;                                       // which of the four is the row's last word
        if ((n & 63) && last >= 0 && last < 4) {
            const uint64_t m = (1ull << (n & 63)) - 1ull;
            const uint32_t m0 = (uint32_t)m, m1 = (uint32_t)(m >> 32);
            if (last == 0)      { lo4.x &= m0; lo4.y &= m1; }
            else if (last == 1) { lo4.z &= m0; lo4.w &= m1; }
            else if (last == 2) { hi4.x &= m0; hi4.y &= m1; }
            else                { hi4.z &= m0; hi4.w &= m1; }
        }
        stg_stream(orow + W, lo4);
        if (W + 2 < wpr) stg_stream(orow + W + 2, hi4);
    }
}

__global__ void __launch_bounds__(256)
k_gather_bits(const uint64_t* __restrict__ in, const int64_t* __restrict__ idx, uint32_t* __restrict__ out32,
              int64_t rows, int64_t n_in, int64_t n_out, int64_t wpr_in, int64_t wpr_out, int64_t chunks_per_row) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t task = warp; task < rows * chunks_per_row; task += nwarps) {
        const int64_t r = task / chunks_per_row, c = task - r * chunks_per_row;
        const uint64_t* row = in + r * wpr_in;
        uint32_t mine = 0;
#pragma unroll 4
        for (int t = 0; t < 32; ++t) {
            const int64_t j = c * 1024 + t * 32 + lane;
            uint32_t bit = 0;
            if (j < n_out) {
                const int64_t s = __ldg(idx + j);
                if (s >= 0 && s < n_in) bit = (uint32_t)(__ldg(row + (s >> 6)) >> (s & 63)) & 1u;   // out of range reads as 0
            }
            const uint32_t word = __ballot_sync(0xffffffffu, bit);
            if (lane == t) mine = word;
        }
        const int64_t w32 = c * 32 + lane;                     // 32-bit word index inside the output row
        if (w32 < 2 * wpr_out) out32[r * 2 * wpr_out + w32] = mine;
    }
}

// scatter (x[..., idx] = value, index_copy_ / index_fill_ along the last axis): thread (j, row)
// writes ONE bit, position idx[j] of its row, with a word-wide atomic (several positions may share
// a word). The source bit is bit j of the row of `src`, or the constant `value` when src is null.
// A thread keeps its j (and idx[j]) and walks the rows.
__global__ void __launch_bounds__(256)
k_scatter_bits(unsigned long long* __restrict__ packed, const int64_t* __restrict__ idx,
               const uint64_t* __restrict__ src, int value,
               int64_t rows, int64_t n, int64_t n_idx, int64_t wpr, int64_t wpr_src) {
    const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n_idx) return;
    const int64_t s = __ldg(idx + j);
    if (s < 0 || s >= n) return;                              // out of range: the caller has checked; write nothing
    const unsigned long long bit = 1ull << (s & 63);
    const int64_t w = s >> 6, ws = j >> 6;
    const int sb = (int)(j & 63);
    for (int64_t r = blockIdx.y; r < rows; r += gridDim.y) {
        const int on = src ? (int)((__ldg(src + r * wpr_src + ws) >> sb) & 1ull) : value;
        if (on) atomicOr(packed + r * wpr + w, bit);
        else    atomicAnd(packed + r * wpr + w, ~bit);
    }
}

}  // namespace bb

namespace bb { int ly_status_bridge() { return tc5_device_status(); } }

using namespace bb;

extern "C" int brute_b200_transpose_bits(const uint64_t* in, uint64_t* out,
                                         int64_t batch, int64_t R, int64_t C, void* stream) {
    BB_REQUIRE(batch >= 0 && R >= 0 && C >= 0, BRUTE_ERR_INVALID_ARG);
    if (batch == 0 || C == 0) return BRUTE_OK;
    const int64_t wpr_in = (C + 63) / 64, wpr_out = (R + 63) / 64;
    if (R == 0) return BRUTE_OK;                           // output rows have no words
    BB_REQUIRE(in != nullptr && out != nullptr && in != out, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(in) && aligned8(out), BRUTE_ERR_MISALIGNED);
    const int64_t gx = (wpr_in + TB_BLOCKS - 1) / TB_BLOCKS, gy = (R + TB_TILE - 1) / TB_TILE;
    // 8 x 8 groups of tiles for DRAM locality; a narrow or short matrix (many small ones in a batch,
    // as signed_bundle's V) would launch mostly empty groups, so it gets exactly its tiles
    const bool grouped = gx >= 8 && gy >= 8;
    const int64_t sgx = grouped ? (gx + 7) / 8 : 0, sgy = (gy + 7) / 8;
    const int64_t ctas = grouped ? sgx * sgy * 64 : gx * gy;
    BB_REQUIRE(ctas <= 0x7fffffffll && batch <= 65535, BRUTE_ERR_UNSUPPORTED);
    const dim3 grid((unsigned)ctas, (unsigned)batch);
    // TMA wants 16-byte aligned bases and row (and batch) pitches, and 32-bit coordinates
    if ((wpr_in & 1) == 0 && (wpr_out & 1) == 0 && aligned16(in) && aligned16(out) &&
        R < (1ll << 31) - TB_TILE && C < (1ll << 31) - TB_TILE) {
        CUtensorMap tmIn, tmOut;
        if (tb_make_map(&tmIn, in, batch, R, wpr_in) && tb_make_map(&tmOut, out, batch, C, wpr_out)) {
            if (!kernel_smem_ready<k_transpose_bits_tma>(TB_TMA_SMEM)) return BRUTE_ERR_LAUNCH;
            k_transpose_bits_tma<<<grid, TB_THREADS, TB_TMA_SMEM, as_stream(stream)>>>(tmIn, tmOut, gx, gy, sgx);
            return launch_status();
        }
    }
    k_transpose_bits<<<grid, TB_THREADS, 0, as_stream(stream)>>>(in, out, R, C, wpr_in, wpr_out, gx, gy, sgx);
    return launch_status();
}

extern "C" int brute_b200_reduce_rows(int op, const uint64_t* in, uint64_t* out,
                                      int64_t outer, int64_t R, int64_t inner, void* stream) {
    BB_REQUIRE(op == BRUTE_OP_OR || op == BRUTE_OP_AND, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(outer >= 0 && R >= 0 && inner >= 0, BRUTE_ERR_INVALID_ARG);
    if (outer == 0 || inner == 0) return BRUTE_OK;
    BB_REQUIRE(out != nullptr && (R == 0 || in != nullptr), BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(in) && aligned8(out), BRUTE_ERR_MISALIGNED);
    BB_REQUIRE(outer <= 65535, BRUTE_ERR_UNSUPPORTED);
    cudaStream_t st = as_stream(stream);
    if (R > 0 && (inner & 1) == 0 && aligned16(in) && aligned16(out)) {
        // whole 16-byte vectors: the slab kernel, rows split over a cluster when the slabs are few
        const bool narrow = ((inner + 63) / 64) * outer * 8 < 2 * (int64_t)kNumSMs;     // very few slabs: 256-byte ones
        const int slab = narrow ? 32 : 64;
        const int64_t slabs = (inner + slab - 1) / slab;
        BB_REQUIRE(slabs <= 0x7fffffffll, BRUTE_ERR_UNSUPPORTED);
        const int lanes = RR_THREADS / (slab / 2);
        int csize = 1;
        while (csize < 8 && slabs * outer * csize < 6 * (int64_t)kNumSMs && R / (2 * csize) >= 4 * lanes) csize *= 2;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)slabs, (unsigned)csize, (unsigned)outer);
        cfg.blockDim = dim3(RR_THREADS);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = (unsigned)csize;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e;
        if (narrow) e = (op == BRUTE_OP_OR) ? cudaLaunchKernelEx(&cfg, k_reduce_rows_slab<true, 16>, in, out, R, inner)
                                            : cudaLaunchKernelEx(&cfg, k_reduce_rows_slab<false, 16>, in, out, R, inner);
        else        e = (op == BRUTE_OP_OR) ? cudaLaunchKernelEx(&cfg, k_reduce_rows_slab<true, 32>, in, out, R, inner)
                                            : cudaLaunchKernelEx(&cfg, k_reduce_rows_slab<false, 32>, in, out, R, inner);
        return e == cudaSuccess ? launch_status() : BRUTE_ERR_LAUNCH;
    }
    // identity of the reduction; an empty axis leaves it (any -> 0, all -> ~0, as torch does)
    if (cudaMemsetAsync(out, op == BRUTE_OP_OR ? 0x00 : 0xFF, (size_t)(outer * inner) * 8, st) != cudaSuccess)
        return BRUTE_ERR_LAUNCH;
    if (R == 0) return BRUTE_OK;
    const int64_t gx = (inner + 255) / 256;
    BB_REQUIRE(gx <= 0x7fffffffll, BRUTE_ERR_UNSUPPORTED);
    // enough row chunks to put about 8 blocks on every SM, at least 16 rows each
    int64_t chunks = (8 * (int64_t)kNumSMs + gx * outer - 1) / (gx * outer);
    if (chunks > (R + 15) / 16) chunks = (R + 15) / 16;
    if (chunks < 1) chunks = 1;
    if (chunks > 65535) chunks = 65535;
    const int64_t rows_per_chunk = (R + chunks - 1) / chunks;
    const dim3 grid((unsigned)gx, (unsigned)((R + rows_per_chunk - 1) / rows_per_chunk), (unsigned)outer);
    if (op == BRUTE_OP_OR)
        k_reduce_rows<true><<<grid, 256, 0, st>>>(in, reinterpret_cast<unsigned long long*>(out), R, inner, rows_per_chunk);
    else
        k_reduce_rows<false><<<grid, 256, 0, st>>>(in, reinterpret_cast<unsigned long long*>(out), R, inner, rows_per_chunk);
    return launch_status();
}

extern "C" int brute_b200_flip_bits(const uint64_t* in, uint64_t* out, int64_t rows, int64_t n, void* stream) {
    BB_REQUIRE(rows >= 0 && n >= 0, BRUTE_ERR_INVALID_ARG);
    if (rows == 0 || n == 0) return BRUTE_OK;
    BB_REQUIRE(in != nullptr && out != nullptr && in != out, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(in) && aligned8(out), BRUTE_ERR_MISALIGNED);
    const int64_t wpr = (n + 63) / 64;
    const int64_t chunks = (wpr + 127) / 128;
    if ((wpr & 1) == 0 && wpr >= 64 && aligned16(in) && aligned16(out) && rows * chunks < (1ll << 31)) {
        k_flip_roll_vec<true><<<stream_grid(rows * chunks, 8, 6), 256, 0, as_stream(stream)>>>(
            in, out, (uint32_t)(rows * chunks), (uint32_t)chunks, n, wpr, 0);
        return launch_status();
    }
    k_flip_roll_bits<true><<<stream_grid(rows * wpr, 256, 8), 256, 0, as_stream(stream)>>>(in, out, rows, n, wpr, 0);
    return launch_status();
}

extern "C" int brute_b200_roll_bits(const uint64_t* in, uint64_t* out, int64_t rows, int64_t n, int64_t shift, void* stream) {
    BB_REQUIRE(rows >= 0 && n >= 0, BRUTE_ERR_INVALID_ARG);
    if (rows == 0 || n == 0) return BRUTE_OK;
    BB_REQUIRE(in != nullptr && out != nullptr && in != out, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(in) && aligned8(out), BRUTE_ERR_MISALIGNED);
    const int64_t wpr = (n + 63) / 64;
    int64_t s = shift % n;
    if (s < 0) s += n;
    const int64_t chunks = (wpr + 127) / 128;
    if ((wpr & 1) == 0 && wpr >= 64 && aligned16(in) && aligned16(out) && rows * chunks < (1ll << 31)) {
        k_flip_roll_vec<false><<<stream_grid(rows * chunks, 8, 6), 256, 0, as_stream(stream)>>>(
            in, out, (uint32_t)(rows * chunks), (uint32_t)chunks, n, wpr, s);
        return launch_status();
    }
    k_flip_roll_bits<false><<<stream_grid(rows * wpr, 256, 8), 256, 0, as_stream(stream)>>>(in, out, rows, n, wpr, s);
    return launch_status();
}

extern "C" int brute_b200_gather_bits(const uint64_t* in, const int64_t* idx, uint64_t* out,
                                      int64_t rows, int64_t n_in, int64_t n_out, void* stream) {
    BB_REQUIRE(rows >= 0 && n_in >= 0 && n_out >= 0, BRUTE_ERR_INVALID_ARG);
    if (rows == 0 || n_out == 0) return BRUTE_OK;
    BB_REQUIRE(out != nullptr && idx != nullptr && (n_in == 0 || in != nullptr) && in != out, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(in) && aligned8(out) && aligned8(idx), BRUTE_ERR_MISALIGNED);
    const int64_t wpr_in = (n_in + 63) / 64, wpr_out = (n_out + 63) / 64;
    const int64_t chunks = (n_out + 1023) / 1024;
    k_gather_bits<<<stream_grid(rows * chunks, 8, 8), 256, 0, as_stream(stream)>>>(
        in, idx, reinterpret_cast<uint32_t*>(out), rows, n_in, n_out, wpr_in, wpr_out, chunks);
    return launch_status();
}

extern "C" int brute_b200_scatter_bits(uint64_t* packed, const int64_t* idx, const uint64_t* src, int value,
                                       int64_t rows, int64_t n, int64_t n_idx, void* stream) {
    BB_REQUIRE(rows >= 0 && n >= 0 && n_idx >= 0, BRUTE_ERR_INVALID_ARG);
    if (rows == 0 || n == 0 || n_idx == 0) return BRUTE_OK;
    BB_REQUIRE(packed != nullptr && idx != nullptr && packed != src, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(packed) && aligned8(idx) && aligned8(src), BRUTE_ERR_MISALIGNED);
    const int64_t gx = (n_idx + 255) / 256;
    BB_REQUIRE(gx <= 0x7fffffffll, BRUTE_ERR_UNSUPPORTED);
    // enough row lanes to fill the SMs a few times over when the index vector is short
    int64_t gy = (8 * (int64_t)kNumSMs + gx - 1) / gx;
    if (gy > rows) gy = rows;
    if (gy > 65535) gy = 65535;
    const dim3 grid((unsigned)gx, (unsigned)gy);
    k_scatter_bits<<<grid, 256, 0, as_stream(stream)>>>(reinterpret_cast<unsigned long long*>(packed), idx, src,
                                                        value != 0, rows, n, n_idx, (n + 63) / 64, (n_idx + 63) / 64);
    return launch_status();
}
