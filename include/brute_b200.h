/*
 * brute_b200 — C ABI of the B200 (sm_100a) kernels behind the `brute.bit1` ops.
 *
 * Every entry point is a stateless launcher: it validates its arguments,
 * enqueues work on `stream` of the CURRENT device and returns immediately.
 * It never throws, never synchronises, never allocates device memory (scratch
 * is passed in by the caller) and never traps the GPU. The return value is
 * BRUTE_OK (0) or a negative BRUTE_ERR_* code; brute_b200_strerror() names it.
 *
 * Conventions shared by all entry points
 *   - bit1 data is packed 64 logical bits per uint64 word along the LAST
 *     dimension, LSB first, little endian; a row of `ld` bits occupies
 *     ceil(ld/64) words and its pad bits are always 0.
 *   - bit value 1 means +1, bit value 0 means -1.
 *   - all pointers are DEVICE pointers unless stated otherwise; `stream` is a
 *     cudaStream_t passed as void* so that this header stays plain C.
 *
 * Each declaration cites the reference (TheoCoombes/Brute) interface it
 * replaces as file:line within that project.
 */
#ifndef BRUTE_B200_H_
#define BRUTE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------ */
#define BRUTE_OK                 0
#define BRUTE_ERR_INVALID_ARG   -1   /* null pointer, negative size, bad enum     */
#define BRUTE_ERR_MISALIGNED    -2   /* pointer / pitch alignment rule violated   */
#define BRUTE_ERR_UNSUPPORTED   -3   /* shape or dtype outside what is built      */
#define BRUTE_ERR_LAUNCH        -4   /* cudaGetLastError() after launch != 0      */
#define BRUTE_ERR_WORKSPACE     -5   /* scratch buffer missing or too small       */
#define BRUTE_ERR_DEVICE_WAIT   -6   /* a bounded in-kernel wait gave up          */
#define BRUTE_ERR_DRIVER        -7   /* a CUDA driver entry point was unavailable */

/* ---- enums ------------------------------------------------------------- */
/* float -> bit threshold convention. The reference front end uses x > 0 for
 * `.to(bit1)` (brute/tensor.py:163-169) and x >= 0 for `randn(dtype=bit1)`
 * (brute/functional.py:131-133). NaN maps to 0 under both. */
#define BRUTE_SIGN_GT0  0
#define BRUTE_SIGN_GE0  1

/* source dtype of brute_b200_pack_sign */
#define BRUTE_DT_F32   0
#define BRUTE_DT_BF16  1
#define BRUTE_DT_F16   2

/* word-wise binary ops of brute_b200_bitwise */
#define BRUTE_OP_AND     0
#define BRUTE_OP_OR      1
#define BRUTE_OP_XOR     2
#define BRUTE_OP_XNOR    3   /* pad bits of each row's last word forced to 0 */
#define BRUTE_OP_ANDNOT  4   /* a & ~b                                       */

/* GEMM instruction path; AUTO picks the fastest one that accepts the shape */
#define BRUTE_GEMM_AUTO     0
#define BRUTE_GEMM_POPC     1   /* CUDA-core __popcll, register blocked, any shape */
#define BRUTE_GEMM_MMA_B1   2   /* legacy mma.sync m16n8k256 .b1 and.popc          */
#define BRUTE_GEMM_TCGEN05  3   /* tcgen05.mma kind::i8 on in-kernel expanded bits  */
#define BRUTE_GEMM_TCGEN05_PAIR 4 /* the same on cta_group::2: two SMs share a 256x256 tile; needs M > 128 */

/* ---- library ----------------------------------------------------------- */
const char* brute_b200_strerror(int code);
/* Bit mask of BRUTE_CAP_*; host only, no GPU needed. */
#define BRUTE_CAP_SM100A        1u
#define BRUTE_CAP_GEMM_POPC     2u
#define BRUTE_CAP_GEMM_MMA_B1   4u
#define BRUTE_CAP_GEMM_TCGEN05  8u
#define BRUTE_CAP_ATTENTION    16u
uint32_t brute_b200_query_caps(void);
/* Reads (device -> host, synchronising the device) and clears the device-side
 * status word that bounded in-kernel waits write when they give up. Returns
 * BRUTE_OK or BRUTE_ERR_DEVICE_WAIT. Meant for tests and diagnostics, not for
 * the per-call path. */
int brute_b200_device_status(void);
/* Self-test of the bounded waits (test and diagnostics entry point; no counterpart in the
 * reference, whose kernels have no in-kernel waits): launches one small kernel that waits on an
 * mbarrier nothing arrives at, with a limit of `limit_us` microseconds (1 .. 100000). The wait
 * gives up, the kernel returns, *gave_up_device (a device int) is set to 3 (1: the waiter saw the
 * timeout, +2: another warp saw the CTA's abort flag), and the next brute_b200_device_status()
 * reports BRUTE_ERR_DEVICE_WAIT once. `relaxed` picks the backing-off form of the wait. */
int brute_b200_selftest_bounded_wait(int64_t limit_us, int relaxed, int* gave_up_device, void* stream);

/* ---- pack / unpack ----------------------------------------------------- */
/* bool bytes [rows, ld] -> packed words [rows, ceil(ld/64)]; any nonzero byte
 * is 1; every output word is written in full (pad bits 0), so the output needs
 * no prior memset.
 * Replaces cbrute::cuda::pack_bool, cbrute/cuda/ops_cuda.cu:54-90 and
 * k_pack_bool_warp/_persistent, cbrute/cuda/kernels/packing.cuh:26-72. */
int brute_b200_pack_bool(const uint8_t* in, uint64_t* out,
                         int64_t rows, int64_t ld, void* stream);

/* float [rows, ld] -> packed words, bit = (x > 0) or (x >= 0) per `mode`,
 * in one pass (no 1-byte-per-element temporary).
 * Replaces the two-kernel path `_to_bool` + pack_bool, brute/tensor.py:163-177
 * and brute/functional.py:131-133. */
int brute_b200_pack_sign(const void* in, int dtype, uint64_t* out,
                         int64_t rows, int64_t ld, int mode, void* stream);

/* packed words [rows, ceil(ll/64)] -> bool bytes [rows, ll] (0/1).
 * Replaces cbrute::cuda::unpack_bool, cbrute/cuda/ops_cuda.cu:112-137 and
 * k_unpack_bool_warp/_persistent, cbrute/cuda/kernels/packing.cuh:76-94,116-143. */
int brute_b200_unpack_bool(const uint64_t* in, uint8_t* out,
                           int64_t rows, int64_t ll, void* stream);

/* packed words -> float32 (+1.0f for bit 1, -1.0f for bit 0); no limit on rows.
 * Replaces cbrute::cuda::unpack_bits, cbrute/cuda/ops_cuda.cu:93-109 and
 * k_unpack_pm1_warp, cbrute/cuda/kernels/packing.cuh:96-114. */
int brute_b200_unpack_pm1_f32(const uint64_t* in, float* out,
                              int64_t rows, int64_t ll, void* stream);

/* ---- popcount / hamming ------------------------------------------------ */
/* per-element popcount of n elements of elem_bytes in {1,2,4,8} -> int32.
 * Replaces cbrute::cuda::popcount, cbrute/cuda/ops_cuda.cu:244-280 and
 * k_popcnt_u8/u16/u32/u64, cbrute/cuda/kernels/popcount.cuh:22-41. */
int brute_b200_popcount_elems(const void* in, int32_t* out,
                              int64_t n, int elem_bytes, void* stream);

/* total popcount of n_bytes bytes -> *out (uint64; the call overwrites it, it need not be zero).
 * One launch: the blocks sum into one of 256 accumulators in static device memory (zero at
 * rest, handed out round robin) and the last block to finish moves the sum to *out. Two
 * totals may therefore not be in flight 256 launches apart on one device, and two captured
 * graphs that contain the same accumulator slot should not be replayed concurrently.
 * Replaces cbrute::cuda::packed_popcount, cbrute/cuda/ops_cuda.cu:283-304 and
 * k_packed_popcount_total/k_popcount_tail_byte, cbrute/cuda/kernels/popcount.cuh:75-98,129-136. */
int brute_b200_popcount_total(const void* in, int64_t n_bytes,
                              uint64_t* out, void* stream);

/* total popcount(a ^ b) over n_bytes bytes -> *out, no XOR temporary; one launch, same
 * accumulator scheme as brute_b200_popcount_total.
 * Replaces cbrute::cuda::bit1_hamming_total, cbrute/cuda/ops_cuda.cu:312-338 and
 * k_hamming_total/k_hamming_tail_byte, cbrute/cuda/kernels/popcount.cuh:101-124,138-149. */
int brute_b200_hamming_total(const void* a, const void* b, int64_t n_bytes,
                             uint64_t* out, void* stream);

/* per-word popcount(a ^ b) for equal-shape word buffers -> int32, fused
 * (the reference materialises the XOR first).
 * Replaces cbrute::cuda::hamming_distance, cbrute/cuda/ops_cuda.cu:307-309. */
int brute_b200_hamming_words(const uint64_t* a, const uint64_t* b, int32_t* out,
                             int64_t n_words, void* stream);

/* ---- bitwise ----------------------------------------------------------- */
/* out = a OP b over [rows, words_per_row]; `last_dim_bits` is only read by
 * XNOR, which clears each row's pad bits. out may be exactly a or exactly b
 * (in place: every word is read and written by the same thread); partial overlap is not allowed.
 * Replaces the ATen int64 bitwise launches of brute/tensor.py:564-598,1494-1537
 * and brute/fast.py:37-83 (eq = xor + bit1_not_packed fused into one XNOR). */
int brute_b200_bitwise(int op, const uint64_t* a, const uint64_t* b, uint64_t* out,
                       int64_t rows, int64_t words_per_row, int64_t last_dim_bits,
                       void* stream);

/* out = ~a with the pad bits of each row's last word kept 0.
 * Replaces bit1_not_packed_composite, cbrute/ext.cpp:27-39 (3 ATen launches). */
int brute_b200_not_masked(const uint64_t* a, uint64_t* out,
                          int64_t rows, int64_t words_per_row, int64_t last_dim_bits,
                          void* stream);

/* out = (cond & a) | (~cond & b), word-wise select.
 * Replaces the 4-launch packed `where` of brute/tensor.py:1863-1883. */
int brute_b200_select(const uint64_t* cond, const uint64_t* a, const uint64_t* b,
                      uint64_t* out, int64_t n_words, void* stream);

/* out[r] = 1 if any bit of row r is set / if all `last_dim_bits` bits are set.
 * Replaces the ATen compositions of brute/tensor.py:1415-1431. */
int brute_b200_row_any(const uint64_t* a, uint8_t* out, int64_t rows,
                       int64_t words_per_row, void* stream);
int brute_b200_row_all(const uint64_t* a, uint8_t* out, int64_t rows,
                       int64_t words_per_row, int64_t last_dim_bits, void* stream);

/* signed_bundle without a workspace argument and without any allocation: the scratch for the
 * transposed V is a fixed 1 MiB array inside the library's device image (one per device), found
 * once per device by a symbol lookup on the first call made with that device current. There is no
 * counterpart in the reference; it exists for callers that may not allocate (or pass) device memory.
 *  - B * D * ceil(N/64) * 8 must not exceed brute_b200_signed_bundle_static_max_bytes() (1 MiB),
 *    otherwise BRUTE_ERR_WORKSPACE and nothing is launched;
 *  - the array is shared by every call on a device: two calls whose kernels can overlap (different
 *    streams, or host threads racing on one stream) overwrite each other's scratch. Keep calls to
 *    this entry point on one stream per device, or order them with events;
 *  - the first call on a device performs the symbol lookup, a runtime query that does not belong
 *    inside a stream capture: make one call per device before capturing a CUDA graph that contains it.
 * Result and argument rules are those of brute_b200_signed_bundle_ws. */
int64_t brute_b200_signed_bundle_static_max_bytes(void);
int brute_b200_signed_bundle_static(const int8_t* W, const uint64_t* V, uint64_t* out,
                                    int64_t B, int64_t M, int64_t N, int64_t Dp, int64_t D,
                                    void* stream);

/* ---- layout on packed words ------------------------------------------- */
/* Bit-matrix transpose: in [batch, R, ceil(C/64)] -> out [batch, C, ceil(R/64)],
 * out bit (c, r) = in bit (r, c); pad bits of `out` are 0. in and out must not overlap.
 * Replaces the unpack -> bool transpose -> re-pack round trip that the reference takes
 * whenever a transpose moves the packed axis (brute/tensor.py:699-775, 1112-1121). */
int brute_b200_transpose_bits(const uint64_t* in, uint64_t* out,
                              int64_t batch, int64_t R, int64_t C, void* stream);

/* OR (BRUTE_OP_OR) or AND (BRUTE_OP_AND) over the middle axis of in [outer, R, inner]
 * words -> out [outer, inner] words: any()/all() over a non-packed dimension in one pass.
 * R == 0 gives the identity (0 / all ones). Rows of whole 16-byte vectors (inner even, 16-byte
 * aligned pointers): one launch, every output word written exactly once. Otherwise the output is
 * preset by a memset on `stream` and the blocks combine with atomics.
 * Replaces the log2(R) halving loop of ATen launches, brute/tensor.py:1440-1457. */
int brute_b200_reduce_rows(int op, const uint64_t* in, uint64_t* out,
                           int64_t outer, int64_t R, int64_t inner, void* stream);

/* Moves along the packed (last) axis without leaving the packed domain; rows of n bits,
 * ceil(n/64) words each, pad bits of the result 0, in and out must not overlap:
 *   flip:   out bit j = in bit n - 1 - j
 *   roll:   out bit j = in bit (j - shift) mod n        (torch.roll semantics, any sign of shift)
 *   gather: out bit j = in bit idx[j], j < n_out; idx is a device array of n_out int64, the same
 *           for every row; an index outside [0, n_in) reads as 0.
 * Replace the unpack -> bool flip/roll/index_select -> re-pack fallback of the reference
 * (brute/tensor.py:699-775, 795-801). */
int brute_b200_flip_bits(const uint64_t* in, uint64_t* out, int64_t rows, int64_t n, void* stream);
int brute_b200_roll_bits(const uint64_t* in, uint64_t* out, int64_t rows, int64_t n, int64_t shift,
                         void* stream);
int brute_b200_gather_bits(const uint64_t* in, const int64_t* idx, uint64_t* out,
                           int64_t rows, int64_t n_in, int64_t n_out, void* stream);

/* Scatter along the packed axis, IN PLACE: for every row of `packed` [rows, ceil(n/64)] and every
 * j < n_idx, bit idx[j] of the row becomes bit j of the row of `src` [rows, ceil(n_idx/64)], or the
 * constant `value` (0 / 1) when src is NULL. idx is a device array of n_idx int64, the same for every
 * row; an index outside [0, n) writes nothing. Positions that idx names twice take one of the
 * candidate bits (as torch's index_copy_ with repeated indices); all other bits keep their value.
 * Replaces the unpack -> bool index_put_ / index_copy_ / index_fill_ -> re-pack round trip the
 * reference takes for a write through a tensor index on the last axis (the packed column scatter of
 * brute/tensor.py:715-775 covers one integer column and a scalar only). */
int brute_b200_scatter_bits(uint64_t* packed, const int64_t* idx, const uint64_t* src, int value,
                            int64_t rows, int64_t n, int64_t n_idx, void* stream);

/* ---- xnor-popcount GEMM ------------------------------------------------ */
/* A [M, Kp] words, B [N, Kp] words (rows of B are output features), K logical
 * bits (K <= 64*Kp, pad bits 0) -> C [M, N] int32 with row pitch ldc elements,
 * C[m,n] = K - 2 * sum_k popcount(A[m,k] ^ B[n,k])  (the +-1 dot product).
 * `impl` is a BRUTE_GEMM_* value. M, N or Kp equal to 0 are legal.
 * Replaces cbrute::cuda::xnor_popcount_matmul, cbrute/cuda/ops_cuda.cu:144-221,
 * CutlassB1XorGemm + KMinusTwoH, cbrute/cuda/kernels/matmul_cutlass.cuh:36-105 and
 * k_xnor_popcount_matmul, cbrute/cuda/kernels/matmul_fallback.cuh:20-59. */
int brute_b200_xnor_gemm(const uint64_t* A, const uint64_t* B, int32_t* C,
                         int64_t M, int64_t N, int64_t Kp, int64_t K, int64_t ldc,
                         int impl, void* stream);

/* The same GEMM (instruction path chosen as by BRUTE_GEMM_AUTO), leaving `leave_sms` SMs of the GPU
 * to kernels of other streams: the persistent tensor-core kernel then walks its tiles with fewer CTA
 * pairs, so that e.g. the all-gather of the previous row block can run under it. Same result, bit
 * for bit; paths that are not persistent ignore the hint. The reference has no counterpart (it has
 * no multi-GPU path); the contraction is that of cbrute/cuda/ops_cuda.cu:144-221. */
int brute_b200_xnor_gemm_leave_sms(const uint64_t* A, const uint64_t* B, int32_t* C,
                                   int64_t M, int64_t N, int64_t Kp, int64_t K, int64_t ldc,
                                   int leave_sms, void* stream);

/* Same contraction with the binarised-MLP epilogue fused: the int32 count is
 * scaled by scale[n] (fp32), thresholded per `mode` and re-packed, so
 * out [M, ceil(N/64)] words holds bit(m,n) = sign(scale[n] * C[m,n]).
 * Replaces the composition xnor_popcount_matmul -> float scale -> `_to_bool` ->
 * pack_bool (cbrute/cuda/ops_cuda.cu:144-221, brute/tensor.py:163-177). */
int brute_b200_xnor_gemm_scale_sign_pack(const uint64_t* A, const uint64_t* B,
                                         const float* scale, uint64_t* out,
                                         int64_t M, int64_t N, int64_t Kp, int64_t K,
                                         int mode, int impl, void* stream);

/* ---- signed vote bundle ------------------------------------------------ */
/* W int8 [B, M, N], V packed [B, N, Dp] words, D logical bits (D <= 64*Dp) ->
 * out packed [B, M, Dp]: bit(b,m,d) = (sum_n W[b,m,n] * pm1(V[b,n,d]) >= 0), pad bits 0.
 * Replaces cbrute::cuda::signed_bundle, cbrute/cuda/ops_cuda.cu:224-241 and k_signed_bundle,
 * cbrute/cuda/kernels/signed_bundle.cuh:18-54 (CPU statement: cbrute/cpu/ops_cpu.cpp:164-213). */
int brute_b200_signed_bundle(const int8_t* W, const uint64_t* V, uint64_t* out,
                             int64_t B, int64_t M, int64_t N, int64_t Dp, int64_t D, void* stream);

/* brute_b200_signed_bundle runs on the tensor cores where the shape allows (W 16-byte aligned, N a
 * multiple of 16 and >= 128, M >= 64, Dp == ceil(D/64)): the vote is an int8 GEMM that streams W once
 * (HBM bound), and the bit transpose of V that it needs happens inside the kernel, block by block.
 * The variant below does that transpose as a pass of its own into a caller-provided `workspace`
 * (the earlier form of the tensor path, kept for callers that hold such a workspace): `workspace` must hold
 * brute_b200_signed_bundle_workspace_bytes(B, N, D) bytes of device memory, 8-byte aligned; the
 * library allocates nothing, so the caller provides it (BRUTE_ERR_WORKSPACE if it is missing or too
 * small). Shapes the tensor path does not take (W not 16-byte aligned, N not a multiple of 16, N < 128,
 * M < 64, rows padded beyond ceil(D/64) words) run the kernel of brute_b200_signed_bundle and ignore the
 * workspace. Same reference lines. */
int64_t brute_b200_signed_bundle_workspace_bytes(int64_t B, int64_t N, int64_t D);
int brute_b200_signed_bundle_ws(const int8_t* W, const uint64_t* V, uint64_t* out,
                                int64_t B, int64_t M, int64_t N, int64_t Dp, int64_t D,
                                void* workspace, int64_t workspace_bytes, void* stream);

/* ---- transport of the GEMM result between GPUs -------------------------- */
/* The reference has no multi-GPU path; these serve the all-gather of the column-sharded GEMM
 * (the result of cbrute/cuda/ops_cuda.cu:144-221 split by B's rows across ranks).
 * narrow: int32 [n] -> int16 [n], exact for |v| <= 32767 (C = K - 2H with K <= 32767), so that the
 * ranks exchange half the bytes.
 * unstack: what an all-gather delivers, the rank blocks stacked as in [world, rows, n_loc]
 * (elem_bytes 2: int16, 4: int32), becomes row-major int32: out[m * ldc + r * n_loc + j] =
 * in[r, m, j]; ldc >= world * n_loc. in and out must not overlap. */
int brute_b200_narrow_i32_i16(const int32_t* in, int16_t* out, int64_t n, void* stream);
/* The GEMM of brute_b200_xnor_gemm_leave_sms with C written as int16 [M, ldc] straight from the
 * epilogue (no int32 result, no narrowing pass): exact for K <= 32767. Tensor-core pair kernel only:
 * BRUTE_ERR_UNSUPPORTED for K > 32767 and for operands that kernel does not take (the caller then uses
 * the int32 GEMM and brute_b200_narrow_i32_i16). */
int brute_b200_xnor_gemm_i16(const uint64_t* A, const uint64_t* B, int16_t* C,
                             int64_t M, int64_t N, int64_t Kp, int64_t K, int64_t ldc,
                             int leave_sms, void* stream);
int brute_b200_unstack_rank_blocks(const void* in, int elem_bytes, int32_t* out,
                                   int64_t world, int64_t rows, int64_t n_loc, int64_t ldc, void* stream);

/* The same exchange over peer memory (no reference counterpart either): gather and widening in one
 * pass, with plain peer loads over NVLink. Every rank keeps its narrowed blocks [M, n_loc] int16 and
 * a few 32-bit flag words in memory that its peers have mapped (the caller provides the mappings:
 * send_ptrs[p] / flag_ptrs[p] are rank p's buffer and flag words as THIS process sees them, host
 * arrays of `world` <= 16 device pointers).
 *  - peer_set_flag: *flag = value with release semantics at system scope, queued on `stream` behind
 *    the work that produced the data the flag announces (flag: this rank's own word).
 *  - gather_peer_widen: for every rank p, waits until flag_ptrs[p][flag_index] has reached `want`
 *    (the own rank's block is not waited for), then out[m, p * n_loc + j] = send_ptrs[p][m, j] for
 *    m in [m0, m1): out is this rank's row-major int32 [M, world * n_loc]. elem_bytes 2: the blocks
 *    are int16 and are widened; 4: int32 blocks (K > 32767), copied. ctas_per_peer CTAs read each
 *    peer (<= 0: 8).
 *  - peer_wait_flags: waits until word `index` of every OTHER rank has reached `want` (before a
 *    send buffer is written again).
 * Flag values are call numbers that only grow, compared as signed differences. Every wait gives up
 * after limit_us and records which rank's flag did not arrive: brute_b200_peer_wait_status()
 * synchronises the device and returns 0, or 1 + that rank, and clears the record. Nothing traps. */
int brute_b200_peer_set_flag(uint32_t* flag, uint32_t value, void* stream);
int brute_b200_peer_wait_flags(const void* const* send_ptrs, const void* const* flag_ptrs, int world, int self,
                               int index, uint32_t want, int64_t limit_us, void* stream);
int brute_b200_gather_peer_widen(const void* const* send_ptrs, const void* const* flag_ptrs, int32_t* out,
                                 int64_t M, int64_t n_loc, int elem_bytes, int64_t m0, int64_t m1, int world, int self,
                                 int flag_index, uint32_t want, int ctas_per_peer, int64_t limit_us, void* stream);
int brute_b200_peer_wait_status(void);

/* ---- binary attention -------------------------------------------------- */
/* Qp, Kp_ [B, H, S, D/64] words (sign-binarised Q and K), V and O bf16
 * [B, H, S, D]; score(i,j) = (D - 2*popcount(q_i ^ k_j)) * scale, optional
 * causal mask (j <= i), softmax in fp32, O = P @ V in bf16. D must be 64 or 128.
 * The reference has no such kernel (one docstring mention, brute/fast.py:122-124);
 * it replaces the composition of xnor_popcount_matmul
 * (cbrute/cuda/ops_cuda.cu:144-221) per (b,h) with torch softmax and matmul. */
int brute_b200_binary_attention_fwd(const uint64_t* Qp, const uint64_t* Kp_,
                                    const void* V, void* O,
                                    int64_t B, int64_t H, int64_t S, int64_t D,
                                    int causal, float scale, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BRUTE_B200_H_ */
