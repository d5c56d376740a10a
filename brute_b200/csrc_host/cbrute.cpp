// _cbrute: host-side helpers of the front end that need the tensor implementation itself, and the
// compiled binding of torch.ops.brute.* to the C ABI of libbrute_b200.so.
//
// The reference loads a pybind module of this name whose only job is to pull in the compiled op
// library (cbrute/ext.cpp:11-13); its ops are C++ functions registered with TORCH_LIBRARY_IMPL
// (cbrute/ext.cpp:106-117) that validate, allocate and launch (cbrute/cuda/ops_cuda.cu). The second
// half of this file is that layer for the sm_100a library: register_cuda_ops() binds the CUDA key of
// every schema (the schemas themselves are defined by brute_b200/ops.py) to a C++ function that does
// what the Python binding in ops.py does - same checks, same messages, same allocation - and calls
// the same extern "C" entry point on the caller's current stream under a device guard.
//
// The helpers are two things Python cannot express:
//
//  * lazy_bool(shape, device): the bool storage of a packed-only bit1 result. The reference
//    allocates the full bool tensor at this point (brute/tensor.py:316, one byte per bit). This
//    returns a tensor with the same sizes and contiguous strides over an EMPTY (0-byte, resizable)
//    storage: nothing is allocated until somebody reads the tensor as bool.
//  * adopt_storage(dst, src): hands src's allocation to dst's storage object, so every alias of
//    dst (views taken before or after) sees the data, without a copy. src is left with 0 bytes.
#include <torch/extension.h>
#include <torch/library.h>
#include <ATen/EmptyTensor.h>
#include <c10/core/CPUAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <memory>

#include "brute_b200.h"

namespace {

at::Tensor lazy_bool(const std::vector<int64_t>& shape, const c10::Device& device) {
    // empty({0}) picks the device's own allocator and dispatch keys and allocates nothing
    at::Tensor t = at::empty({0}, at::TensorOptions().dtype(at::kBool).device(device));
    std::vector<int64_t> strides(shape.size());
    int64_t run = 1;
    for (int64_t i = static_cast<int64_t>(shape.size()) - 1; i >= 0; --i) {
        strides[i] = run;
        run *= shape[i] > 1 ? shape[i] : 1;
    }
    t.unsafeGetTensorImpl()->set_sizes_and_strides(shape, strides);
    return t;
}

void adopt_storage(const at::Tensor& dst, const at::Tensor& src) {
    TORCH_CHECK(dst.device() == src.device(), "adopt_storage: device mismatch");
    TORCH_CHECK(dst.dtype() == src.dtype(), "adopt_storage: dtype mismatch");
    TORCH_CHECK(src.is_contiguous() && src.storage_offset() == 0, "adopt_storage: src must own a dense storage");
    // src must be a fresh result that no other tensor aliases (the caller's contract: it is the
    // output of unpack_bool); a Python storage wrapper that somebody made of it may still exist
    c10::StorageImpl* d = dst.storage().unsafeGetStorageImpl();
    c10::StorageImpl* s = src.storage().unsafeGetStorageImpl();
    TORCH_CHECK(d != s, "adopt_storage: dst and src are the same storage");
    const auto nbytes = s->sym_nbytes();
    at::DataPtr old = d->set_data_ptr(s->set_data_ptr(at::DataPtr(nullptr, src.device())));
    d->set_nbytes(nbytes);
    s->set_nbytes(0);
    // `old` (dst's previous allocation, normally empty) is released here
}

// =====================================================================================
// compiled binding: torch.ops.brute.* (CUDA key) -> the C ABI
// =====================================================================================
using at::Tensor;

inline int64_t words(int64_t n_bits) { return (n_bits + 63) / 64; }

// every tensor argument must be a CUDA tensor on the first one's device (the kernels take raw pointers)
inline void same_device(const char* name, std::initializer_list<const Tensor*> ts) {
    const Tensor* first = nullptr;
    for (const Tensor* t : ts) {
        if (!t->defined()) continue;
        if (!first) {
            first = t;
            TORCH_CHECK(t->is_cuda(), name, ": expected CUDA tensors, got a tensor on ", t->device());
        } else {
            TORCH_CHECK(t->device() == first->device(), name, ": expected all tensors to be on the same device, "
                        "but found at least two devices, ", first->device(), " and ", t->device());
        }
    }
}

inline void* cur_stream(const Tensor& t) {
    return static_cast<void*>(c10::cuda::getCurrentCUDAStream(t.device().index()).stream());
}

inline void ok(int rc, const char* what) {
    TORCH_CHECK(rc == BRUTE_OK, what, ": ", brute_b200_strerror(rc), " (brute_b200 status ", rc, ")");
}

template <typename T> inline T* ptr(const Tensor& t) { return t.numel() ? static_cast<T*>(t.data_ptr()) : nullptr; }

Tensor pack_bool(const Tensor& input) {
    TORCH_CHECK(input.dim() >= 1, "pack_bool: input must have >= 1 dim");
    TORCH_CHECK(input.scalar_type() == at::kBool, "pack_bool: input must be torch.bool");
    same_device("pack_bool", {&input});
    const c10::cuda::CUDAGuard guard(input.device());
    Tensor inp = input.contiguous();
    const int64_t ld = inp.size(-1);
    auto shape = inp.sizes().vec();
    shape.back() = words(ld);
    Tensor out = at::empty(shape, inp.options().dtype(at::kLong));
    if (out.numel() == 0) return out;
    ok(brute_b200_pack_bool(static_cast<const uint8_t*>(inp.data_ptr()), static_cast<uint64_t*>(out.data_ptr()),
                            inp.numel() / ld, ld, cur_stream(inp)), "pack_bool");
    return out;
}

Tensor pack_sign(const Tensor& input, int64_t mode) {
    TORCH_CHECK(input.dim() >= 1, "pack_sign: input must have >= 1 dim");
    int dt = -1;
    if (input.scalar_type() == at::kFloat) dt = BRUTE_DT_F32;
    else if (input.scalar_type() == at::kBFloat16) dt = BRUTE_DT_BF16;
    else if (input.scalar_type() == at::kHalf) dt = BRUTE_DT_F16;
    TORCH_CHECK(dt >= 0, "pack_sign: input must be float32, bfloat16 or float16");
    same_device("pack_sign", {&input});
    const c10::cuda::CUDAGuard guard(input.device());
    Tensor inp = input.contiguous();
    const int64_t ld = inp.size(-1);
    auto shape = inp.sizes().vec();
    shape.back() = words(ld);
    Tensor out = at::empty(shape, inp.options().dtype(at::kLong));
    if (out.numel() == 0) return out;
    ok(brute_b200_pack_sign(inp.data_ptr(), dt, static_cast<uint64_t*>(out.data_ptr()), inp.numel() / ld, ld,
                            static_cast<int>(mode), cur_stream(inp)), "pack_sign");
    return out;
}

template <bool PM1>
Tensor unpack_any(const Tensor& packed, at::IntArrayRef logical_shape) {
    const char* name = PM1 ? "unpack_bits" : "unpack_bool";
    same_device(name, {&packed});
    const c10::cuda::CUDAGuard guard(packed.device());
    Tensor p = packed.contiguous();
    TORCH_CHECK(logical_shape.size() >= 1, name, ": logical_shape must have >= 1 dim");
    const int64_t ll = logical_shape.back();
    Tensor out = at::empty(logical_shape, p.options().dtype(PM1 ? at::kFloat : at::kBool));
    if (ll == 0 || p.numel() == 0) return out;
    TORCH_CHECK(p.scalar_type() == at::kLong, name, ": packed must be torch.int64");
    int64_t rows = 1;
    for (size_t i = 0; i + 1 < logical_shape.size(); ++i) rows *= logical_shape[i];
    TORCH_CHECK(p.size(-1) == words(ll) && p.numel() == rows * words(ll), name, ": packed shape does not match logical_shape");
    if (PM1) ok(brute_b200_unpack_pm1_f32(static_cast<const uint64_t*>(p.data_ptr()), static_cast<float*>(out.data_ptr()),
                                          p.numel() / p.size(-1), ll, cur_stream(p)), name);
    else     ok(brute_b200_unpack_bool(static_cast<const uint64_t*>(p.data_ptr()), static_cast<uint8_t*>(out.data_ptr()),
                                       p.numel() / p.size(-1), ll, cur_stream(p)), name);
    return out;
}

void gemm_args(const Tensor& A, const Tensor& B, int64_t K, const char* name) {
    TORCH_CHECK(A.dim() == 2 && B.dim() == 2, name, ": inputs must be 2-D");
    TORCH_CHECK(A.size(1) == B.size(1), name, ": packed K mismatch");
    TORCH_CHECK(A.scalar_type() == at::kLong && B.scalar_type() == at::kLong, name, ": inputs must be int64 packed buffers");
    TORCH_CHECK(A.device() == B.device(), name, ": inputs must be on the same device");
    TORCH_CHECK(0 <= K && K <= 64 * A.size(1), name, ": K out of range for the packed width");
    same_device(name, {&A, &B});
}

Tensor xnor_popcount_matmul_impl(const Tensor& A, const Tensor& B, int64_t K, int64_t impl) {
    gemm_args(A, B, K, "xnor_popcount_matmul");
    const c10::cuda::CUDAGuard guard(A.device());
    Tensor Ac = A.contiguous(), Bc = B.contiguous();
    const int64_t M = Ac.size(0), N = Bc.size(0), Kp = Ac.size(1);
    Tensor C = at::empty({M, N}, Ac.options().dtype(at::kInt));
    if (M == 0 || N == 0) return C;
    ok(brute_b200_xnor_gemm(ptr<const uint64_t>(Ac), ptr<const uint64_t>(Bc), static_cast<int32_t*>(C.data_ptr()),
                            M, N, Kp, K, N, static_cast<int>(impl), cur_stream(Ac)), "xnor_popcount_matmul");
    return C;
}

Tensor xnor_popcount_matmul(const Tensor& A, const Tensor& B, int64_t K) {
    return xnor_popcount_matmul_impl(A, B, K, BRUTE_GEMM_AUTO);
}

Tensor& xnor_popcount_matmul_out(const Tensor& A, const Tensor& B, int64_t K, int64_t leave_sms, Tensor& out) {
    gemm_args(A, B, K, "xnor_popcount_matmul");
    same_device("xnor_popcount_matmul", {&A, &out});
    const c10::cuda::CUDAGuard guard(A.device());
    Tensor Ac = A.contiguous(), Bc = B.contiguous();
    const int64_t M = Ac.size(0), N = Bc.size(0), Kp = Ac.size(1);
    TORCH_CHECK(out.scalar_type() == at::kInt && out.dim() == 2 && out.size(0) == M && out.size(1) == N && out.is_contiguous(),
                "xnor_popcount_matmul_out: out must be a contiguous int32 [M, N] tensor");
    if (M && N)
        ok(brute_b200_xnor_gemm_leave_sms(ptr<const uint64_t>(Ac), ptr<const uint64_t>(Bc), static_cast<int32_t*>(out.data_ptr()),
                                          M, N, Kp, K, N, static_cast<int>(leave_sms), cur_stream(Ac)), "xnor_popcount_matmul");
    return out;
}

Tensor xnor_popcount_matmul_leave_sms(const Tensor& A, const Tensor& B, int64_t K, int64_t leave_sms) {
    gemm_args(A, B, K, "xnor_popcount_matmul");
    const c10::cuda::CUDAGuard guard(A.device());
    Tensor C = at::empty({A.size(0), B.size(0)}, A.options().dtype(at::kInt));
    return xnor_popcount_matmul_out(A, B, K, leave_sms, C);
}

Tensor xnor_matmul_scale_sign_pack(const Tensor& A, const Tensor& B, const Tensor& scale, int64_t K, int64_t mode) {
    gemm_args(A, B, K, "xnor_matmul_scale_sign_pack");
    same_device("xnor_matmul_scale_sign_pack", {&A, &scale});
    const c10::cuda::CUDAGuard guard(A.device());
    Tensor Ac = A.contiguous(), Bc = B.contiguous();
    const int64_t M = Ac.size(0), N = Bc.size(0), Kp = Ac.size(1);
    TORCH_CHECK(scale.scalar_type() == at::kFloat && scale.numel() == N,
                "xnor_matmul_scale_sign_pack: scale must be float32 [N] on the inputs' device");
    Tensor sc = scale.contiguous();
    Tensor out = at::empty({M, words(N)}, Ac.options());
    if (out.numel() == 0) return out;
    ok(brute_b200_xnor_gemm_scale_sign_pack(ptr<const uint64_t>(Ac), ptr<const uint64_t>(Bc), static_cast<const float*>(sc.data_ptr()),
                                            static_cast<uint64_t*>(out.data_ptr()), M, N, Kp, K, static_cast<int>(mode),
                                            BRUTE_GEMM_AUTO, cur_stream(Ac)), "xnor_matmul_scale_sign_pack");
    return out;
}

Tensor signed_bundle(const Tensor& W, const Tensor& V, int64_t D) {
    TORCH_CHECK(W.dim() == 3 && V.dim() == 3, "signed_bundle: W (B,M,N), V packed (B,N,Dp)");
    TORCH_CHECK(W.scalar_type() == at::kChar, "signed_bundle: W must be int8");
    const int64_t B = W.size(0), M = W.size(1), N = W.size(2), Dp = V.size(2);
    TORCH_CHECK(V.size(0) == B && V.size(1) == N, "signed_bundle: W (B,M,N) / V (B,N,Dp) batch or N mismatch");
    TORCH_CHECK(V.scalar_type() == at::kLong && 0 <= D && D <= 64 * Dp, "signed_bundle: V must be int64 packed with D <= 64*Dp");
    same_device("signed_bundle", {&W, &V});
    const c10::cuda::CUDAGuard guard(V.device());
    Tensor Wc = W.contiguous(), Vc = V.contiguous();
    Tensor out = at::empty({B, M, Dp}, Vc.options());
    if (out.numel())      // one launch, no scratch: the tensor-core kernel transposes V's bit blocks itself
        ok(brute_b200_signed_bundle(ptr<const int8_t>(Wc), ptr<const uint64_t>(Vc), static_cast<uint64_t*>(out.data_ptr()),
                                    B, M, N, Dp, D, cur_stream(Vc)), "signed_bundle");
    return out;
}

Tensor popcount(const Tensor& x) {
    same_device("popcount", {&x});
    const c10::cuda::CUDAGuard guard(x.device());
    Tensor p = x.contiguous();
    int eb = 0;
    switch (p.scalar_type()) {
        case at::kByte: case at::kBool: case at::kChar: eb = 1; break;
        case at::kShort: eb = 2; break;
        case at::kInt: eb = 4; break;
        case at::kLong: eb = 8; break;
        default: TORCH_CHECK(false, "popcount: unsupported dtype ", p.scalar_type());
    }
    Tensor out = at::empty(p.sizes(), p.options().dtype(at::kInt));
    if (p.numel() == 0) return out;
    ok(brute_b200_popcount_elems(p.data_ptr(), static_cast<int32_t*>(out.data_ptr()), p.numel(), eb, cur_stream(p)), "popcount");
    return out;
}

Tensor packed_popcount(const Tensor& x) {
    same_device("packed_popcount", {&x});
    const c10::cuda::CUDAGuard guard(x.device());
    Tensor p = x.contiguous();
    Tensor out = at::empty({}, p.options().dtype(at::kLong));           // zeroed by the call itself
    ok(brute_b200_popcount_total(ptr<const void>(p), p.numel() * p.element_size(), static_cast<uint64_t*>(out.data_ptr()),
                                 cur_stream(p)), "packed_popcount");
    return out;
}

Tensor bit1_hamming_total(const Tensor& A, const Tensor& B) {
    TORCH_CHECK(A.sizes() == B.sizes(), "bit1_hamming_total: shape mismatch");
    TORCH_CHECK(A.scalar_type() == B.scalar_type(), "bit1_hamming_total: dtype mismatch");
    same_device("bit1_hamming_total", {&A, &B});
    const c10::cuda::CUDAGuard guard(A.device());
    Tensor Ac = A.contiguous(), Bc = B.contiguous();
    Tensor out = at::empty({}, Ac.options().dtype(at::kLong));
    ok(brute_b200_hamming_total(ptr<const void>(Ac), ptr<const void>(Bc), Ac.numel() * Ac.element_size(),
                                static_cast<uint64_t*>(out.data_ptr()), cur_stream(Ac)), "bit1_hamming_total");
    return out;
}

Tensor hamming_distance(const Tensor& A, const Tensor& B) {
    same_device("hamming_distance", {&A, &B});
    if (A.sizes() == B.sizes() && A.scalar_type() == at::kLong && B.scalar_type() == at::kLong) {
        const c10::cuda::CUDAGuard guard(A.device());
        Tensor Ac = A.contiguous(), Bc = B.contiguous();
        Tensor out = at::empty(Ac.sizes(), Ac.options().dtype(at::kInt));
        if (Ac.numel())
            ok(brute_b200_hamming_words(static_cast<const uint64_t*>(Ac.data_ptr()), static_cast<const uint64_t*>(Bc.data_ptr()),
                                        static_cast<int32_t*>(out.data_ptr()), Ac.numel(), cur_stream(Ac)), "hamming_distance");
        return out;
    }
    return popcount(at::bitwise_xor(A, B));                                // broadcasting / other dtypes
}

Tensor bit1_not_packed(const Tensor& A, int64_t last_dim_bits) {
    TORCH_CHECK(A.scalar_type() == at::kLong, "bit1_not_packed: input must be int64");
    same_device("bit1_not_packed", {&A});
    const c10::cuda::CUDAGuard guard(A.device());
    Tensor Ac = A.contiguous();
    Tensor out = at::empty_like(Ac);
    if (Ac.numel() == 0) return out;
    const int64_t wpr = Ac.dim() ? Ac.size(-1) : 1;
    ok(brute_b200_not_masked(static_cast<const uint64_t*>(Ac.data_ptr()), static_cast<uint64_t*>(out.data_ptr()),
                             Ac.numel() / wpr, wpr, last_dim_bits, cur_stream(Ac)), "bit1_not_packed");
    return out;
}

Tensor bitwise_packed(const Tensor& A, const Tensor& B, int64_t op, int64_t last_dim_bits) {
    TORCH_CHECK(A.sizes() == B.sizes(), "bitwise_packed: shape mismatch");
    TORCH_CHECK(A.scalar_type() == at::kLong && B.scalar_type() == at::kLong, "bitwise_packed: inputs must be int64");
    same_device("bitwise_packed", {&A, &B});
    const c10::cuda::CUDAGuard guard(A.device());
    Tensor Ac = A.contiguous(), Bc = B.contiguous();
    Tensor out = at::empty_like(Ac);
    if (Ac.numel() == 0) return out;
    const int64_t wpr = Ac.dim() ? Ac.size(-1) : 1;
    ok(brute_b200_bitwise(static_cast<int>(op), static_cast<const uint64_t*>(Ac.data_ptr()), static_cast<const uint64_t*>(Bc.data_ptr()),
                          static_cast<uint64_t*>(out.data_ptr()), Ac.numel() / wpr, wpr, last_dim_bits, cur_stream(Ac)),
       "bitwise_packed");
    return out;
}

Tensor select_packed(const Tensor& cond, const Tensor& A, const Tensor& B) {
    TORCH_CHECK(cond.sizes() == A.sizes() && A.sizes() == B.sizes(), "select_packed: shape mismatch");
    same_device("select_packed", {&cond, &A, &B});
    const c10::cuda::CUDAGuard guard(A.device());
    Tensor c = cond.contiguous(), a = A.contiguous(), b = B.contiguous();
    Tensor out = at::empty_like(a);
    if (a.numel())
        ok(brute_b200_select(static_cast<const uint64_t*>(c.data_ptr()), static_cast<const uint64_t*>(a.data_ptr()),
                             static_cast<const uint64_t*>(b.data_ptr()), static_cast<uint64_t*>(out.data_ptr()), a.numel(),
                             cur_stream(a)), "select_packed");
    return out;
}

template <bool ALL>
Tensor row_reduce(const Tensor& A, int64_t last_dim_bits) {
    const char* name = ALL ? "row_all" : "row_any";
    TORCH_CHECK(A.dim() >= 1 && A.scalar_type() == at::kLong, name, ": input must be int64 with >= 1 dim");
    same_device(name, {&A});
    const c10::cuda::CUDAGuard guard(A.device());
    Tensor Ac = A.contiguous();
    Tensor out = at::empty(Ac.sizes().slice(0, Ac.dim() - 1), Ac.options().dtype(at::kBool));
    if (out.numel()) {
        if (ALL) ok(brute_b200_row_all(ptr<const uint64_t>(Ac), static_cast<uint8_t*>(out.data_ptr()), out.numel(), Ac.size(-1),
                                       last_dim_bits, cur_stream(Ac)), name);
        else     ok(brute_b200_row_any(ptr<const uint64_t>(Ac), static_cast<uint8_t*>(out.data_ptr()), out.numel(), Ac.size(-1),
                                       cur_stream(Ac)), name);
    }
    return out;
}
Tensor row_any(const Tensor& A) { return row_reduce<false>(A, 0); }
Tensor row_all(const Tensor& A, int64_t bits) { return row_reduce<true>(A, bits); }

Tensor transpose_packed(const Tensor& packed, int64_t rows, int64_t cols) {
    TORCH_CHECK(packed.dim() >= 2 && packed.scalar_type() == at::kLong, "transpose_packed: input must be int64 with >= 2 dims");
    TORCH_CHECK(packed.size(-2) == rows && packed.size(-1) == words(cols),
                "transpose_packed: packed shape must be [..., rows, ceil(cols/64)]");
    same_device("transpose_packed", {&packed});
    const c10::cuda::CUDAGuard guard(packed.device());
    Tensor pc = packed.contiguous();
    int64_t batch = 1;
    auto shape = pc.sizes().vec();
    for (size_t i = 0; i + 2 < shape.size(); ++i) batch *= shape[i];
    shape[shape.size() - 2] = cols;
    shape[shape.size() - 1] = words(rows);
    Tensor out = at::empty(shape, pc.options());
    if (out.numel())
        ok(brute_b200_transpose_bits(static_cast<const uint64_t*>(pc.data_ptr()), static_cast<uint64_t*>(out.data_ptr()),
                                     batch, rows, cols, cur_stream(pc)), "transpose_packed");
    return out;
}

Tensor reduce_rows_packed(const Tensor& packed, int64_t dim, bool use_or) {
    TORCH_CHECK(packed.scalar_type() == at::kLong && packed.dim() >= 2, "reduce_rows_packed: input must be int64 with >= 2 dims");
    const int64_t nd = packed.dim();
    const int64_t d = dim >= 0 ? dim : nd + dim;
    TORCH_CHECK(0 <= d && d < nd - 1, "reduce_rows_packed: dim must be a non-packed dimension");
    same_device("reduce_rows_packed", {&packed});
    const c10::cuda::CUDAGuard guard(packed.device());
    Tensor pc = packed.contiguous();
    int64_t outer = 1, inner = 1;
    std::vector<int64_t> shape;
    for (int64_t i = 0; i < nd; ++i) {
        if (i < d) outer *= pc.size(i);
        if (i > d) inner *= pc.size(i);
        if (i != d) shape.push_back(pc.size(i));
    }
    Tensor out = at::empty(shape, pc.options());
    if (out.numel())
        ok(brute_b200_reduce_rows(use_or ? BRUTE_OP_OR : BRUTE_OP_AND, ptr<const uint64_t>(pc), static_cast<uint64_t*>(out.data_ptr()),
                                  outer, pc.size(d), inner, cur_stream(pc)), "reduce_rows_packed");
    return out;
}

Tensor packed_rows(const Tensor& packed, int64_t n, const char* what, int64_t& rows) {
    TORCH_CHECK(packed.dim() >= 1 && packed.scalar_type() == at::kLong, what, ": input must be int64 with >= 1 dim");
    TORCH_CHECK(packed.size(-1) == words(n), what, ": last dimension must be ceil(n/64) words");
    same_device(what, {&packed});
    Tensor pc = packed.contiguous();
    rows = pc.size(-1) ? pc.numel() / pc.size(-1) : 0;
    return pc;
}

Tensor flip_packed(const Tensor& packed, int64_t n) {
    int64_t rows;
    const c10::cuda::OptionalCUDAGuard guard(packed.is_cuda() ? c10::make_optional(packed.device()) : c10::nullopt);
    Tensor pc = packed_rows(packed, n, "flip_packed", rows);
    Tensor out = at::empty_like(pc);
    if (out.numel())
        ok(brute_b200_flip_bits(static_cast<const uint64_t*>(pc.data_ptr()), static_cast<uint64_t*>(out.data_ptr()), rows, n,
                                cur_stream(pc)), "flip_packed");
    return out;
}

Tensor roll_packed(const Tensor& packed, int64_t n, int64_t shift) {
    int64_t rows;
    const c10::cuda::OptionalCUDAGuard guard(packed.is_cuda() ? c10::make_optional(packed.device()) : c10::nullopt);
    Tensor pc = packed_rows(packed, n, "roll_packed", rows);
    Tensor out = at::empty_like(pc);
    if (out.numel())
        ok(brute_b200_roll_bits(static_cast<const uint64_t*>(pc.data_ptr()), static_cast<uint64_t*>(out.data_ptr()), rows, n, shift,
                                cur_stream(pc)), "roll_packed");
    return out;
}

Tensor gather_packed(const Tensor& packed, const Tensor& idx, int64_t n_in) {
    int64_t rows;
    const c10::cuda::OptionalCUDAGuard guard(packed.is_cuda() ? c10::make_optional(packed.device()) : c10::nullopt);
    Tensor pc = packed_rows(packed, n_in, "gather_packed", rows);
    TORCH_CHECK(idx.dim() == 1 && idx.scalar_type() == at::kLong && idx.device() == pc.device(),
                "gather_packed: idx must be a 1-D int64 tensor on the input's device");
    Tensor ic = idx.contiguous();
    const int64_t n_out = ic.numel();
    auto shape = pc.sizes().vec();
    shape.back() = words(n_out);
    Tensor out = at::empty(shape, pc.options());
    if (out.numel())
        ok(brute_b200_gather_bits(ptr<const uint64_t>(pc), static_cast<const int64_t*>(ic.data_ptr()),
                                  static_cast<uint64_t*>(out.data_ptr()), pc.size(-1) ? rows : out.numel() / out.size(-1),
                                  n_in, n_out, cur_stream(pc)), "gather_packed");
    return out;
}

Tensor& scatter_packed_(Tensor& packed, const Tensor& idx, const c10::optional<Tensor>& src, bool value, int64_t n) {
    TORCH_CHECK(packed.dim() >= 1 && packed.scalar_type() == at::kLong && packed.is_contiguous(),
                "scatter_packed_: packed must be a contiguous int64 tensor with >= 1 dim");
    TORCH_CHECK(packed.size(-1) == words(n), "scatter_packed_: last dimension must be ceil(n/64) words");
    TORCH_CHECK(idx.dim() == 1 && idx.scalar_type() == at::kLong, "scatter_packed_: idx must be a 1-D int64 tensor");
    same_device("scatter_packed_", {&packed, &idx});
    const c10::cuda::CUDAGuard guard(packed.device());
    Tensor ic = idx.contiguous();
    const int64_t n_idx = ic.numel();
    const int64_t rows = packed.size(-1) ? packed.numel() / packed.size(-1) : 0;
    Tensor sc;
    if (src.has_value() && src->defined()) {
        auto want = packed.sizes().vec();
        want.back() = words(n_idx);
        TORCH_CHECK(src->scalar_type() == at::kLong && src->sizes().vec() == want,
                    "scatter_packed_: src must be int64 packed [..., ceil(len(idx)/64)] with packed's leading shape");
        same_device("scatter_packed_", {&packed, &*src});
        sc = src->contiguous();
    }
    if (rows && n_idx)
        ok(brute_b200_scatter_bits(static_cast<uint64_t*>(packed.data_ptr()), static_cast<const int64_t*>(ic.data_ptr()),
                                   sc.defined() ? static_cast<const uint64_t*>(sc.data_ptr()) : nullptr, value ? 1 : 0, rows, n, n_idx,
                                   cur_stream(packed)), "scatter_packed_");
    return packed;
}

Tensor narrow_i32_i16(const Tensor& x) {
    TORCH_CHECK(x.scalar_type() == at::kInt, "narrow_i32_i16: input must be int32");
    same_device("narrow_i32_i16", {&x});
    const c10::cuda::CUDAGuard guard(x.device());
    Tensor xc = x.contiguous();
    Tensor out = at::empty(xc.sizes(), xc.options().dtype(at::kShort));
    if (xc.numel())
        ok(brute_b200_narrow_i32_i16(static_cast<const int32_t*>(xc.data_ptr()), static_cast<int16_t*>(out.data_ptr()), xc.numel(),
                                     cur_stream(xc)), "narrow_i32_i16");
    return out;
}

Tensor& narrow_i32_i16_out(const Tensor& x, Tensor& out) {
    TORCH_CHECK(x.scalar_type() == at::kInt && out.scalar_type() == at::kShort && x.is_contiguous() && out.is_contiguous() &&
                x.numel() == out.numel(), "narrow_i32_i16_out: contiguous int32 input and int16 output of one size");
    same_device("narrow_i32_i16_out", {&x, &out});
    const c10::cuda::CUDAGuard guard(x.device());
    if (x.numel())
        ok(brute_b200_narrow_i32_i16(static_cast<const int32_t*>(x.data_ptr()), static_cast<int16_t*>(out.data_ptr()), x.numel(),
                                     cur_stream(x)), "narrow_i32_i16");
    return out;
}

Tensor& unstack_rank_blocks(const Tensor& stacked, Tensor& out, int64_t row0) {
    TORCH_CHECK(stacked.dim() == 3 && (stacked.scalar_type() == at::kShort || stacked.scalar_type() == at::kInt) && stacked.is_contiguous(),
                "unstack_rank_blocks: stacked must be a contiguous int16/int32 [world, rows, n_loc] tensor");
    const int64_t world = stacked.size(0), rows = stacked.size(1), n_loc = stacked.size(2);
    TORCH_CHECK(out.dim() == 2 && out.scalar_type() == at::kInt && out.is_contiguous() && out.size(1) == world * n_loc,
                "unstack_rank_blocks: out must be a contiguous int32 [M, world * n_loc] tensor");
    TORCH_CHECK(0 <= row0 && row0 + rows <= out.size(0), "unstack_rank_blocks: rows out of range");
    same_device("unstack_rank_blocks", {&stacked, &out});
    const c10::cuda::CUDAGuard guard(out.device());
    if (stacked.numel())
        ok(brute_b200_unstack_rank_blocks(stacked.data_ptr(), static_cast<int>(stacked.element_size()),
                                          static_cast<int32_t*>(out.data_ptr()) + row0 * out.size(1), world, rows, n_loc, out.size(1),
                                          cur_stream(out)), "unstack_rank_blocks");
    return out;
}

Tensor& randomize_bits(Tensor& out) {
    out.random_();              // cbrute/cuda/ops_cuda.cu:340, a plain ATen call
    return out;
}

Tensor binary_attention(const Tensor& Qp, const Tensor& Kp, const Tensor& V, bool causal, double scale) {
    TORCH_CHECK(V.dim() == 4 && Qp.dim() == 4 && Kp.dim() == 4, "binary_attention: Qp, Kp, V must be 4-D [B,H,S,*]");
    const int64_t B = V.size(0), H = V.size(1), S = V.size(2), D = V.size(3);
    TORCH_CHECK(V.scalar_type() == at::kBFloat16, "binary_attention: V must be bfloat16");
    TORCH_CHECK(Qp.scalar_type() == at::kLong && Kp.scalar_type() == at::kLong, "binary_attention: Qp, Kp must be int64 packed");
    TORCH_CHECK(D == 64 || D == 128, "binary_attention: head dim must be 64 or 128");
    const std::vector<int64_t> want = {B, H, S, D / 64};
    TORCH_CHECK(Qp.sizes().vec() == want && Kp.sizes().vec() == want, "binary_attention: packed Q/K shape must be [B,H,S,D/64]");
    same_device("binary_attention", {&Qp, &Kp, &V});
    const c10::cuda::CUDAGuard guard(V.device());
    Tensor q = Qp.contiguous(), k = Kp.contiguous(), v = V.contiguous();
    Tensor out = at::empty_like(v);
    if (out.numel())
        ok(brute_b200_binary_attention_fwd(static_cast<const uint64_t*>(q.data_ptr()), static_cast<const uint64_t*>(k.data_ptr()),
                                           v.data_ptr(), out.data_ptr(), B, H, S, D, causal ? 1 : 0, static_cast<float>(scale),
                                           cur_stream(v)), "binary_attention");
    return out;
}

std::unique_ptr<torch::Library> g_cuda_impl;

// Bind the CUDA key of every brute schema to the functions above. The schemas must exist already.
bool register_cuda_ops(const std::string& key) {
    if (g_cuda_impl) return false;
    g_cuda_impl = std::make_unique<torch::Library>(torch::Library::IMPL, "brute", c10::make_optional(c10::parseDispatchKey(key)),
                                                   __FILE__, __LINE__);
    torch::Library& m = *g_cuda_impl;
    // the reference's eleven (cbrute/ext.cpp:46-65)
    m.impl("pack_bool", &pack_bool);
    m.impl("unpack_bits", &unpack_any<true>);
    m.impl("unpack_bool", &unpack_any<false>);
    m.impl("xnor_popcount_matmul", &xnor_popcount_matmul);
    m.impl("signed_bundle", &signed_bundle);
    m.impl("popcount", &popcount);
    m.impl("packed_popcount", &packed_popcount);
    m.impl("hamming_distance", &hamming_distance);
    m.impl("bit1_hamming_total", &bit1_hamming_total);
    m.impl("bit1_not_packed", &bit1_not_packed);
    m.impl("randomize_bits", &randomize_bits);
    // additions
    m.impl("pack_sign", &pack_sign);
    m.impl("bitwise_packed", &bitwise_packed);
    m.impl("select_packed", &select_packed);
    m.impl("row_any", &row_any);
    m.impl("row_all", &row_all);
    m.impl("xnor_popcount_matmul_impl", &xnor_popcount_matmul_impl);
    m.impl("xnor_popcount_matmul_leave_sms", &xnor_popcount_matmul_leave_sms);
    m.impl("xnor_popcount_matmul_out", &xnor_popcount_matmul_out);
    m.impl("xnor_matmul_scale_sign_pack", &xnor_matmul_scale_sign_pack);
    m.impl("binary_attention", &binary_attention);
    m.impl("transpose_packed", &transpose_packed);
    m.impl("reduce_rows_packed", &reduce_rows_packed);
    m.impl("flip_packed", &flip_packed);
    m.impl("roll_packed", &roll_packed);
    m.impl("gather_packed", &gather_packed);
    m.impl("scatter_packed_", &scatter_packed_);
    m.impl("narrow_i32_i16", &narrow_i32_i16);
    m.impl("narrow_i32_i16_out", &narrow_i32_i16_out);
    m.impl("unstack_rank_blocks", &unstack_rank_blocks);
    return true;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("lazy_bool", &lazy_bool, "bool tensor of the given shape over an empty storage");
    m.def("adopt_storage", &adopt_storage, "move src's allocation into dst's storage object");
    m.def("_check_status", [](int rc) { ok(rc, "status"); }, "raise RuntimeError for a nonzero library status (tests)");
    m.def("register_cuda_ops", &register_cuda_ops, pybind11::arg("key") = "CUDA",
          "bind one dispatch key (CUDA) of torch.ops.brute.* to the compiled functions");
}
