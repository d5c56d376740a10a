// _cbrute: host-side helpers of the front end that need the tensor implementation itself.
//
// The reference loads a pybind module of this name whose only job is to pull in the compiled op
// library (cbrute/ext.cpp:11-13). Here it carries two things Python cannot express:
//
//  * lazy_bool(shape, device): the bool storage of a packed-only bit1 result. The reference
//    allocates the full bool tensor at this point (brute/tensor.py:316, one byte per bit). This
//    returns a tensor with the same sizes and contiguous strides over an EMPTY (0-byte, resizable)
//    storage: nothing is allocated until somebody reads the tensor as bool.
//  * adopt_storage(dst, src): hands src's allocation to dst's storage object, so every alias of
//    dst (views taken before or after) sees the data, without a copy. src is left with 0 bytes.
#include <torch/extension.h>
#include <ATen/EmptyTensor.h>
#include <c10/core/CPUAllocator.h>

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

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("lazy_bool", &lazy_bool, "bool tensor of the given shape over an empty storage");
    m.def("adopt_storage", &adopt_storage, "move src's allocation into dst's storage object");
}
