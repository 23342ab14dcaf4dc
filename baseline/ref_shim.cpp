// Compatibility shim for loading the UNMODIFIED reference extension under PyTorch 2.11.
//
// The reference calls `tensor.data_ptr<void>()` once (csrc/supergrok2_mamba_peer_kernels.cu:1875).  PyTorch 2.11
// declares the member template but exports instantiations for the scalar types only, so the reference's
// shared object fails to load with an undefined symbol.  This library supplies exactly that one
// specialisation (it returns the untyped data pointer, which is what the call means) and is loaded with
// RTLD_GLOBAL before the reference is imported.  No reference source file is changed.
#include <ATen/core/TensorBase.h>

namespace at {
template <>
void* TensorBase::data_ptr<void>() const {
    return this->data_ptr();
}
}  // namespace at
