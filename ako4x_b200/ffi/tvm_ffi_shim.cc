// TVM-FFI binding of two entry points of the C ABI, for the reference's `language = "cuda"` route
// (its builder compiles sources against TVM-FFI and looks up the symbol exported with
// TVM_FFI_DLL_EXPORT_TYPED_FUNC; templates/skills/cuda/cuda.md:8-31 of the reference). Destination
// passing style: the engine supplies the outputs, and an operator that needs scratch takes it as
// one more tensor. Built by tests/test_tvm_ffi_shim.py with the host compiler alone (no nvcc: the
// kernels live in libako4x_b200.so); the other operators bind the same way.
#include <tvm/ffi/container/tensor.h>
#include <tvm/ffi/extra/c_env_api.h>
#include <tvm/ffi/function.h>

#include "ako4x_b200.h"

namespace {

void* stream_of(const tvm::ffi::TensorView& t) {
  return TVMFFIEnvGetStream(t.device().device_type, t.device().device_id);
}

// run(hidden_states, weight, out)
void rmsnorm_h128(tvm::ffi::TensorView x, tvm::ffi::TensorView w, tvm::ffi::TensorView y) {
  const int rc = ako4x_rmsnorm_h128(x.data_ptr(), w.data_ptr(), y.data_ptr(), x.size(0), stream_of(x));
  TVM_FFI_ICHECK_EQ(rc, 0) << "ako4x_rmsnorm_h128 returned " << rc;
}

// run(q, k_cache, v_cache, kv_indptr, kv_indices, sm_scale, o, lse, workspace)
void gqa_paged_decode(tvm::ffi::TensorView q, tvm::ffi::TensorView k_cache, tvm::ffi::TensorView v_cache,
                      tvm::ffi::TensorView kv_indptr, tvm::ffi::TensorView kv_indices, double sm_scale,
                      tvm::ffi::TensorView o, tvm::ffi::TensorView lse, tvm::ffi::TensorView workspace) {
  const int64_t batch = q.size(0), n_idx = kv_indices.size(0), page_size = k_cache.size(1);
  const size_t need = ako4x_gqa_paged_decode_workspace_bytes(batch, n_idx, page_size);
  TVM_FFI_ICHECK_GE((size_t)workspace.numel(), need) << "workspace tensor (uint8) too small";
  const int rc = ako4x_gqa_paged_decode(
      q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), static_cast<const int32_t*>(kv_indptr.data_ptr()),
      static_cast<const int32_t*>(kv_indices.data_ptr()), static_cast<float>(sm_scale), o.data_ptr(),
      static_cast<float*>(lse.data_ptr()), batch, n_idx, page_size, workspace.data_ptr(), (size_t)workspace.numel(),
      stream_of(q));
  TVM_FFI_ICHECK_EQ(rc, 0) << "ako4x_gqa_paged_decode returned " << rc;
}

}  // namespace

TVM_FFI_DLL_EXPORT_TYPED_FUNC(rmsnorm_h128, rmsnorm_h128);
TVM_FFI_DLL_EXPORT_TYPED_FUNC(gqa_paged_decode, gqa_paged_decode);
