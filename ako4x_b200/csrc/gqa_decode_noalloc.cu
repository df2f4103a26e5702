// Paged GQA decode for callers that cannot provide scratch memory.
//
// The regular entry point needs a caller-allocated workspace for its split-KV partials. Two kinds
// of caller have none to give: a plug-in host that hands an operator only its input and output
// tensors (destination-passing style, no workspace argument and no allocator handle), and a
// serving process that has committed all free HBM to its KV-cache pool at start-up, where a
// cudaMalloc in the decode loop fails or stalls behind the pool. For them this file keeps a fixed
// scratch array inside the library image and runs the same kernels on it.
//
// Costs and rules, all consequences of the scratch being one static array:
//   * every GPU that loads the library holds kScratchBytes (16 MiB) of device memory until exit;
//   * a call whose partials would not fit is refused with AKO4X_ETOOLARGE, nothing is launched;
//   * all calls on a device share the array, so two calls that may overlap on the GPU (different
//     streams, or different host threads) race; serialise them on one stream;
//   * the array keeps the previous call's contents, which is harmless here: every partial that
//     the merge kernel reads is written by the split kernel of the same call, nothing must start
//     at zero;
//   * the first call on each device resolves the array's device address (cudaGetSymbolAddress).
//     Make that first call during start-up, before any stream capture begins.
#include <atomic>

#include "common.cuh"

namespace {

constexpr size_t kScratchBytes = 16u << 20;

// In host code this name is only a handle for the runtime, not a device address: it must go
// through cudaGetSymbolAddress before a kernel can be given the memory.
static __device__ __align__(256) unsigned char g_gqa_scratch[kScratchBytes];

// Device address of g_gqa_scratch on the current device, resolved once per device.
int scratch_address(void** out) {
  static std::atomic<void*> addr[64] = {};  // host threads may race here: the value is idempotent
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return AKO4X_ELAUNCH;
  if (addr[dev].load(std::memory_order_acquire) == nullptr) {
    void* p = nullptr;
    // the device `dev` is current here, so the address belongs to its copy of the array
    if (cudaGetSymbolAddress(&p, g_gqa_scratch) != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();
      return AKO4X_ELAUNCH;
    }
    addr[dev].store(p, std::memory_order_release);
  }
  *out = addr[dev].load(std::memory_order_acquire);
  return AKO4X_OK;
}

}  // namespace

extern "C" size_t ako4x_gqa_paged_decode_noalloc_max_scratch_bytes(void) { return kScratchBytes; }

extern "C" int ako4x_gqa_paged_decode_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                              const int32_t* kv_indptr, const int32_t* kv_indices,
                                              float sm_scale, void* o, float* lse, int64_t batch,
                                              int64_t num_kv_indices, int64_t page_size,
                                              void* stream) {
  if (batch < 0 || num_kv_indices < 0 || page_size < 1) return AKO4X_EINVAL;
  const size_t need = ako4x_gqa_paged_decode_workspace_bytes(batch, num_kv_indices, page_size);
  if (need > kScratchBytes) return AKO4X_ETOOLARGE;
  void* scratch = nullptr;
  if (need > 0) {
    const int rc = scratch_address(&scratch);
    if (rc != AKO4X_OK) return rc;
  }
  return ako4x_gqa_paged_decode(q, k_cache, v_cache, kv_indptr, kv_indices, sm_scale, o, lse, batch,
                                num_kv_indices, page_size, scratch, need, stream);
}
