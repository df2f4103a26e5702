// Internal interface between mla_attention.cu (C-ABI entry points) and mla_prefill_tc.cu.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

// Scratch the tensor-core prefill needs: a contiguous copy of the keys and a transposed copy of V.
size_t ako_mla_prefill_tc_workspace_bytes(int64_t batch, int64_t num_kv_indices, int64_t page_size);

// Returns an AKO4X_* status. All pointers are device pointers; nothing is read on the host.
int ako_mla_prefill_tc_launch(const void* q_nope, const void* q_pe, const void* ckv_cache, const void* kpe_cache,
                              const int32_t* qo_indptr, const int32_t* kv_indptr, const int32_t* kv_indices,
                              float sm_scale, void* o, float* lse, int64_t total_q, int64_t batch,
                              int64_t num_kv_indices, int64_t page_size, void* workspace, size_t workspace_bytes,
                              cudaStream_t stream);

// Device status word of the kernel's bounded waits (0 = ok); synchronises the device.
int ako_mla_prefill_tc_status();
