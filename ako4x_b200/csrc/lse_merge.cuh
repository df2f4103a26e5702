// Split-KV partial format and merge shared by the attention kernels.
// A partial is (m, l, acc[D]) in the base-2 domain: m = running max of logit*log2(e),
// l = sum 2^(logit2 - m), acc = sum 2^(logit2 - m) * v. An empty partial is (m=-inf, l=0).
// Merged: M = max m_s, L = sum l_s 2^(m_s-M), o = sum acc_s 2^(m_s-M) / L, lse = M + log2 L.
#pragma once
#include "common.cuh"

namespace ako {

// One block per (row, head) pair `rh`; blockDim.x * VEC == D. partial_acc is laid out as
// [rh][split][D], partial_ml as [rh][split][2].
template <int D, int VEC>
__global__ void lse_merge_kernel(const float* __restrict__ partial_acc,
                                 const float* __restrict__ partial_ml, __nv_bfloat16* __restrict__ o,
                                 float* __restrict__ lse, int num_splits) {
  pdl_wait();
  const int64_t rh = blockIdx.x;
  const float* ml = partial_ml + rh * num_splits * 2;
  float M = -INFINITY;
  for (int s = 0; s < num_splits; ++s) M = fmaxf(M, ml[2 * s]);
  float L = 0.f;
  float acc[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
  const float* pa = partial_acc + rh * num_splits * D + threadIdx.x * VEC;
  if (M > -INFINITY) {
    for (int s = 0; s < num_splits; ++s) {
      const float ms = ml[2 * s];
      if (ms == -INFINITY) continue;
      const float w = exp2f(ms - M);
      L = fmaf(ml[2 * s + 1], w, L);
      if constexpr (VEC == 4) {
        const float4 p4 = *reinterpret_cast<const float4*>(pa + (int64_t)s * D);
        acc[0] = fmaf(p4.x, w, acc[0]);
        acc[1] = fmaf(p4.y, w, acc[1]);
        acc[2] = fmaf(p4.z, w, acc[2]);
        acc[3] = fmaf(p4.w, w, acc[3]);
      } else {
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[v] = fmaf(pa[(int64_t)s * D + v], w, acc[v]);
      }
    }
  }
  const float inv = (L > 0.f) ? 1.f / L : 0.f;
  __nv_bfloat16* op = o + rh * D + threadIdx.x * VEC;
  if constexpr (VEC == 4) {
    uint2 pk;
    pk.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
    pk.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
    *reinterpret_cast<uint2*>(op) = pk;
  } else {
#pragma unroll
    for (int v = 0; v < VEC; ++v) op[v] = __float2bfloat16_rn(acc[v] * inv);
  }
  if (threadIdx.x == 0) lse[rh] = (L > 0.f) ? M + log2f(L) : -INFINITY;
}

}  // namespace ako
