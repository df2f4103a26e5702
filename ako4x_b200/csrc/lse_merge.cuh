// Split-KV partial format and merge shared by the attention kernels.
// A partial is (m, l, acc[D]) in the base-2 domain: m = running max of logit*log2(e),
// l = sum 2^(logit2 - m), acc = sum 2^(logit2 - m) * v. An empty partial is (m=-inf, l=0).
// Merged: M = max m_s, L = sum l_s 2^(m_s-M), o = sum acc_s 2^(m_s-M) / L, lse = M + log2 L.
#pragma once
#include "common.cuh"

namespace ako {

// One block per (row, head) pair `rh`; blockDim.x * VEC == D. partial_acc is laid out as
// [rh][split][D], partial_ml as [rh][split][2].
// The (m, l) pairs are read by all threads at once (one split per thread and pass) and the weights
// 2^(m_s - M) go through shared memory, so the only serial loop left is the accumulation, whose
// loads are independent of one another: a merge over 40 splits used to be 80 dependent L2 round
// trips (10 us for a single-sequence decode). The sums run in the same order as before (L over
// s ascending, acc over s ascending): the results are bit-identical to the serial form.
constexpr int kMergeChunk = 128;
template <int D, int VEC>
__global__ void lse_merge_kernel(const float* __restrict__ partial_acc,
                                 const float* __restrict__ partial_ml, __nv_bfloat16* __restrict__ o,
                                 float* __restrict__ lse, int num_splits) {
  constexpr int NT = D / VEC;
  __shared__ float s_w[kMergeChunk], s_l[kMergeChunk];
  __shared__ float s_red[32];
  pdl_wait();
  const int tid = threadIdx.x;
  const int64_t rh = blockIdx.x;
  const float* ml = partial_ml + rh * num_splits * 2;
  float M = -INFINITY;
  for (int s = tid; s < num_splits; s += NT) M = fmaxf(M, ml[2 * s]);
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
  if constexpr (NT > 32) {
    if ((tid & 31) == 0) s_red[tid >> 5] = M;
    __syncthreads();
    M = s_red[0];
#pragma unroll
    for (int w = 1; w < NT / 32; ++w) M = fmaxf(M, s_red[w]);
  }
  float L = 0.f;
  float acc[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
  const float* pa = partial_acc + rh * num_splits * D + tid * VEC;
  if (M > -INFINITY) {
    for (int base = 0; base < num_splits; base += kMergeChunk) {
      const int cnt = min(kMergeChunk, num_splits - base);
      if (base > 0) __syncthreads();            // the previous chunk's weights are no longer read
      for (int i = tid; i < cnt; i += NT) {
        const float2 x = *reinterpret_cast<const float2*>(ml + 2 * (base + i));
        const float w = (x.x == -INFINITY) ? 0.f : exp2f(x.x - M);
        s_w[i] = w;
        s_l[i] = (x.x == -INFINITY) ? 0.f : x.y;
      }
      __syncthreads();
      const float* pc = pa + (int64_t)base * D;
      int i = 0;
      if constexpr (VEC == 4) {
        for (; i + 4 <= cnt; i += 4) {          // four independent 16-byte loads in flight
          float4 p4[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) p4[u] = *reinterpret_cast<const float4*>(pc + (int64_t)(i + u) * D);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float w = s_w[i + u];
            L = fmaf(s_l[i + u], w, L);
            if (w > 0.f) {                      // an empty partial's acc is undefined: never touched
              acc[0] = fmaf(p4[u].x, w, acc[0]);
              acc[1] = fmaf(p4[u].y, w, acc[1]);
              acc[2] = fmaf(p4[u].z, w, acc[2]);
              acc[3] = fmaf(p4[u].w, w, acc[3]);
            }
          }
        }
      }
      for (; i < cnt; ++i) {
        const float w = s_w[i];
        L = fmaf(s_l[i], w, L);
        if (w > 0.f) {
#pragma unroll
          for (int v = 0; v < VEC; ++v) acc[v] = fmaf(pc[(int64_t)i * D + v], w, acc[v]);
        }
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
