// The two producers that sit in front of the operator set inside a DeepSeek-V3.2 layer:
//   - the FP8 activation quantiser that makes the MoE's `hidden_states` (e4m3) and
//     `hidden_states_scale` ([H/128, tokens], block-major) out of bf16 activations, with the rule of
//     reference/moe-fp8-block-scale/variants/fused_routing_v2/kernel.py:495-503:
//     scale = amax / 448 per 128 consecutive values (1.0 when amax <= 1e-10), q = e4m3(x / scale);
//   - the index-K cache writer that stores new index keys into the indexer's paged cache: per page
//     8448 bytes = 64 x 128 e4m3 values followed by 64 fp32 scales, one scale per token
//     (layout: reference/dsa-topk-indexer/variants/v8_radix_bt256/kernel.py:562, 621-625).
// Both are bandwidth-bound and use the mapping of the RMSNorm kernel: 16 lanes x 16 bytes cover one
// 128-value block, a warp instruction covers two blocks, reductions are four shuffles.
#include "common.cuh"

namespace {

__device__ __forceinline__ float block_amax16(const uint4& v) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) m = fmaxf(m, fmaxf(fabsf(ako::bf16_lo(w[i])), fabsf(ako::bf16_hi(w[i]))));
#pragma unroll
  for (int off = 8; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));  // 16-lane groups
  return m;
}

// 8 bf16 values / scale -> 8 e4m3 bytes (round to nearest even, saturating)
__device__ __forceinline__ uint2 quantize8(const uint4& v, float scale) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
  uint32_t out[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float a = __fdiv_rn(ako::bf16_lo(w[i]), scale), b = __fdiv_rn(ako::bf16_hi(w[i]), scale);
    const uint32_t pair = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    out[i >> 1] |= pair << (16 * (i & 1));
  }
  return make_uint2(out[0], out[1]);
}

// One half-warp per 128-value block; blocks are numbered row-major over [rows, blocks_per_row].
__global__ void __launch_bounds__(256) fp8_quantize_1x128_kernel(const __nv_bfloat16* __restrict__ x,
                                                                 uint8_t* __restrict__ q, float* __restrict__ scale,
                                                                 int64_t rows, int blocks_per_row) {
  const int lane16 = threadIdx.x & 15;
  const int64_t nblocks = rows * blocks_per_row;
  for (int64_t b = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 4; b < ako::round_up(nblocks, 2);
       b += ((int64_t)gridDim.x * blockDim.x) >> 4) {
    const bool live = b < nblocks;   // the partner half-warp of an odd tail still takes part in the shuffles
    uint4 v = make_uint4(0, 0, 0, 0);
    if (live) v = __ldcs(reinterpret_cast<const uint4*>(x + b * 128) + lane16);
    const float amax = block_amax16(v);
    const float s = (amax > 1e-10f) ? __fdiv_rn(amax, 448.0f) : 1.0f;
    if (live) {
      __stcs(reinterpret_cast<uint2*>(q + b * 128) + lane16, quantize8(v, s));
      if (lane16 == 0) {
        const int64_t r = b / blocks_per_row;
        const int kb = (int)(b - r * blocks_per_row);
        scale[(int64_t)kb * rows + r] = s;
      }
    }
  }
}

constexpr int PAGE_TOKENS = 64, KDIM = 128, PAGE_BYTES = PAGE_TOKENS * KDIM + PAGE_TOKENS * 4;

// One half-warp per token: its 128 index-key values become e4m3 with one fp32 scale, written to the
// token's slot of its cache page.
__global__ void __launch_bounds__(256) index_k_cache_write_kernel(const __nv_bfloat16* __restrict__ k,
                                                                 const int32_t* __restrict__ slot_mapping,
                                                                 uint8_t* __restrict__ cache, int64_t tokens,
                                                                 int64_t num_pages) {
  const int lane16 = threadIdx.x & 15;
  const int64_t t = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
  const bool in_range = t < tokens;
  uint4 v = make_uint4(0, 0, 0, 0);
  if (in_range) v = __ldcs(reinterpret_cast<const uint4*>(k + t * KDIM) + lane16);
  const float amax = block_amax16(v);
  const float s = (amax > 1e-10f) ? __fdiv_rn(amax, 448.0f) : 1.0f;
  if (!in_range) return;
  const int64_t slot = slot_mapping[t];
  if (slot < 0 || slot >= num_pages * PAGE_TOKENS) return;   // -1: a padding token, nothing is stored
  uint8_t* page = cache + (slot / PAGE_TOKENS) * PAGE_BYTES;
  const int in_page = (int)(slot % PAGE_TOKENS);
  *(reinterpret_cast<uint2*>(page + in_page * KDIM) + lane16) = quantize8(v, s);
  if (lane16 == 0) reinterpret_cast<float*>(page + PAGE_TOKENS * KDIM)[in_page] = s;
}

}  // namespace

extern "C" int ako4x_fp8_quantize_1x128(const void* x, void* q, float* scale, int64_t rows, int64_t cols,
                                        void* stream) {
  if (rows < 0 || cols < 0 || (cols % 128) != 0 || cols > (1 << 24) || rows > (1LL << 40)) return AKO4X_EINVAL;
  if (rows == 0 || cols == 0) return AKO4X_OK;
  if (!x || !q || !scale) return AKO4X_EINVAL;
  if (((uintptr_t)x & 15) || ((uintptr_t)q & 7)) return AKO4X_EINVAL;
  const int64_t nblocks = rows * (cols / 128);
  int64_t grid = ako::cdiv(nblocks, 16);
  const int64_t cap = (int64_t)ako::sm_count() * 16;   // grid-stride above this: enough CTAs to fill the GPU
  if (grid > cap) grid = cap;
  fp8_quantize_1x128_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (uint8_t*)q, scale, rows, (int)(cols / 128));
  AKO_CHECK_LAUNCH();
  return AKO4X_OK;
}

extern "C" int ako4x_dsa_index_k_cache_write(const void* k, const int32_t* slot_mapping, void* k_index_cache,
                                             int64_t tokens, int64_t num_cache_pages, void* stream) {
  if (tokens < 0 || num_cache_pages < 0 || tokens > (1LL << 31)) return AKO4X_EINVAL;
  if (tokens == 0) return AKO4X_OK;
  if (!k || !slot_mapping || !k_index_cache) return AKO4X_EINVAL;
  if (((uintptr_t)k & 15) || ((uintptr_t)k_index_cache & 15)) return AKO4X_EINVAL;
  index_k_cache_write_kernel<<<(unsigned)ako::cdiv(tokens, 16), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)k, slot_mapping, (uint8_t*)k_index_cache, tokens, num_cache_pages);
  AKO_CHECK_LAUNCH();
  return AKO4X_OK;
}
