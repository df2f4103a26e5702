// Gated Delta Net decode, one token per sequence (definition gdn_decode_qk4_v8_d128_k_last):
// 4 q/k heads, 8 v heads (v head h uses q/k head h / 2), head size 128, recurrent state fp32
// [batch, 8, 128 (v), 128 (k)] with the k dimension last.
//   g = exp(-exp(A_log[h]) * softplus(a + dt_bias[h])),  beta = sigmoid(b)
//   kdot[v] = sum_k S[v,k] k[k]        qs[v] = sum_k S[v,k] q[k]        qk = sum_k q[k] k[k]
//   delta[v] = beta * (v[v] - g * kdot[v])
//   S'[v,k] = g * S[v,k] + delta[v] * k[k]
//   out[v]  = scale * (g * qs[v] + qk * delta[v])          ( = scale * q . S' )
// which is the delta rule of reference/gdn-decode/variants/cuda_bv32_register_resident/kernel.py
// (:257-326) written per state row. The operator is a 128 KB read-modify-write per (sequence,
// head): HBM-bound. A warp owns 8 state rows; a lane holds four consecutive k of every row (one
// 16-byte load per row, all eight issued before anything is used), so the state passes through
// registers once. The 16 dot products of a warp (8 rows x {k, q}) are reduced together by a
// halving butterfly (17 shuffles instead of 80); the lane that ends up with a row's pair computes
// delta and the output value, and delta goes back to all lanes with one shuffle per row.
#include "common.cuh"

namespace {

constexpr int HQ = 4, HV = 8, D = 128;
constexpr int ROWS_PER_WARP = 8;

template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32) gdn_decode_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
    const float* __restrict__ state, const float* __restrict__ A_log, const __nv_bfloat16* __restrict__ a,
    const float* __restrict__ dt_bias, const __nv_bfloat16* __restrict__ b, float scale,
    __nv_bfloat16* __restrict__ out, float* __restrict__ new_state) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // one linear grid: the row groups of a (sequence, head) are neighbours (they share q and k)
  constexpr int GROUPS = D / ROWS_PER_WARP / WARPS;
  const int bh = blockIdx.x / GROUPS;        // sequence * 8 + v head
  const int bi = bh / HV, h = bh % HV;
  const int row0 = ((blockIdx.x % GROUPS) * WARPS + warp) * ROWS_PER_WARP;
  const int64_t sbase = ((int64_t)bh * D + row0) * D + lane * 4;

  // the state rows first: everything else hides behind these loads
  float4 s[ROWS_PER_WARP];
  if (state != nullptr) {
#pragma unroll
    for (int r = 0; r < ROWS_PER_WARP; ++r) s[r] = __ldcs(reinterpret_cast<const float4*>(state + sbase + (int64_t)r * D));
  } else {
#pragma unroll
    for (int r = 0; r < ROWS_PER_WARP; ++r) s[r] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const int hq = h / (HV / HQ);
  const uint2 qr = __ldg(reinterpret_cast<const uint2*>(q + ((int64_t)bi * HQ + hq) * D + lane * 4));
  const uint2 kr = __ldg(reinterpret_cast<const uint2*>(k + ((int64_t)bi * HQ + hq) * D + lane * 4));
  const float qv[4] = {ako::bf16_lo(qr.x), ako::bf16_hi(qr.x), ako::bf16_lo(qr.y), ako::bf16_hi(qr.y)};
  const float kv[4] = {ako::bf16_lo(kr.x), ako::bf16_hi(kr.x), ako::bf16_lo(kr.y), ako::bf16_hi(kr.y)};
  const float x = __bfloat162float(a[bh]) + dt_bias[h];
  const float softplus = (x > 20.f) ? x : log1pf(expf(x));
  const float g = expf(-expf(A_log[h]) * softplus);
  const float beta = 1.f / (1.f + expf(-__bfloat162float(b[bh])));
  // v of the row this lane will finish (see below): rows are spread over lanes by the butterfly

  // partial dot products of this lane: index 2r = row r with k, 2r+1 = row r with q
  float part[16];
#pragma unroll
  for (int r = 0; r < ROWS_PER_WARP; ++r) {
    part[2 * r] = s[r].x * kv[0] + s[r].y * kv[1] + s[r].z * kv[2] + s[r].w * kv[3];
    part[2 * r + 1] = s[r].x * qv[0] + s[r].y * qv[1] + s[r].z * qv[2] + s[r].w * qv[3];
  }
  float qk = qv[0] * kv[0] + qv[1] * kv[1] + qv[2] * kv[2] + qv[3] * kv[3];
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) qk += __shfl_xor_sync(0xffffffffu, qk, off);
  // halving butterfly: 8 + 4 + 2 + 1 exchanges leave one of the 16 sums in every lane (reduced over
  // 16 lanes), a last full exchange completes it. The index a lane holds is bits 4..1 of its id.
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4, b1 = lane & 2;
  float a8[8], a4[4], a2[2], a1;
#pragma unroll
  for (int j = 0; j < 8; ++j) a8[j] = (b4 ? part[8 + j] : part[j]) + __shfl_xor_sync(0xffffffffu, b4 ? part[j] : part[8 + j], 16);
#pragma unroll
  for (int j = 0; j < 4; ++j) a4[j] = (b3 ? a8[4 + j] : a8[j]) + __shfl_xor_sync(0xffffffffu, b3 ? a8[j] : a8[4 + j], 8);
#pragma unroll
  for (int j = 0; j < 2; ++j) a2[j] = (b2 ? a4[2 + j] : a4[j]) + __shfl_xor_sync(0xffffffffu, b2 ? a4[j] : a4[2 + j], 4);
  a1 = (b1 ? a2[1] : a2[0]) + __shfl_xor_sync(0xffffffffu, b1 ? a2[0] : a2[1], 2);
  a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
  // lane L now holds sum number idx = (L >> 1) & 15: row idx >> 1, with k (idx even) or q (idx odd).
  // The q sum of a row sits two lanes above its k sum.
  const int idx = (lane >> 1) & 15;
  const int my_row = idx >> 1;
  const float other = __shfl_xor_sync(0xffffffffu, a1, 2);   // the partner sum of the same row
  const float kdot = (idx & 1) ? other : a1;
  const float qs = (idx & 1) ? a1 : other;
  const float vval = __bfloat162float(v[(int64_t)bh * D + row0 + my_row]);
  const float delta_mine = beta * (vval - g * kdot);
  if ((lane & 3) == 0)   // one lane per row writes the output value
    out[(int64_t)bh * D + row0 + my_row] = __float2bfloat16_rn(scale * (g * qs + qk * delta_mine));

#pragma unroll
  for (int r = 0; r < ROWS_PER_WARP; ++r) {
    const float delta = __shfl_sync(0xffffffffu, delta_mine, 4 * r);   // lane 4r holds row r
    float4 o;
    o.x = fmaf(g, s[r].x, delta * kv[0]);
    o.y = fmaf(g, s[r].y, delta * kv[1]);
    o.z = fmaf(g, s[r].z, delta * kv[2]);
    o.w = fmaf(g, s[r].w, delta * kv[3]);
    __stcs(reinterpret_cast<float4*>(new_state + sbase + (int64_t)r * D), o);
  }
}

}  // namespace

extern "C" int ako4x_gdn_decode(const void* q, const void* k, const void* v, const float* state, const float* A_log,
                                const void* a, const float* dt_bias, const void* b, float scale, void* out,
                                float* new_state, int64_t batch, void* stream) {
  if (batch < 0 || batch > (1 << 20)) return AKO4X_EINVAL;
  if (batch == 0) return AKO4X_OK;
  if (!q || !k || !v || !A_log || !a || !dt_bias || !b || !out || !new_state) return AKO4X_EINVAL;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)state | (uintptr_t)new_state) & 15) return AKO4X_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  const __nv_bfloat16 *qp = (const __nv_bfloat16*)q, *kp = (const __nv_bfloat16*)k, *vp = (const __nv_bfloat16*)v;
  const __nv_bfloat16 *ap = (const __nv_bfloat16*)a, *bp = (const __nv_bfloat16*)b;
  // few sequences: one warp per CTA so that the 16 x batch x 8 row groups spread over all SMs;
  // many: four warps per CTA
  if (batch * HV * (D / ROWS_PER_WARP) <= 4096) {
    gdn_decode_kernel<1><<<(unsigned)(batch * HV * (D / ROWS_PER_WARP)), 32, 0, st>>>(
        qp, kp, vp, state, A_log, ap, dt_bias, bp, scale, (__nv_bfloat16*)out, new_state);
  } else {
    gdn_decode_kernel<4><<<(unsigned)(batch * HV * (D / ROWS_PER_WARP / 4)), 128, 0, st>>>(
        qp, kp, vp, state, A_log, ap, dt_bias, bp, scale, (__nv_bfloat16*)out, new_state);
  }
  AKO_CHECK_LAUNCH();
  return AKO4X_OK;
}
