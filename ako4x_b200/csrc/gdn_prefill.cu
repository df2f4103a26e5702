// Gated Delta Net prefill (definition gdn_prefill_qk4_v8_d128_k_last): variable-length sequences
// packed along the token axis, 4 q/k heads, 8 v heads, head size 128, fp32 state
// [sequence, 8, 128 (v), 128 (k)] with k last. Per token t of a sequence, per v head:
//   g = exp(-exp(A_log) softplus(a_t + dt_bias)),  beta = sigmoid(b_t)
//   delta[v] = beta (v_t[v] - g S[v,:].k_t),  S[v,:] = g S[v,:] + delta[v] k_t,
//   out_t[v] = scale S[v,:].q_t = scale (g S_old[v,:].q_t + (q_t.k_t) delta[v])
// (the recurrence reference/gdn-prefill/variants/cuda_graph_v5/kernel.py evaluates in chunked form,
// :1333-1400 for its entry point). The rows S[v,:] of a state never interact, so this first
// version runs the recurrence as it is written, token by token, with all the parallelism the rows
// give: a CTA owns 16 rows of one (sequence, head) -- 64 CTAs per sequence --, a row is held by 8
// lanes (16 state values each, in registers for the whole sequence), q_t / k_t pass through shared
// memory as fp32 in double-buffered chunks of 16 tokens fetched one chunk ahead. The serial chain
// per token is one 16-term dot product, three shuffle levels and the update. The state crosses
// HBM once each way; outputs leave in 32-byte pieces per token and CTA.
#include "common.cuh"

namespace {

constexpr int P_HQ = 4, P_HV = 8, P_D = 128;
constexpr int P_ROWS = 16;          // state rows per CTA
constexpr int P_CHUNK = 16;         // tokens per staging chunk
constexpr int P_THREADS = 128;      // 4 warps x 4 rows x 8 lanes

struct Staged {       // what one thread fetches for one chunk: 32 of the chunk's 4096 q/k values
  uint4 w[4];
};

__global__ void __launch_bounds__(P_THREADS) gdn_prefill_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
    const float* __restrict__ state, const float* __restrict__ A_log, const __nv_bfloat16* __restrict__ a,
    const float* __restrict__ dt_bias, const __nv_bfloat16* __restrict__ b, const int64_t* __restrict__ cu_seqlens,
    float scale, __nv_bfloat16* __restrict__ out, float* __restrict__ new_state) {
  __shared__ __align__(16) float s_kq[2][P_CHUNK][2][P_D];     // [buffer][token][k | q][128]  32 KB
  __shared__ float s_g[2][P_CHUNK], s_beta[2][P_CHUNK];
  __shared__ float s_v[2][P_CHUNK][P_ROWS];
  __shared__ __align__(16) __nv_bfloat16 s_out[P_CHUNK][P_ROWS];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rg = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
  const int hq = h / (P_HV / P_HQ);
  const int64_t t0 = cu_seqlens[seq], t1 = cu_seqlens[seq + 1];
  const int len = (int)(t1 - t0);
  const int row_local = warp * 4 + (lane >> 3);        // 0..15
  const int row = rg * P_ROWS + row_local;
  const int seg = lane & 7;                            // k elements seg*16 .. seg*16+15
  float* ns = new_state + (((int64_t)seq * P_HV + h) * P_D + row) * P_D + seg * 16;

  float S[16];
  if (len <= 0) {   // the definition leaves the new state of an empty sequence at zero
#pragma unroll
    for (int i = 0; i < 16; i += 4) *reinterpret_cast<float4*>(ns + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    return;
  }
  if (state != nullptr) {
    const float* sp = state + (((int64_t)seq * P_HV + h) * P_D + row) * P_D + seg * 16;
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
      const float4 x = __ldcs(reinterpret_cast<const float4*>(sp + i));
      S[i] = x.x; S[i + 1] = x.y; S[i + 2] = x.z; S[i + 3] = x.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) S[i] = 0.f;
  }
  const float neg_A = -expf(A_log[h]);
  const float dtb = dt_bias[h];

  // staging: thread `tid` fetches, for chunk token j = tid / 8 and part = tid % 8, 16 k values and
  // 16 q values (elements part*16 .. +15 of head hq), as 2 x 16 bytes each
  const int st_tok = tid >> 3, st_part = tid & 7;
  auto fetch = [&](int c, Staged& r, float& gv, float& bv, float& vv) {
    const int64_t t = t0 + (int64_t)c * P_CHUNK + st_tok;
    if (t < t1) {
      const uint4* kp = reinterpret_cast<const uint4*>(k + (t * P_HQ + hq) * P_D + st_part * 16);
      const uint4* qp = reinterpret_cast<const uint4*>(q + (t * P_HQ + hq) * P_D + st_part * 16);
      r.w[0] = __ldg(kp); r.w[1] = __ldg(kp + 1); r.w[2] = __ldg(qp); r.w[3] = __ldg(qp + 1);
    } else {
      r.w[0] = r.w[1] = r.w[2] = r.w[3] = make_uint4(0u, 0u, 0u, 0u);
    }
    // token j = tid / 8 again for v: the 8 threads of a token fetch its 16 v values, two each
    gv = 0.f; bv = 0.f; vv = 0.f;
    if (t < t1) {
      const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(v + (t * P_HV + h) * P_D + rg * P_ROWS + st_part * 2);
      vv = __bfloat162float(v2.x);
      bv = __bfloat162float(v2.y);   // carried in bv for the store below
      if (st_part == 0) {
        const float x = __bfloat162float(a[t * P_HV + h]) + dtb;
        const float sp = (x > 20.f) ? x : log1pf(expf(x));
        gv = expf(neg_A * sp);
      } else if (st_part == 1) {
        gv = 1.f / (1.f + expf(-__bfloat162float(b[t * P_HV + h])));
      }
    }
  };
  auto stash = [&](int buf, const Staged& r, float gv, float bv, float vv) {
    float* kd = &s_kq[buf][st_tok][0][st_part * 16];
    float* qd = &s_kq[buf][st_tok][1][st_part * 16];
    const uint32_t kw[8] = {r.w[0].x, r.w[0].y, r.w[0].z, r.w[0].w, r.w[1].x, r.w[1].y, r.w[1].z, r.w[1].w};
    const uint32_t qw[8] = {r.w[2].x, r.w[2].y, r.w[2].z, r.w[2].w, r.w[3].x, r.w[3].y, r.w[3].z, r.w[3].w};
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      *reinterpret_cast<float4*>(kd + 2 * i) = make_float4(ako::bf16_lo(kw[i]), ako::bf16_hi(kw[i]), ako::bf16_lo(kw[i + 1]), ako::bf16_hi(kw[i + 1]));
      *reinterpret_cast<float4*>(qd + 2 * i) = make_float4(ako::bf16_lo(qw[i]), ako::bf16_hi(qw[i]), ako::bf16_lo(qw[i + 1]), ako::bf16_hi(qw[i + 1]));
    }
    s_v[buf][st_tok][st_part * 2] = vv;
    s_v[buf][st_tok][st_part * 2 + 1] = bv;
    if (st_part == 0) s_g[buf][st_tok] = gv;
    if (st_part == 1) s_beta[buf][st_tok] = gv;
  };

  const int chunks = (len + P_CHUNK - 1) / P_CHUNK;
  Staged r;
  float gv, bv, vv;
  fetch(0, r, gv, bv, vv);
  stash(0, r, gv, bv, vv);
  __syncthreads();
  for (int c = 0; c < chunks; ++c) {
    const int buf = c & 1;
    if (c + 1 < chunks) fetch(c + 1, r, gv, bv, vv);     // in flight while this chunk is computed
    const int ntok = min(P_CHUNK, len - c * P_CHUNK);
    for (int j = 0; j < ntok; ++j) {
      float kk[16], qq[16];
#pragma unroll
      for (int i = 0; i < 16; i += 4) {
        const float4 x = *reinterpret_cast<const float4*>(&s_kq[buf][j][0][seg * 16 + i]);
        const float4 y = *reinterpret_cast<const float4*>(&s_kq[buf][j][1][seg * 16 + i]);
        kk[i] = x.x; kk[i + 1] = x.y; kk[i + 2] = x.z; kk[i + 3] = x.w;
        qq[i] = y.x; qq[i + 1] = y.y; qq[i + 2] = y.z; qq[i + 3] = y.w;
      }
      const float g = s_g[buf][j], beta = s_beta[buf][j], vval = s_v[buf][j][row_local];
      float d1a = 0.f, d1b = 0.f, d2a = 0.f, d2b = 0.f, d3a = 0.f, d3b = 0.f;
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        d1a = fmaf(S[i], kk[i], d1a); d1b = fmaf(S[i + 1], kk[i + 1], d1b);
        d2a = fmaf(S[i], qq[i], d2a); d2b = fmaf(S[i + 1], qq[i + 1], d2b);
        d3a = fmaf(kk[i], qq[i], d3a); d3b = fmaf(kk[i + 1], qq[i + 1], d3b);
      }
      float d1 = d1a + d1b, d2 = d2a + d2b, d3 = d3a + d3b;
#pragma unroll
      for (int off = 1; off <= 4; off <<= 1) {
        d1 += __shfl_xor_sync(0xffffffffu, d1, off);
        d2 += __shfl_xor_sync(0xffffffffu, d2, off);
        d3 += __shfl_xor_sync(0xffffffffu, d3, off);
      }
      const float delta = beta * (vval - g * d1);
#pragma unroll
      for (int i = 0; i < 16; ++i) S[i] = fmaf(g, S[i], delta * kk[i]);
      if (seg == 0) s_out[j][row_local] = __float2bfloat16_rn(scale * (g * d2 + d3 * delta));
    }
    __syncthreads();                       // s_out complete; buffer buf ^ 1 no longer read
    // outputs of the chunk: token j, 16 rows = 32 bytes; thread tid < 2 * ntok moves 16 bytes
    if (tid < 2 * ntok) {
      const int j = tid >> 1, part = tid & 1;
      const int64_t t = t0 + (int64_t)c * P_CHUNK + j;
      *reinterpret_cast<uint4*>(out + (t * P_HV + h) * P_D + rg * P_ROWS + part * 8) =
          *reinterpret_cast<const uint4*>(&s_out[j][part * 8]);
    }
    if (c + 1 < chunks) stash(buf ^ 1, r, gv, bv, vv);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 16; i += 4) __stcs(reinterpret_cast<float4*>(ns + i), make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]));
}

}  // namespace

extern "C" int ako4x_gdn_prefill(const void* q, const void* k, const void* v, const float* state, const float* A_log,
                                 const void* a, const float* dt_bias, const void* b, const int64_t* cu_seqlens,
                                 float scale, void* out, float* new_state, int64_t total_tokens, int64_t num_seqs,
                                 void* stream) {
  if (total_tokens < 0 || num_seqs < 0 || num_seqs > 65535) return AKO4X_EINVAL;
  if (num_seqs == 0) return AKO4X_OK;
  if (!A_log || !dt_bias || !cu_seqlens || !new_state) return AKO4X_EINVAL;
  if (total_tokens > 0 && (!q || !k || !v || !a || !b || !out)) return AKO4X_EINVAL;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out | (uintptr_t)state | (uintptr_t)new_state) & 15)
    return AKO4X_EINVAL;
  gdn_prefill_kernel<<<dim3(P_D / P_ROWS, P_HV, (unsigned)num_seqs), P_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, state, A_log, (const __nv_bfloat16*)a,
      dt_bias, (const __nv_bfloat16*)b, cu_seqlens, scale, (__nv_bfloat16*)out, new_state);
  AKO_CHECK_LAUNCH();
  return AKO4X_OK;
}
