// Gated Delta Net prefill (definition gdn_prefill_qk4_v8_d128_k_last): variable-length sequences
// packed along the token axis, 4 q/k heads, 8 v heads, head size 128, fp32 state
// [sequence, 8, 128 (v), 128 (k)] with k last. Per token t of a sequence, per v head:
//   g = exp(-exp(A_log) softplus(a_t + dt_bias)),  beta = sigmoid(b_t)
//   delta[v] = beta (v_t[v] - g S[v,:].k_t),  S[v,:] = g S[v,:] + delta[v] k_t,
//   out_t[v] = scale S[v,:].q_t = scale (g S_old[v,:].q_t + (q_t.k_t) delta[v])
// (the recurrence reference/gdn-prefill/variants/cuda_graph_v5/kernel.py evaluates in chunked form,
// :1333-1400 for its entry point). The rows S[v,:] of a state never interact, so this first
// version runs the recurrence as it is written, token by token, with all the parallelism the rows
// give: a row is held by 8 or 16 lanes (16 or 8 state values each, in registers for the whole
// sequence), a CTA of four warps owns 16 or 8 rows of one (sequence, head) -- 64 or 128 CTAs per
// sequence --, q_t / k_t pass through shared memory as fp32 in double-buffered chunks of 16 tokens
// fetched one chunk ahead. The serial chain per token is one short dot product, three or four
// shuffle levels and the update; measured about 270 cycles per token and 100 more per token of
// chunk hand-over, so a single sequence of 8 192 tokens takes 1.5 ms. The chunked form of the
// recurrence (gdn_prefill_chunk.cuh, fp32 on the CUDA cores) is used for one or two sequences;
// a tensor-core form is not built. The state crosses HBM once each
// way; outputs leave in 16- or 32-byte pieces per token and CTA. Processing two tokens per
// reduction round (both products taken from the same state, the second delta corrected with
// k1.k2) was built and measured slower (1.97 ms against 1.52 ms): eight values per shuffle level.
#include "common.cuh"

namespace {

constexpr int P_HQ = 4, P_HV = 8, P_D = 128;
constexpr int P_CHUNK = 16;         // tokens per staging chunk
constexpr int P_THREADS = 128;      // 4 warps; a row is held by LPR lanes, 32 / LPR rows per warp

struct Staged {       // what one thread fetches for one chunk: 32 of the chunk's 4096 q/k values
  uint4 w[4];
};

template <int LPR>
__global__ void __launch_bounds__(P_THREADS) gdn_prefill_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
    const float* __restrict__ state, const float* __restrict__ A_log, const __nv_bfloat16* __restrict__ a,
    const float* __restrict__ dt_bias, const __nv_bfloat16* __restrict__ b, const int64_t* __restrict__ cu_seqlens,
    float scale, __nv_bfloat16* __restrict__ out, float* __restrict__ new_state) {
  constexpr int EPL = P_D / LPR;            // state values per lane (16 or 8)
  constexpr int NI = EPL / 4;               // float4 pieces per lane
  constexpr int ISTR = 4 * LPR;             // elements between a lane's pieces
  constexpr int RPW = 32 / LPR;             // rows per warp
  constexpr int P_ROWS = 4 * RPW;           // rows per CTA (16 or 8)
  __shared__ __align__(16) float s_kq[2][P_CHUNK][2][P_D];     // [buffer][token][k | q][128]  32 KB
  __shared__ float s_g[2][P_CHUNK], s_beta[2][P_CHUNK];
  __shared__ float s_v[2][P_CHUNK][P_ROWS];
  __shared__ __align__(16) __nv_bfloat16 s_out[P_CHUNK][P_ROWS];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rg = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
  const int hq = h / (P_HV / P_HQ);
  const int64_t t0 = cu_seqlens[seq], t1 = cu_seqlens[seq + 1];
  const int len = (int)(t1 - t0);
  const int row_local = warp * RPW + lane / LPR;
  const int row = rg * P_ROWS + row_local;
  // lane `seg` of a row holds k elements ISTR i + 4 seg + c (c = 0..3): for a given i the lanes of
  // a row read consecutive bytes, from global memory (coalesced) and from shared memory (no bank
  // conflict; the other rows of the warp read the same addresses, a broadcast)
  const int seg = lane % LPR;
  float* ns = new_state + (((int64_t)seq * P_HV + h) * P_D + row) * P_D + seg * 4;

  float S[EPL];
  if (len <= 0) {   // the definition leaves the new state of an empty sequence at zero
#pragma unroll
    for (int i = 0; i < NI; ++i) *reinterpret_cast<float4*>(ns + ISTR * i) = make_float4(0.f, 0.f, 0.f, 0.f);
    return;
  }
  if (state != nullptr) {
    const float* sp = state + (((int64_t)seq * P_HV + h) * P_D + row) * P_D + seg * 4;
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const float4 x = __ldcs(reinterpret_cast<const float4*>(sp + ISTR * i));
      S[4 * i] = x.x; S[4 * i + 1] = x.y; S[4 * i + 2] = x.z; S[4 * i + 3] = x.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < EPL; ++i) S[i] = 0.f;
  }
  const float neg_A = -expf(A_log[h]);
  const float dtb = dt_bias[h];

  // staging: thread `tid` fetches, for chunk token j = tid / 8 and part = tid % 8, 16 k values and
  // 16 q values (elements part*16 .. +15 of head hq), as 2 x 16 bytes each
  const int st_tok = tid >> 3, st_part = tid & 7;
  // fetch() only issues loads (nothing here may depend on a loaded value: the thread would wait
  // for HBM before it starts the chunk it already has); stash() converts and computes the gates
  // after that chunk is done.
  auto fetch = [&](int c, Staged& r, uint32_t& vraw, uint32_t& graw) {
    const int64_t t = t0 + (int64_t)c * P_CHUNK + st_tok;
    r.w[0] = r.w[1] = r.w[2] = r.w[3] = make_uint4(0u, 0u, 0u, 0u);
    vraw = 0u;
    graw = 0u;
    if (t < t1) {
      const uint4* kp = reinterpret_cast<const uint4*>(k + (t * P_HQ + hq) * P_D + st_part * 16);
      const uint4* qp = reinterpret_cast<const uint4*>(q + (t * P_HQ + hq) * P_D + st_part * 16);
      r.w[0] = __ldg(kp); r.w[1] = __ldg(kp + 1); r.w[2] = __ldg(qp); r.w[3] = __ldg(qp + 1);
      // the 8 threads of a token fetch its v values, two each; thread 0 the gate input a, thread 1 b
      if (st_part * 2 < P_ROWS)
        vraw = __ldg(reinterpret_cast<const uint32_t*>(v + (t * P_HV + h) * P_D + rg * P_ROWS + st_part * 2));
      if (st_part == 0) graw = __ldg(reinterpret_cast<const unsigned short*>(a + t * P_HV + h));
      if (st_part == 1) graw = __ldg(reinterpret_cast<const unsigned short*>(b + t * P_HV + h));
    }
  };
  auto stash = [&](int buf, const Staged& r, uint32_t vraw, uint32_t graw) {
    float* kd = &s_kq[buf][st_tok][0][st_part * 16];
    float* qd = &s_kq[buf][st_tok][1][st_part * 16];
    const uint32_t kw[8] = {r.w[0].x, r.w[0].y, r.w[0].z, r.w[0].w, r.w[1].x, r.w[1].y, r.w[1].z, r.w[1].w};
    const uint32_t qw[8] = {r.w[2].x, r.w[2].y, r.w[2].z, r.w[2].w, r.w[3].x, r.w[3].y, r.w[3].z, r.w[3].w};
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      *reinterpret_cast<float4*>(kd + 2 * i) = make_float4(ako::bf16_lo(kw[i]), ako::bf16_hi(kw[i]), ako::bf16_lo(kw[i + 1]), ako::bf16_hi(kw[i + 1]));
      *reinterpret_cast<float4*>(qd + 2 * i) = make_float4(ako::bf16_lo(qw[i]), ako::bf16_hi(qw[i]), ako::bf16_lo(qw[i + 1]), ako::bf16_hi(qw[i + 1]));
    }
    if (st_part * 2 < P_ROWS) {
      s_v[buf][st_tok][st_part * 2] = ako::bf16_lo(vraw);
      s_v[buf][st_tok][st_part * 2 + 1] = ako::bf16_hi(vraw);
    }
    const float x = __uint_as_float(graw << 16);
    if (st_part == 0) {
      const float y = x + dtb;
      const float sp = (y > 20.f) ? y : log1pf(expf(y));
      s_g[buf][st_tok] = expf(neg_A * sp);
    }
    if (st_part == 1) s_beta[buf][st_tok] = 1.f / (1.f + expf(-x));
  };

  const int chunks = (len + P_CHUNK - 1) / P_CHUNK;
  Staged r;
  uint32_t vraw, graw;
  fetch(0, r, vraw, graw);
  stash(0, r, vraw, graw);
  __syncthreads();
  for (int c = 0; c < chunks; ++c) {
    const int buf = c & 1;
    if (c + 1 < chunks) fetch(c + 1, r, vraw, graw);     // in flight while this chunk is computed
    const int ntok = min(P_CHUNK, len - c * P_CHUNK);
    // q_t / k_t of the next token are read while the current one is computed: the loads, the q.k
    // product and S.q are off the serial chain (S.k -> three shuffles -> delta -> update)
    auto load_tok = [&](int j, float (&kk)[EPL], float (&qq)[EPL]) {
#pragma unroll
      for (int i = 0; i < NI; ++i) {
        const float4 x = *reinterpret_cast<const float4*>(&s_kq[buf][j][0][ISTR * i + 4 * seg]);
        const float4 y = *reinterpret_cast<const float4*>(&s_kq[buf][j][1][ISTR * i + 4 * seg]);
        kk[4 * i] = x.x; kk[4 * i + 1] = x.y; kk[4 * i + 2] = x.z; kk[4 * i + 3] = x.w;
        qq[4 * i] = y.x; qq[4 * i + 1] = y.y; qq[4 * i + 2] = y.z; qq[4 * i + 3] = y.w;
      }
    };
    auto step = [&](int j, const float (&kk)[EPL], const float (&qq)[EPL]) {
      const float g = s_g[buf][j], beta = s_beta[buf][j], vval = s_v[buf][j][row_local];
      float d1[4] = {0.f, 0.f, 0.f, 0.f}, d2[4] = {0.f, 0.f, 0.f, 0.f}, d3[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < EPL; i += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          d1[u] = fmaf(S[i + u], kk[i + u], d1[u]);
          d2[u] = fmaf(S[i + u], qq[i + u], d2[u]);
          d3[u] = fmaf(kk[i + u], qq[i + u], d3[u]);
        }
      }
      float e1 = (d1[0] + d1[1]) + (d1[2] + d1[3]);
      float e2 = (d2[0] + d2[1]) + (d2[2] + d2[3]);
      float e3 = (d3[0] + d3[1]) + (d3[2] + d3[3]);
#pragma unroll
      for (int off = 1; off < LPR; off <<= 1) {
        e1 += __shfl_xor_sync(0xffffffffu, e1, off);
        e2 += __shfl_xor_sync(0xffffffffu, e2, off);
        e3 += __shfl_xor_sync(0xffffffffu, e3, off);
      }
      const float delta = beta * (vval - g * e1);
#pragma unroll
      for (int i = 0; i < EPL; ++i) S[i] = fmaf(g, S[i], delta * kk[i]);
      if (seg == 0) s_out[j][row_local] = __float2bfloat16_rn(scale * (g * e2 + e3 * delta));
    };
    {
      float kA[EPL], qA[EPL], kB[EPL], qB[EPL];
      load_tok(0, kA, qA);
      for (int j = 0; j < ntok; j += 2) {
        if (j + 1 < ntok) load_tok(j + 1, kB, qB);
        step(j, kA, qA);
        if (j + 1 < ntok) {
          if (j + 2 < ntok) load_tok(j + 2, kA, qA);
          step(j + 1, kB, qB);
        }
      }
    }
    __syncthreads();                       // s_out complete; buffer buf ^ 1 no longer read
    // outputs of the chunk: token j, P_ROWS rows = 32 or 16 bytes, moved in 16-byte pieces
    constexpr int PIECES = P_ROWS / 8;
    if (tid < PIECES * ntok) {
      const int j = tid / PIECES, part = tid % PIECES;
      const int64_t t = t0 + (int64_t)c * P_CHUNK + j;
      *reinterpret_cast<uint4*>(out + (t * P_HV + h) * P_D + rg * P_ROWS + part * 8) =
          *reinterpret_cast<const uint4*>(&s_out[j][part * 8]);
    }
    if (c + 1 < chunks) stash(buf ^ 1, r, vraw, graw);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < NI; ++i)
    __stcs(reinterpret_cast<float4*>(ns + ISTR * i), make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]));
}

#include "gdn_prefill_chunk.cuh"

}  // namespace

extern "C" size_t ako4x_gdn_prefill_workspace_bytes(int64_t total_tokens, int64_t num_seqs) {
  if (total_tokens <= 0 || num_seqs <= 0) return 0;
  return (size_t)(total_tokens / C_TOK + num_seqs + 1) * P_HQ * C_GSTRIDE * sizeof(float);
}

extern "C" int ako4x_gdn_prefill(const void* q, const void* k, const void* v, const float* state, const float* A_log,
                                 const void* a, const float* dt_bias, const void* b, const int64_t* cu_seqlens,
                                 float scale, void* out, float* new_state, int64_t total_tokens, int64_t num_seqs,
                                 void* workspace, size_t workspace_bytes, void* stream) {
  if (total_tokens < 0 || num_seqs < 0 || num_seqs > 65535) return AKO4X_EINVAL;
  if (num_seqs == 0) return AKO4X_OK;
  if (!A_log || !dt_bias || !cu_seqlens || !new_state) return AKO4X_EINVAL;
  if (total_tokens > 0 && (!q || !k || !v || !a || !b || !out)) return AKO4X_EINVAL;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out | (uintptr_t)state | (uintptr_t)new_state) & 15)
    return AKO4X_EINVAL;
  // The chunked form pays per 16 tokens what the token-by-token form pays per 4-5 tokens on its
  // serial chain, but does more work per token in total: it wins while the GPU has idle SMs (one or
  // two sequences: 8 192 tokens in 1.18 ms against 1.52 ms) and loses once every SM holds several
  // CTAs (8 x 1 024: 0.96 against 0.64 ms), so it is used for up to two sequences.
  if (workspace != nullptr && num_seqs <= 2) {
    // chunked form: the token-only tables first, then 128 CTAs per sequence over 16-token chunks
    if (((uintptr_t)workspace & 15) || workspace_bytes < ako4x_gdn_prefill_workspace_bytes(total_tokens, num_seqs))
      return AKO4X_EWORKSPACE;
    if (total_tokens > 0) {
      gdn_gram_kernel<<<dim3((unsigned)num_seqs, P_HQ, C_GRAM_Z), 256, 0, (cudaStream_t)stream>>>(
          (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, cu_seqlens, (float*)workspace);
      AKO_CHECK_LAUNCH();
    }
    gdn_prefill_chunk_kernel<<<dim3(P_D / C_ROWS, P_HV, (unsigned)num_seqs), P_THREADS, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, state, A_log, (const __nv_bfloat16*)a,
        dt_bias, (const __nv_bfloat16*)b, cu_seqlens, scale, (__nv_bfloat16*)out, new_state, (const float*)workspace);
    AKO_CHECK_LAUNCH();
    return AKO4X_OK;
  }
  // Without a workspace: the token-sequential kernel. Few sequences: 16 lanes per row (128 CTAs per
  // sequence, the shorter serial chain per token); many: 8 lanes per row (half the instructions
  // per row and token).
  if (num_seqs * 128 <= 4 * ako::sm_count()) {
    gdn_prefill_kernel<16><<<dim3(P_D / 8, P_HV, (unsigned)num_seqs), P_THREADS, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, state, A_log, (const __nv_bfloat16*)a,
        dt_bias, (const __nv_bfloat16*)b, cu_seqlens, scale, (__nv_bfloat16*)out, new_state);
  } else {
    gdn_prefill_kernel<8><<<dim3(P_D / 16, P_HV, (unsigned)num_seqs), P_THREADS, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, state, A_log, (const __nv_bfloat16*)a,
        dt_bias, (const __nv_bfloat16*)b, cu_seqlens, scale, (__nv_bfloat16*)out, new_state);
  }
  AKO_CHECK_LAUNCH();
  return AKO4X_OK;
}
