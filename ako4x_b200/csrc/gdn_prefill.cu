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
// sequence), four compute warps own 16 or 8 rows of one (sequence, head) -- 64 or 128 CTAs per
// sequence --, q_t / k_t pass through shared memory as fp32 in double-buffered chunks of 16 tokens
// that a fifth warp stages one chunk ahead (it also stores the finished chunk's outputs). The serial chain per token is one short dot product, three or four
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
constexpr int P_CONSUMERS = 128;    // 4 warps; a row is held by LPR lanes, 32 / LPR rows per warp
constexpr int P_THREADS = 160;      // + one producer warp that stages the next chunk and stores the last one's outputs

// The producer warp's work for one 16-token chunk `c` of the sequence [t0, t1): q and k of head hq
// as fp32 into kq[token][k | q][128] (token r is one coalesced 512-byte read, lane L converts its 16
// bytes and writes 32 consecutive bytes: no bank conflict), the v values of the CTA's ROWS rows,
// and per token the gate pair: gate[token] = g (or log2 g when LOG2) and beta[token]. Tokens past
// the end of the sequence are staged as nothing-happens tokens (k = q = v = 0, g = 1, beta = 0).
template <int ROWS, bool LOG2>
__device__ __forceinline__ void gdn_stage_chunk(int lane, int c, int64_t t0, int64_t t1, int hq, int h, int rg,
                                                const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                const __nv_bfloat16* __restrict__ v, const __nv_bfloat16* __restrict__ a,
                                                const __nv_bfloat16* __restrict__ b, float neg_A, float dtb,
                                                float (*kq)[2][P_D], float* gate, float* beta, float (*vs)[ROWS]) {
  const int64_t tb = t0 + (int64_t)c * P_CHUNK;
  uint4 w[P_CHUNK];
#pragma unroll
  for (int r = 0; r < P_CHUNK; ++r) {
    w[r] = make_uint4(0u, 0u, 0u, 0u);
    if (tb + r < t1) {
      const __nv_bfloat16* src = ((lane < 16) ? k : q) + ((tb + r) * P_HQ + hq) * P_D + (lane & 15) * 8;
      w[r] = __ldg(reinterpret_cast<const uint4*>(src));
    }
  }
  // lanes 0-15: the v values of token `lane`; lanes 0-15 also a, lanes 16-31 b of token lane & 15
  const int tok = lane & 15;
  const bool valid = tb + tok < t1;
  uint4 vw[ROWS / 8];
#pragma unroll
  for (int i = 0; i < ROWS / 8; ++i) {
    vw[i] = make_uint4(0u, 0u, 0u, 0u);
    if (valid && lane < 16) vw[i] = __ldg(reinterpret_cast<const uint4*>(v + ((tb + tok) * P_HV + h) * P_D + rg * ROWS) + i);
  }
  unsigned short graw = 0;
  if (valid) graw = __ldg(reinterpret_cast<const unsigned short*>(((lane < 16) ? a : b) + (tb + tok) * P_HV + h));
#pragma unroll
  for (int r = 0; r < P_CHUNK; ++r) {
    float* dst = &kq[r][lane >> 4][(lane & 15) * 8];
    *reinterpret_cast<float4*>(dst) = make_float4(ako::bf16_lo(w[r].x), ako::bf16_hi(w[r].x), ako::bf16_lo(w[r].y), ako::bf16_hi(w[r].y));
    *reinterpret_cast<float4*>(dst + 4) = make_float4(ako::bf16_lo(w[r].z), ako::bf16_hi(w[r].z), ako::bf16_lo(w[r].w), ako::bf16_hi(w[r].w));
  }
  if (lane < 16) {
#pragma unroll
    for (int i = 0; i < ROWS / 8; ++i) {
      const uint32_t x[4] = {vw[i].x, vw[i].y, vw[i].z, vw[i].w};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        vs[tok][8 * i + 2 * u] = ako::bf16_lo(x[u]);
        vs[tok][8 * i + 2 * u + 1] = ako::bf16_hi(x[u]);
      }
    }
    const float y = __uint_as_float((uint32_t)graw << 16) + dtb;
    const float sp = (y > 20.f) ? y : log1pf(expf(y));
    gate[tok] = !valid ? (LOG2 ? 0.f : 1.f) : (LOG2 ? neg_A * 1.4426950408889634f * sp : expf(neg_A * sp));
  } else {
    beta[tok] = valid ? 1.f / (1.f + expf(-__uint_as_float((uint32_t)graw << 16))) : 0.f;
  }
}

// The producer's other job: the bf16 outputs of a finished chunk (ROWS values per token) to global memory.
template <int ROWS>
__device__ __forceinline__ void gdn_store_chunk(int lane, int c, int64_t t0, int len, int h, int rg,
                                                const __nv_bfloat16 (*so)[ROWS], __nv_bfloat16* __restrict__ out) {
  constexpr int PIECES = ROWS / 8;
  const int ntok = min(P_CHUNK, len - c * P_CHUNK);
  for (int idx = lane; idx < ntok * PIECES; idx += 32) {
    const int j = idx / PIECES, part = idx % PIECES;
    const int64_t t = t0 + (int64_t)c * P_CHUNK + j;
    *reinterpret_cast<uint4*>(out + (t * P_HV + h) * P_D + rg * ROWS + part * 8) = *reinterpret_cast<const uint4*>(&so[j][part * 8]);
  }
}

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
  __shared__ __align__(16) __nv_bfloat16 s_out[2][P_CHUNK][P_ROWS];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool producer = warp == P_CONSUMERS / 32;
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
    if (!producer) {
#pragma unroll
      for (int i = 0; i < NI; ++i) *reinterpret_cast<float4*>(ns + ISTR * i) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    return;
  }
  if (producer) {
#pragma unroll
    for (int i = 0; i < EPL; ++i) S[i] = 0.f;
  } else if (state != nullptr) {
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

  // One warp runs ahead of the four that hold the state: while they compute chunk c it stores the
  // outputs of chunk c - 1 and stages chunk c + 1 (global loads, conversion, gate math), so that a
  // chunk costs the compute warps one barrier and nothing else.
  const int chunks = (len + P_CHUNK - 1) / P_CHUNK;
  if (producer) gdn_stage_chunk<P_ROWS, false>(lane, 0, t0, t1, hq, h, rg, q, k, v, a, b, neg_A, dtb, s_kq[0], s_g[0], s_beta[0], s_v[0]);
  __syncthreads();
  for (int c = 0; c < chunks; ++c) {
    const int buf = c & 1;
    if (producer) {
      if (c > 0) gdn_store_chunk<P_ROWS>(lane, c - 1, t0, len, h, rg, s_out[buf ^ 1], out);
      if (c + 1 < chunks)
        gdn_stage_chunk<P_ROWS, false>(lane, c + 1, t0, t1, hq, h, rg, q, k, v, a, b, neg_A, dtb, s_kq[buf ^ 1], s_g[buf ^ 1],
                                       s_beta[buf ^ 1], s_v[buf ^ 1]);
      __syncthreads();
      continue;
    }
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
      if (seg == 0) s_out[buf][j][row_local] = __float2bfloat16_rn(scale * (g * e2 + e3 * delta));
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
    __syncthreads();                       // chunk c done, chunk c + 1 staged
  }
  if (producer) {
    gdn_store_chunk<P_ROWS>(lane, chunks - 1, t0, len, h, rg, s_out[(chunks - 1) & 1], out);
    return;
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
  // serial chain, but does more work per token in total: it wins while SMs would otherwise idle.
  // Measured, chunked against token by token: 1 x 8 192 tokens 1.00 against 1.40 ms, 2 x 4 096 0.79
  // against 0.90, 4 x 2 048 0.80 against 0.74, 64 x 128 0.64 against 0.51: used for one or two sequences.
  if (workspace != nullptr && num_seqs <= 2) {
    // chunked form: the token-only tables first, then 128 CTAs per sequence over 16-token chunks
    if (((uintptr_t)workspace & 15) || workspace_bytes < ako4x_gdn_prefill_workspace_bytes(total_tokens, num_seqs))
      return AKO4X_EWORKSPACE;
    if (total_tokens > 0) {
      gdn_gram_kernel<<<dim3((unsigned)num_seqs, P_HQ, C_GRAM_Z), 256, 0, (cudaStream_t)stream>>>(
          (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, cu_seqlens, (float*)workspace);
      AKO_CHECK_LAUNCH();
    }
    if (num_seqs == 1) {
      gdn_prefill_chunk_kernel<false><<<dim3(P_D / C_ROWS, P_HV, 1), P_THREADS, 0, (cudaStream_t)stream>>>(
          (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, state, A_log, (const __nv_bfloat16*)a,
          dt_bias, (const __nv_bfloat16*)b, cu_seqlens, scale, (__nv_bfloat16*)out, new_state, (const float*)workspace);
    } else {
      gdn_prefill_chunk_kernel<true><<<dim3(P_D / C_ROWS, P_HV, (unsigned)num_seqs), P_THREADS, 0, (cudaStream_t)stream>>>(
          (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, state, A_log, (const __nv_bfloat16*)a,
          dt_bias, (const __nv_bfloat16*)b, cu_seqlens, scale, (__nv_bfloat16*)out, new_state, (const float*)workspace);
    }
    AKO_CHECK_LAUNCH();
    return AKO4X_OK;
  }
  // Three sequences or more (or no workspace): token by token. One or two sequences: 16 lanes per
  // row (128 CTAs per sequence, the shorter serial chain per token); more: 8 lanes per row (half the
  // instructions per row and token; measured better from three sequences on, 4 x 2 048: 675 against 734 us).
  if (num_seqs <= 2) {
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
