// Chunked form of the Gated Delta Net prefill recurrence, in fp32 on the CUDA cores; included by
// gdn_prefill.cu inside its anonymous namespace.
//
// For a chunk of C = 16 tokens with state S0 at its start, Lc_i = sum_{l<=i} log2 g_l and
// R_ij = 2^(Lc_i - Lc_j) (the decay between tokens j and i), unrolling
//   delta_i = beta_i (v_i - g_i S_{i-1} k_i),   S_i = g_i S_{i-1} + delta_i k_i^T
// gives, for every state row on its own,
//   delta_i = beta_i (v_i - 2^Lc_i (S0 k_i) - sum_{j<i} R_ij (k_i.k_j) delta_j)      (a triangular solve)
//   out_i   = scale (2^Lc_i (S0 q_i) + sum_{j<=i} R_ij (q_i.k_j) delta_j)
//   S_C     = 2^Lc_C S0 + sum_j R_Cj delta_j k_j^T
// so the only serial part is the 16-step substitution, one shuffle and two FMAs per step, instead
// of a full dot product, a reduction and an update per token. The products with S0 are 32 dot
// products per row with no dependence between them; the 16 x 16 tables k_i.k_j and q_i.k_j depend
// on the tokens only and are computed once per (chunk, q/k head) by a small kernel in front
// (every state row of the two v heads that share the q/k head reads them).
//
// A row is held by 16 lanes (8 state values each); lane i of the group is also token i of the
// chunk: a halving butterfly leaves S0.k_i and S0.q_i in lane i, lane i carries row i of the
// triangular system, and step j of the substitution broadcasts delta_j from lane j.
#pragma once

constexpr int C_TOK = 16;                 // tokens per chunk
constexpr int C_GSTRIDE = 2 * C_TOK * C_TOK;   // floats per (slot, q/k head): k.k table then q.k table
constexpr int C_GRAM_Z = 32;              // chunk lanes per sequence in the table kernel's grid

// Table slot of chunk c of sequence `seq` that starts at token t0: unique over all sequences
// without a scan of cu_seqlens (every sequence start costs at most one extra partial chunk).
__device__ __forceinline__ int64_t gdn_chunk_slot(int64_t t0, int seq, int c) { return t0 / C_TOK + seq + c; }

// tables[slot][hq][0][i][j] = k_i . k_j, tables[slot][hq][1][i][j] = q_i . k_j (tokens past the end
// of the sequence count as zero vectors). Grid (sequence, q/k head, C_GRAM_Z), 256 threads = (i, j).
__global__ void __launch_bounds__(256) gdn_gram_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                       const int64_t* __restrict__ cu_seqlens, float* __restrict__ tables) {
  __shared__ float s_k[C_TOK][P_D + 1], s_q[C_TOK][P_D + 1];
  const int seq = blockIdx.x, hq = blockIdx.y, tid = threadIdx.x;
  const int64_t t0 = cu_seqlens[seq], t1 = cu_seqlens[seq + 1];
  const int chunks = (int)((t1 - t0 + C_TOK - 1) / C_TOK);
  const int i = tid >> 4, j = tid & 15;
  for (int c = blockIdx.z; c < chunks; c += gridDim.z) {
    // 16 tokens x 128 values x {k, q}: thread tid loads 8 k and 8 q values of token tid / 16
    {
      const int tok = tid >> 4, part = tid & 15;
      const int64_t t = t0 + (int64_t)c * C_TOK + tok;
      uint4 kw = make_uint4(0u, 0u, 0u, 0u), qw = kw;
      if (t < t1) {
        kw = __ldg(reinterpret_cast<const uint4*>(k + (t * P_HQ + hq) * P_D + part * 8));
        qw = __ldg(reinterpret_cast<const uint4*>(q + (t * P_HQ + hq) * P_D + part * 8));
      }
      const uint32_t ka[4] = {kw.x, kw.y, kw.z, kw.w}, qa[4] = {qw.x, qw.y, qw.z, qw.w};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        s_k[tok][part * 8 + 2 * u] = ako::bf16_lo(ka[u]);
        s_k[tok][part * 8 + 2 * u + 1] = ako::bf16_hi(ka[u]);
        s_q[tok][part * 8 + 2 * u] = ako::bf16_lo(qa[u]);
        s_q[tok][part * 8 + 2 * u + 1] = ako::bf16_hi(qa[u]);
      }
    }
    __syncthreads();
    float kk = 0.f, qk = 0.f;
#pragma unroll 8
    for (int e = 0; e < P_D; ++e) {
      const float kj = s_k[j][e];
      kk = fmaf(s_k[i][e], kj, kk);
      qk = fmaf(s_q[i][e], kj, qk);
    }
    float* dst = tables + (gdn_chunk_slot(t0, seq, c) * P_HQ + hq) * C_GSTRIDE;
    dst[tid] = kk;
    dst[C_TOK * C_TOK + tid] = qk;
    __syncthreads();
  }
}

constexpr int C_ROWS = 8;                 // state rows per CTA: 4 warps x 2 groups of 16 lanes
constexpr int C_TPAD = 20;                // padded row length of the tables in shared memory

// LEAN: a scheduling fence every four tokens of the product loop keeps four tokens' loads in flight
// instead of sixteen: 124 registers instead of 243, three CTAs per SM instead of one. One sequence
// (128 CTAs) is faster without it, two sequences with it.
template <bool LEAN>
__global__ void __launch_bounds__(P_THREADS) gdn_prefill_chunk_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
    const float* __restrict__ state, const float* __restrict__ A_log, const __nv_bfloat16* __restrict__ a,
    const float* __restrict__ dt_bias, const __nv_bfloat16* __restrict__ b, const int64_t* __restrict__ cu_seqlens,
    float scale, __nv_bfloat16* __restrict__ out, float* __restrict__ new_state, const float* __restrict__ tables) {
  __shared__ __align__(16) float s_kq[2][C_TOK][2][P_D];          // [buffer][token][k | q][128]
  __shared__ __align__(16) float s_tab[2][2][C_TOK][C_TPAD];      // [buffer][k.k | q.k][i][j]
  __shared__ float s_lg[2][C_TOK], s_beta[2][C_TOK];              // log2 of the decay, beta
  __shared__ float s_v[2][C_TOK][C_ROWS];
  __shared__ __align__(16) __nv_bfloat16 s_out[2][C_TOK][C_ROWS];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool producer = warp == P_CONSUMERS / 32;
  const int rg = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
  const int hq = h / (P_HV / P_HQ);
  const int64_t t0 = cu_seqlens[seq], t1 = cu_seqlens[seq + 1];
  const int len = (int)(t1 - t0);
  const int i = lane & 15;                             // lane of the row's group = token of the chunk
  const int row_local = warp * 2 + (lane >> 4);
  const int row = rg * C_ROWS + row_local;
  // the lane holds state elements 64 p + 4 i + c (p = 0, 1; c = 0..3)
  float* ns = new_state + (((int64_t)seq * P_HV + h) * P_D + row) * P_D + 4 * i;
  float S[8];
  if (len <= 0) {   // the definition leaves the new state of an empty sequence at zero
    if (!producer) {
      *reinterpret_cast<float4*>(ns) = make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4*>(ns + 64) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    return;
  }
  if (producer) {
#pragma unroll
    for (int e = 0; e < 8; ++e) S[e] = 0.f;
  } else if (state != nullptr) {
    const float* sp = state + (((int64_t)seq * P_HV + h) * P_D + row) * P_D + 4 * i;
    const float4 x = __ldcs(reinterpret_cast<const float4*>(sp)), y = __ldcs(reinterpret_cast<const float4*>(sp + 64));
    S[0] = x.x; S[1] = x.y; S[2] = x.z; S[3] = x.w; S[4] = y.x; S[5] = y.y; S[6] = y.z; S[7] = y.w;
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) S[e] = 0.f;
  }
  const float neg_A = -expf(A_log[h]);
  const float dtb = dt_bias[h];

  // The producer warp stages chunk c + 1 (and the chunk's two tables, 2 KB) and stores the outputs
  // of chunk c - 1 while the four compute warps work on chunk c: one barrier per chunk.
  auto stage = [&](int c, int buf) {
    gdn_stage_chunk<C_ROWS, true>(lane, c, t0, t1, hq, h, rg, q, k, v, a, b, neg_A, dtb, s_kq[buf], s_lg[buf], s_beta[buf],
                                  s_v[buf]);
    const uint4* tp = reinterpret_cast<const uint4*>(tables + (gdn_chunk_slot(t0, seq, c) * P_HQ + hq) * C_GSTRIDE);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int f = lane + 32 * u;                      // float4 number f of the 128 that make both tables
      const uint4 x = __ldg(tp + f);
      *reinterpret_cast<uint4*>(&s_tab[buf][f >> 6][(f & 63) >> 2][(f & 3) * 4]) = x;
    }
  };
  const int chunks = (len + C_TOK - 1) / C_TOK;
  if (producer) stage(0, 0);
  __syncthreads();
  const bool b3 = (i & 8) != 0, b2 = (i & 4) != 0, b1 = (i & 2) != 0, b0 = (i & 1) != 0;
  for (int c = 0; c < chunks; ++c) {
    const int buf = c & 1;
    if (producer) {
      if (c > 0) gdn_store_chunk<C_ROWS>(lane, c - 1, t0, len, h, rg, s_out[buf ^ 1], out);
      if (c + 1 < chunks) stage(c + 1, buf ^ 1);
      __syncthreads();
      continue;
    }

    // 1. this lane's part of S0.k_j and S0.q_j for the 16 tokens: 32 independent short dot products
    float pa[C_TOK], pc[C_TOK];
#pragma unroll
    for (int j = 0; j < C_TOK; ++j) {
      const float4 k0 = *reinterpret_cast<const float4*>(&s_kq[buf][j][0][4 * i]);
      const float4 k1 = *reinterpret_cast<const float4*>(&s_kq[buf][j][0][64 + 4 * i]);
      const float4 q0 = *reinterpret_cast<const float4*>(&s_kq[buf][j][1][4 * i]);
      const float4 q1 = *reinterpret_cast<const float4*>(&s_kq[buf][j][1][64 + 4 * i]);
      pa[j] = fmaf(S[0], k0.x, fmaf(S[1], k0.y, fmaf(S[2], k0.z, S[3] * k0.w))) +
              fmaf(S[4], k1.x, fmaf(S[5], k1.y, fmaf(S[6], k1.z, S[7] * k1.w)));
      pc[j] = fmaf(S[0], q0.x, fmaf(S[1], q0.y, fmaf(S[2], q0.z, S[3] * q0.w))) +
              fmaf(S[4], q1.x, fmaf(S[5], q1.y, fmaf(S[6], q1.z, S[7] * q1.w)));
      if (LEAN && (j & 3) == 3) asm volatile("" ::: "memory");
    }
    // 2. halving butterfly over the row's 16 lanes: lane i ends with the complete sums of token i
    float ai, ci;
    {
      float x8[8], x4[4], x2[2];
#pragma unroll
      for (int t = 0; t < 8; ++t) x8[t] = (b3 ? pa[8 + t] : pa[t]) + __shfl_xor_sync(0xffffffffu, b3 ? pa[t] : pa[8 + t], 8);
#pragma unroll
      for (int t = 0; t < 4; ++t) x4[t] = (b2 ? x8[4 + t] : x8[t]) + __shfl_xor_sync(0xffffffffu, b2 ? x8[t] : x8[4 + t], 4);
#pragma unroll
      for (int t = 0; t < 2; ++t) x2[t] = (b1 ? x4[2 + t] : x4[t]) + __shfl_xor_sync(0xffffffffu, b1 ? x4[t] : x4[2 + t], 2);
      ai = (b0 ? x2[1] : x2[0]) + __shfl_xor_sync(0xffffffffu, b0 ? x2[0] : x2[1], 1);
#pragma unroll
      for (int t = 0; t < 8; ++t) x8[t] = (b3 ? pc[8 + t] : pc[t]) + __shfl_xor_sync(0xffffffffu, b3 ? pc[t] : pc[8 + t], 8);
#pragma unroll
      for (int t = 0; t < 4; ++t) x4[t] = (b2 ? x8[4 + t] : x8[t]) + __shfl_xor_sync(0xffffffffu, b2 ? x8[t] : x8[4 + t], 4);
#pragma unroll
      for (int t = 0; t < 2; ++t) x2[t] = (b1 ? x4[2 + t] : x4[t]) + __shfl_xor_sync(0xffffffffu, b1 ? x4[t] : x4[2 + t], 2);
      ci = (b0 ? x2[1] : x2[0]) + __shfl_xor_sync(0xffffffffu, b0 ? x2[0] : x2[1], 1);
    }
    // 3. row i of the triangular system and of the output sum
    float lc[C_TOK];            // Lc_j for every token of the chunk
    float Lci = 0.f;
    {
      float run = 0.f;
#pragma unroll
      for (int j = 0; j < C_TOK; ++j) {
        run += s_lg[buf][j];
        lc[j] = run;
        if (j == i) Lci = run;
      }
    }
    const float beta_i = s_beta[buf][i];
    float ca[C_TOK], co[C_TOK];  // ca[j] = beta_i R_ij (k_i.k_j) for j < i; co[j] = R_ij (q_i.k_j) for j <= i
#pragma unroll
    for (int j4 = 0; j4 < C_TOK; j4 += 4) {
      const float4 g4 = *reinterpret_cast<const float4*>(&s_tab[buf][0][i][j4]);
      const float4 m4 = *reinterpret_cast<const float4*>(&s_tab[buf][1][i][j4]);
      const float gg[4] = {g4.x, g4.y, g4.z, g4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = j4 + u;
        const float rij = exp2f(fminf(Lci - lc[j], 0.f));
        ca[j] = (j < i) ? beta_i * rij * gg[u] : 0.f;
        co[j] = (j <= i) ? rij * mm[u] : 0.f;
      }
    }
    const float gam_i = exp2f(Lci);
    float rhs = beta_i * (s_v[buf][i][row_local] - gam_i * ai);
    float o = gam_i * ci;
    // 4. forward substitution: delta_j is final in lane j when step j starts
    float d[C_TOK];
#pragma unroll
    for (int j = 0; j < C_TOK; ++j) {
      const float dj = __shfl_sync(0xffffffffu, rhs, j, 16);
      d[j] = dj;
      rhs = fmaf(-ca[j], dj, rhs);
      o = fmaf(co[j], dj, o);
    }
    s_out[buf][i][row_local] = __float2bfloat16_rn(scale * o);
    // 5. the state at the end of the chunk
    {
      const float lend = lc[C_TOK - 1];
      const float gC = exp2f(lend);
#pragma unroll
      for (int e = 0; e < 8; ++e) S[e] *= gC;
#pragma unroll
      for (int j = 0; j < C_TOK; ++j) {
        const float w = exp2f(lend - lc[j]) * d[j];
        const float4 k0 = *reinterpret_cast<const float4*>(&s_kq[buf][j][0][4 * i]);
        const float4 k1 = *reinterpret_cast<const float4*>(&s_kq[buf][j][0][64 + 4 * i]);
        S[0] = fmaf(w, k0.x, S[0]); S[1] = fmaf(w, k0.y, S[1]); S[2] = fmaf(w, k0.z, S[2]); S[3] = fmaf(w, k0.w, S[3]);
        S[4] = fmaf(w, k1.x, S[4]); S[5] = fmaf(w, k1.y, S[5]); S[6] = fmaf(w, k1.z, S[6]); S[7] = fmaf(w, k1.w, S[7]);
      }
    }
    __syncthreads();                       // chunk c done, chunk c + 1 staged
  }
  if (producer) {
    gdn_store_chunk<C_ROWS>(lane, chunks - 1, t0, len, h, rg, s_out[(chunks - 1) & 1], out);
    return;
  }
  __stcs(reinterpret_cast<float4*>(ns), make_float4(S[0], S[1], S[2], S[3]));
  __stcs(reinterpret_cast<float4*>(ns + 64), make_float4(S[4], S[5], S[6], S[7]));
}
