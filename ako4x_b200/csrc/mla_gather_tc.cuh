// Paged MLA decode and DSA sparse attention on the 5th-generation tensor cores (tcgen05 + TMEM),
// included by mla_attention.cu inside its anonymous namespace (it uses Params, RowDesc and
// describe_row defined there).
//
// One CTA owns (query token, KV split) and walks its keys in tiles of 128 tokens. Tokens are the M
// dimension of both products, so the 16 heads need no padding:
//   S^T [128 tokens x 16 heads]  = K [128 x 576] . Q^T          36 MMAs  M128 N16 K16 (kind::f16)
//   O^T [512 dims  x 16 heads]  += V^T [512 x 128 tokens] . P^T  32 MMAs  M128 N16 K16, 4 M blocks
// V is the ckv part of the very rows staged for K: a tile is kept in shared memory as nine blocks of
// [128 tokens x 64 features] (128-byte rows, 128-byte swizzle). As the A operand of S^T a block is
// K-major; two neighbouring blocks read "MN-major" are the A operand V^T of one 128-feature block
// of O^T. Nothing is staged twice and nothing is transposed by hand.
//
// The gather: page size 1 means every token is a random 1152-byte row. Four producer warps copy
// rows with 16-byte cp.async straight to their swizzled place, 256 contiguous bytes of a row per
// half-warp (the piece size at which random gathers measured fastest on B200: 6.6 TB/s against
// 5.5 TB/s for 1 KB pieces and 4.6 TB/s for 128-byte pieces; 1 KB bulk copies: 5.4 TB/s). A tile
// is 144 KB, so the ring is kept per block pair (32 KB = one M block of O^T) rather than per tile:
// five pair slots and two kpe slots; a pair is released by the commit of the PV MMAs that read it,
// and the next tile's pairs are in flight while this tile's softmax and PV run.
//
// Roles (16 warps = 4 warpgroups of 128 registers per thread, re-balanced with setmaxnreg:
// softmax 160, fold 200, producers 80, issuer group 72; 160 + 200 + 80 + 72 = 4 x 128):
//   warps 0-3   softmax: thread = token (TMEM lane). S^T row out of TMEM, per-head maximum over the
//               128 tokens by a 16-shuffle butterfly plus a 4-entry exchange in shared memory,
//               exp2, P^T as bf16 into a K-major [16 heads x 128 tokens] B operand, per-thread
//               partial row sums (reduced once, at the end);
//   warps 4-7   fold: thread = output feature. PV of a tile is a fresh accumulator; it is folded
//               into registers as O * 2^(m_old - m_new) + PV, so TMEM contents are never rescaled;
//   warps 8-11  producers (above);
//   warp 12     lane 0 issues every MMA; the warp allocates and frees TMEM (warps 13-15 only
//               donate their registers).
// Every mbarrier wait is bounded (tcgen05.cuh); a wait that gives up sets the CTA's error word,
// every role unwinds to the common exit, and the device status word records the code.
#pragma once

namespace tcg {

constexpr int TOK = 128;                      // tokens per tile
constexpr int BLK = TOK * 128;                // one block: 128 tokens x 64 features (16 KB)
constexpr int PAIR = 2 * BLK;                 // two blocks = one 128-feature block of V^T
constexpr int NPAIR = 5, NKPE = 2;
constexpr int QCH = H * 128;                  // one 64-feature chunk of Q: 16 heads x 128 B
constexpr int Q_BYTES = 9 * QCH;
constexpr int P_BYTES = 2 * QCH;              // P^T: two chunks of 64 tokens
constexpr int OFF_KPE = NPAIR * PAIR;
constexpr int OFF_Q = OFF_KPE + NKPE * BLK;
constexpr int OFF_P = OFF_Q + Q_BYTES;
constexpr int SMEM = OFF_P + P_BYTES + 1024;  // + slack for 1024-byte alignment
constexpr int THREADS = 16 * 32;
constexpr int REGS_SOFTMAX = 160, REGS_FOLD = 200, REGS_PRODUCER = 80, REGS_ISSUER = 72;
constexpr int PRODUCERS = 128;
constexpr int TMEM_COLS = 128;                // S^T at column 0 (16), PV at column 32 (4 x 16)
constexpr uint32_t IDESC_S = ako::tc::idesc_bf16_f32(TOK, H);
constexpr uint32_t IDESC_PV = ako::tc::idesc_bf16_f32(128, H) | ako::tc::kIdescAMnMajor;

enum : int { kErrSoftmaxS = 31, kErrSoftmaxX = 32, kErrSoftmaxP = 33, kErrFold = 34, kErrFoldFin = 35,
             kErrProdPair = 36, kErrProdKpe = 37, kErrMmaS = 38, kErrMmaPair = 39, kErrMmaKpe = 40,
             kErrMmaP = 41, kErrMmaPv = 42 };

// Max over the 32 lanes of 16 values each: after four halving exchanges every lane holds one
// head, after the fifth the maximum over the warp. 16 shuffles instead of 80. The head a lane ends
// up with is ((lane >> 1) & 15) read as bits 4..1 of the lane id, most significant first.
template <bool SUM>
__device__ __forceinline__ float warp_reduce16(const float (&v)[16], int lane) {
  auto op = [](float a, float b) { return SUM ? a + b : fmaxf(a, b); };
  float a8[8], a4[4], a2[2], a1;
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4, b1 = lane & 2;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float send = b4 ? v[j] : v[8 + j];
    const float keep = b4 ? v[8 + j] : v[j];
    a8[j] = op(keep, __shfl_xor_sync(0xffffffffu, send, 16));
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float send = b3 ? a8[j] : a8[4 + j];
    const float keep = b3 ? a8[4 + j] : a8[j];
    a4[j] = op(keep, __shfl_xor_sync(0xffffffffu, send, 8));
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float send = b2 ? a4[j] : a4[2 + j];
    const float keep = b2 ? a4[2 + j] : a4[j];
    a2[j] = op(keep, __shfl_xor_sync(0xffffffffu, send, 4));
  }
  {
    const float send = b1 ? a2[0] : a2[1];
    const float keep = b1 ? a2[1] : a2[0];
    a1 = op(keep, __shfl_xor_sync(0xffffffffu, send, 2));
  }
  return op(a1, __shfl_xor_sync(0xffffffffu, a1, 1));
}
// the head index that warp_reduce16 leaves in a lane
__device__ __forceinline__ int reduce16_head(int lane) {
  return ((lane & 16) ? 8 : 0) + ((lane & 8) ? 4 : 0) + ((lane & 4) ? 2 : 0) + ((lane & 2) ? 1 : 0);
}

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1) mla_gather_tc_kernel(Params p) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t b_pair_full[NPAIR], b_pair_empty[NPAIR];
  __shared__ __align__(8) uint64_t b_kpe_full[NKPE], b_kpe_empty[NKPE];
  __shared__ __align__(8) uint64_t b_s_full, b_s_empty, b_p_full, b_p_empty, b_pv_full, b_pv_empty, b_x, b_fin;
  __shared__ uint32_t s_tmem;
  __shared__ int s_err;
  __shared__ __align__(16) float s_xm[4][H];       // per softmax warp: tile maxima (then: row sums)
  __shared__ __align__(16) float s_alpha[2][H];    // 2^(m_old - m_new) of a tile, by tile parity
  __shared__ __align__(16) float s_ml[2][H];       // final m and l of the split

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x % p.num_splits;
  const int64_t row = blockIdx.x / p.num_splits;

  ako::pdl_trigger();
  const RowDesc rd = describe_row<MODE>(p, row);
  int chunk = (int)ako::round_up(ako::cdiv(rd.count, p.num_splits), TOK);
  if (chunk < TOK) chunk = TOK;
  const int tok_begin = min(rd.count, split * chunk);
  const int tok_end = min(rd.count, tok_begin + chunk);
  const int ntiles = (tok_end - tok_begin + TOK - 1) / TOK;

  if (ntiles == 0) {  // nothing in this split: an empty partial (or an empty row)
    if (p.num_splits > 1) {
      if (tid < H) {
        float* ml = p.part_ml + ((row * H + tid) * p.num_splits + split) * 2;
        ml[0] = -INFINITY;
        ml[1] = 0.f;
      }
    } else {
      for (int i = tid; i < H * DC / 8; i += THREADS)
        reinterpret_cast<uint4*>(p.o + row * H * DC)[i] = make_uint4(0, 0, 0, 0);
      if (tid < H) p.lse[row * H + tid] = -INFINITY;
    }
    return;
  }

  const uint32_t base = (ako::smem_u32(smem_raw) + 1023u) & ~1023u;
  if (tid == 0) {
    for (int s = 0; s < NPAIR; ++s) {
      ako::tc::mbar_init(ako::smem_u32(&b_pair_full[s]), PRODUCERS);
      ako::tc::mbar_init(ako::smem_u32(&b_pair_empty[s]), 1);
    }
    for (int s = 0; s < NKPE; ++s) {
      ako::tc::mbar_init(ako::smem_u32(&b_kpe_full[s]), PRODUCERS);
      ako::tc::mbar_init(ako::smem_u32(&b_kpe_empty[s]), 1);
    }
    ako::tc::mbar_init(ako::smem_u32(&b_s_full), 1);
    ako::tc::mbar_init(ako::smem_u32(&b_s_empty), 4);
    ako::tc::mbar_init(ako::smem_u32(&b_p_full), 4);
    ako::tc::mbar_init(ako::smem_u32(&b_p_empty), 1);
    ako::tc::mbar_init(ako::smem_u32(&b_pv_full), 1);
    ako::tc::mbar_init(ako::smem_u32(&b_pv_empty), 4);
    ako::tc::mbar_init(ako::smem_u32(&b_x), 4);
    ako::tc::mbar_init(ako::smem_u32(&b_fin), 1);
    ako::tc::mbar_init_fence();
    s_err = 0;
  }
  if (warp == 12) ako::tc::tmem_alloc(ako::smem_u32(&s_tmem), TMEM_COLS);
  if (warp >= 8 && warp < 12) {
    // Q as the B operand of S^T: nine K-major chunks [16 heads x 64 features], 128-byte swizzle
    const int t = tid - 256;
    for (int i = t; i < H * 72; i += PRODUCERS) {
      const int h = i / 72, c16 = i % 72;           // 16-byte piece c16 of head h's 1152-byte row
      const int ch = c16 >> 3, j = c16 & 7;
      const void* src = (ch < 8) ? (const void*)(p.q_nope + (row * H + h) * DC + c16 * 8)
                                 : (const void*)(p.q_pe + (row * H + h) * DP + j * 8);
      ako::cp_async16(base + OFF_Q + ch * QCH + h * 128 + ((j ^ (h & 7)) << 4), src);
    }
    ako::cp_async_commit();
    ako::cp_async_wait<0>();
    ako::tc::fence_proxy_async_smem();
  }
  ako::tc::fence_before_thread_sync();
  __syncthreads();
  ako::tc::fence_after_thread_sync();
  const uint32_t tmem = s_tmem;
  int* err = &s_err;

  // raw index entry of token `k` of tile `tile` (clamped to the chunk; callers test validity)
  auto entry_at = [&](int tile, int k) -> int32_t {
    const int pos = min(tok_begin + tile * TOK + k, tok_end - 1);
    return __ldg(rd.idx + (p.page_size == 1 ? pos : pos / p.page_size));
  };

  if (warp < 4) {
    // ===================================== softmax =============================================
    ako::tc::reg_inc<REGS_SOFTMAX>();
    const int tok = 32 * warp + lane;
    const int hsel = reduce16_head(lane);
    float m_run[H], l_part[H];
#pragma unroll
    for (int h = 0; h < H; ++h) { m_run[h] = -INFINITY; l_part[h] = 0.f; }
    int32_t ent_next = entry_at(0, tok);
    const uint32_t p_dst = base + OFF_P + (tok >> 6) * QCH + (tok & 7) * 2;
    const int c16 = (tok & 63) >> 3;
    bool ok = true;
    uint32_t xph = 0;
    for (int it = 0; it < ntiles; ++it) {
      const int32_t ent = ent_next;
      if (it + 1 < ntiles) ent_next = entry_at(it + 1, tok);
      const bool valid = (tok_begin + it * TOK + tok < tok_end) && (MODE != kSparse || ent >= 0);
      if (!ako::tc::mbar_wait_warp(ako::smem_u32(&b_s_full), (uint32_t)(it & 1), err, kErrSoftmaxS)) { ok = false; break; }
      ako::tc::fence_after_thread_sync();
      float x[H];
      ako::tc::tmem_ld16(tmem + ((uint32_t)(32 * warp) << 16), x);
      ako::tc::tmem_ld_wait_regs16(x);
      ako::tc::fence_before_thread_sync();
      __syncwarp();
      if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&b_s_empty));
#pragma unroll
      for (int h = 0; h < H; ++h) x[h] = valid ? x[h] * p.scale_log2 : -INFINITY;
      const float wmax = warp_reduce16<false>(x, lane);
      if ((lane & 1) == 0) s_xm[warp][hsel] = wmax;
      __syncwarp();
      if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&b_x));
      if (!ako::tc::mbar_wait_warp(ako::smem_u32(&b_x), xph, err, kErrSoftmaxX)) { ok = false; break; }
      xph ^= 1u;
      float pr[H];
#pragma unroll
      for (int h4 = 0; h4 < H; h4 += 4) {
        const float4 m0 = *reinterpret_cast<const float4*>(&s_xm[0][h4]);
        const float4 m1 = *reinterpret_cast<const float4*>(&s_xm[1][h4]);
        const float4 m2 = *reinterpret_cast<const float4*>(&s_xm[2][h4]);
        const float4 m3 = *reinterpret_cast<const float4*>(&s_xm[3][h4]);
        const float mt[4] = {fmaxf(fmaxf(m0.x, m1.x), fmaxf(m2.x, m3.x)), fmaxf(fmaxf(m0.y, m1.y), fmaxf(m2.y, m3.y)),
                             fmaxf(fmaxf(m0.z, m1.z), fmaxf(m2.z, m3.z)), fmaxf(fmaxf(m0.w, m1.w), fmaxf(m2.w, m3.w))};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int h = h4 + k;
          const float m_new = fmaxf(m_run[h], mt[k]);
          const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
          const float alpha = ako::fast_exp2(m_run[h] - m_use);
          pr[h] = ako::fast_exp2(x[h] - m_use);
          l_part[h] = fmaf(l_part[h], alpha, pr[h]);
          m_run[h] = m_new;
          if (warp == 0 && lane == h) s_alpha[it & 1][h] = alpha;
        }
      }
      // P^T may be overwritten once the PV MMAs of the previous tile have read it
      if (it > 0 && !ako::tc::mbar_wait_warp(ako::smem_u32(&b_p_empty), (uint32_t)((it - 1) & 1), err, kErrSoftmaxP)) { ok = false; break; }
#pragma unroll
      for (int h = 0; h < H; ++h) {
        const __nv_bfloat16 pb = __float2bfloat16_rn(pr[h]);
        asm volatile("st.shared.b16 [%0], %1;\n" ::"r"(p_dst + h * 128 + ((c16 ^ (h & 7)) << 4)),
                     "h"(*reinterpret_cast<const unsigned short*>(&pb))
                     : "memory");
      }
      ako::tc::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&b_p_full));
    }
    if (ok) {
      // row sums: per-thread partials -> warp -> CTA; m is the same in every thread
      const float wsum = warp_reduce16<true>(l_part, lane);
      // the last tile's maxima have been read by every warp before its p_full arrival, and every
      // warp passes the exchange barrier below only after all four wrote their sums
      if (ntiles > 0 && !ako::tc::mbar_wait_warp(ako::smem_u32(&b_p_empty), (uint32_t)((ntiles - 1) & 1), err, kErrSoftmaxP)) ok = false;
      if (ok) {
        if ((lane & 1) == 0) s_xm[warp][hsel] = wsum;
        __syncwarp();
        if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&b_x));
        if (ako::tc::mbar_wait_warp(ako::smem_u32(&b_x), xph, err, kErrSoftmaxX)) {
          if (warp == 0) {
#pragma unroll
            for (int h = 0; h < H; ++h) {
              if (lane == h) {
                s_ml[0][h] = m_run[h];
                s_ml[1][h] = s_xm[0][h] + s_xm[1][h] + s_xm[2][h] + s_xm[3][h];
              }
            }
            __syncwarp();
            if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&b_fin));
          }
        }
      }
    }
  } else if (warp < 8) {
    // ====================================== fold ===============================================
    ako::tc::reg_inc<REGS_FOLD>();
    const int q = warp - 4;
    float O[4][H];
#pragma unroll
    for (int mb = 0; mb < 4; ++mb)
#pragma unroll
      for (int h = 0; h < H; ++h) O[mb][h] = 0.f;
    bool ok = true;
    for (int it = 0; it < ntiles; ++it) {
      if (!ako::tc::mbar_wait_warp(ako::smem_u32(&b_pv_full), (uint32_t)(it & 1), err, kErrFold)) { ok = false; break; }
      ako::tc::fence_after_thread_sync();
      float v[4][H];
      const uint32_t ta = tmem + ((uint32_t)(32 * q) << 16) + 32;
#pragma unroll
      for (int mb = 0; mb < 4; ++mb) ako::tc::tmem_ld16(ta + 16 * mb, v[mb]);
#pragma unroll
      for (int mb = 0; mb < 4; ++mb) ako::tc::tmem_ld_wait_regs16(v[mb]);
      ako::tc::fence_before_thread_sync();
      __syncwarp();
      if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&b_pv_empty));
#pragma unroll
      for (int h4 = 0; h4 < H; h4 += 4) {
        const float4 a4 = *reinterpret_cast<const float4*>(&s_alpha[it & 1][h4]);
        const float a[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
        for (int k = 0; k < 4; ++k)
#pragma unroll
          for (int mb = 0; mb < 4; ++mb) O[mb][h4 + k] = fmaf(O[mb][h4 + k], a[k], v[mb][h4 + k]);
      }
    }
    if (ok && ako::tc::mbar_wait_warp(ako::smem_u32(&b_fin), 0u, err, kErrFoldFin)) {
      const int f = 32 * q + lane;  // feature inside a 128-feature block
      if (p.num_splits == 1) {
#pragma unroll
        for (int h = 0; h < H; ++h) {
          const float l = s_ml[1][h];
          const float inv = (l > 0.f) ? 1.f / l : 0.f;
          __nv_bfloat16* op = p.o + (row * H + h) * DC + f;
#pragma unroll
          for (int mb = 0; mb < 4; ++mb) op[128 * mb] = __float2bfloat16_rn(O[mb][h] * inv);
        }
        if (q == 0 && lane < H) {
          const float l = s_ml[1][lane];
          p.lse[row * H + lane] = (l > 0.f) ? s_ml[0][lane] + log2f(l) : -INFINITY;
        }
      } else {
#pragma unroll
        for (int h = 0; h < H; ++h) {
          float* pa = p.part_acc + ((row * H + h) * p.num_splits + split) * DC + f;
#pragma unroll
          for (int mb = 0; mb < 4; ++mb) pa[128 * mb] = O[mb][h];
        }
        if (q == 0 && lane < H) {
          float* ml = p.part_ml + ((row * H + lane) * p.num_splits + split) * 2;
          ml[0] = s_ml[0][lane];
          ml[1] = s_ml[1][lane];
        }
      }
    }
  } else if (warp < 12) {
    // ==================================== producers ============================================
    ako::tc::reg_dec<REGS_PRODUCER>();
    const int pw = warp - 8;
    const int half = lane >> 4, l16 = lane & 15;  // half-warp = one row's 256-byte piece
    const int fb = l16 >> 3, j = l16 & 7;
    const int kq = lane >> 3, kj = lane & 7;      // kpe: 8 lanes per row, 4 rows per instruction
    int32_t ent_next = entry_at(0, 32 * pw + lane);
    bool ok = true;
    for (int it = 0; it < ntiles && ok; ++it) {
      const int32_t ent = ent_next;
      if (it + 1 < ntiles) ent_next = entry_at(it + 1, 32 * pw + lane);
      // cache row (or -1) of this lane's token; rows of other lanes come by shuffle
      const int mypos = tok_begin + it * TOK + 32 * pw + lane;
      int64_t myrow = -1;
      if (mypos < tok_end && (MODE != kSparse || ent >= 0))
        myrow = (p.page_size == 1) ? (int64_t)ent : (int64_t)ent * p.page_size + mypos % p.page_size;
      const int rlo = (int)(myrow & 0xffffffffLL), rhi = (int)(myrow >> 32);
      for (int pr = 0; pr < 4; ++pr) {
        const int g = it * 4 + pr, slot = g % NPAIR;
        if (!ako::tc::mbar_wait_warp(ako::smem_u32(&b_pair_empty[slot]), (uint32_t)(((g / NPAIR) & 1) ^ 1), err, kErrProdPair)) { ok = false; break; }
        const uint32_t dst0 = base + slot * PAIR + fb * BLK;
#pragma unroll 4
        for (int i = 0; i < 16; ++i) {
          const int src_lane = 2 * i + half;
          const int64_t r = ((int64_t)__shfl_sync(0xffffffffu, rhi, src_lane) << 32) |
                            (uint32_t)__shfl_sync(0xffffffffu, rlo, src_lane);
          const int t = 32 * pw + src_lane;
          const bool valid = r >= 0;
          ako::cp_async16(dst0 + t * 128 + ((j ^ (t & 7)) << 4),
                          p.ckv + (valid ? r : 0) * CKV_ROW + pr * 256 + l16 * 16, valid);
        }
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(ako::smem_u32(&b_pair_full[slot]))
                     : "memory");
      }
      if (!ok) break;
      const int ks = it % NKPE;
      if (!ako::tc::mbar_wait_warp(ako::smem_u32(&b_kpe_empty[ks]), (uint32_t)(((it / NKPE) & 1) ^ 1), err, kErrProdKpe)) { ok = false; break; }
      const uint32_t kdst = base + OFF_KPE + ks * BLK;
#pragma unroll 4
      for (int i = 0; i < 8; ++i) {
        const int src_lane = 4 * i + kq;
        const int64_t r = ((int64_t)__shfl_sync(0xffffffffu, rhi, src_lane) << 32) |
                          (uint32_t)__shfl_sync(0xffffffffu, rlo, src_lane);
        const int t = 32 * pw + src_lane;
        const bool valid = r >= 0;
        ako::cp_async16(kdst + t * 128 + ((kj ^ (t & 7)) << 4), p.kpe + (valid ? r : 0) * KPE_ROW + kj * 16, valid);
      }
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(ako::smem_u32(&b_kpe_full[ks]))
                   : "memory");
    }
    ako::cp_async_wait<0>();  // nothing of this thread is in flight when the CTA leaves
  } else {
    ako::tc::reg_dec<REGS_ISSUER>();
    if (warp == 12 && lane == 0) {
    // =================================== MMA issuer ============================================
    const uint32_t q_lo = ako::tc::smem_desc_lo(base + OFF_Q);
    const uint32_t p_lo = ako::tc::smem_desc_lo(base + OFF_P);
    const uint32_t d_s = tmem, d_pv = tmem + 32;
    bool ok = true;
    for (int it = 0; it < ntiles && ok; ++it) {
      // ---- S^T = K Q^T ----
      if (it > 0 && !ako::tc::mbar_wait(ako::smem_u32(&b_s_empty), (uint32_t)((it - 1) & 1), err, kErrMmaS)) { ok = false; break; }
      for (int pr = 0; pr < 4 && ok; ++pr) {
        const int g = it * 4 + pr, slot = g % NPAIR;
        if (!ako::tc::mbar_wait(ako::smem_u32(&b_pair_full[slot]), (uint32_t)((g / NPAIR) & 1), err, kErrMmaPair)) { ok = false; break; }
        ako::tc::fence_proxy_async_smem();  // cp.async wrote the pair through the generic proxy
        ako::tc::fence_after_thread_sync();
#pragma unroll
        for (int fbk = 0; fbk < 8; ++fbk) {
          const int f2 = fbk >> 2, k = fbk & 3;
          const uint32_t a_lo = ako::tc::smem_desc_lo(base + slot * PAIR + f2 * BLK) + 2 * k;
          const uint32_t b_lo = q_lo + (uint32_t)((2 * pr + f2) * (QCH >> 4)) + 2 * k;
          ako::tc::mma_bf16_lohi(d_s, a_lo, b_lo, IDESC_S, (pr | fbk) ? 1u : 0u);
        }
      }
      if (!ok) break;
      const int ks = it % NKPE;
      if (!ako::tc::mbar_wait(ako::smem_u32(&b_kpe_full[ks]), (uint32_t)((it / NKPE) & 1), err, kErrMmaKpe)) { ok = false; break; }
      ako::tc::fence_proxy_async_smem();
      ako::tc::fence_after_thread_sync();
#pragma unroll
      for (int k = 0; k < 4; ++k)
        ako::tc::mma_bf16_lohi(d_s, ako::tc::smem_desc_lo(base + OFF_KPE + ks * BLK) + 2 * k,
                               q_lo + (uint32_t)(8 * (QCH >> 4)) + 2 * k, IDESC_S, 1u);
      ako::tc::mma_commit(ako::smem_u32(&b_kpe_empty[ks]));
      ako::tc::mma_commit(ako::smem_u32(&b_s_full));
      // ---- O^T partial = V^T P^T ----
      if (!ako::tc::mbar_wait(ako::smem_u32(&b_p_full), (uint32_t)(it & 1), err, kErrMmaP)) { ok = false; break; }
      if (it > 0 && !ako::tc::mbar_wait(ako::smem_u32(&b_pv_empty), (uint32_t)((it - 1) & 1), err, kErrMmaPv)) { ok = false; break; }
      ako::tc::fence_after_thread_sync();
      for (int mb = 0; mb < 4; ++mb) {
        const int g = it * 4 + mb, slot = g % NPAIR;
        const uint32_t a0 = ako::tc::smem_desc_lo_mn(base + slot * PAIR, BLK);
#pragma unroll
        for (int kt = 0; kt < 8; ++kt)  // 16 tokens per MMA: two 8-token groups of 1024 bytes
          ako::tc::mma_bf16_lohi(d_pv + 16 * mb, a0 + (uint32_t)(kt * (2048 >> 4)),
                                 p_lo + (uint32_t)((kt >> 2) * (QCH >> 4)) + 2 * (kt & 3), IDESC_PV, kt ? 1u : 0u);
        ako::tc::mma_commit(ako::smem_u32(&b_pair_empty[slot]));
      }
      ako::tc::mma_commit(ako::smem_u32(&b_pv_full));
      ako::tc::mma_commit(ako::smem_u32(&b_p_empty));
    }
    }
  }

  // ===================================== common exit ============================================
  ako::tc::fence_before_thread_sync();
  __syncthreads();
  if (tid == 0 && s_err != 0) atomicCAS(&g_mla_status, 0, s_err);
  if (warp == 12) {
    ako::tc::fence_after_thread_sync();
    ako::tc::tmem_dealloc(tmem, TMEM_COLS);
  }
}

}  // namespace tcg
