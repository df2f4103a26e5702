// Paged MLA decode and DSA sparse attention on the 5th-generation tensor cores (tcgen05 + TMEM),
// included by mla_attention.cu inside its anonymous namespace (it uses Params, RowDesc and
// describe_row defined there).
//
// Keys are walked in tiles of 128 tokens. Tokens are the M dimension of both products, so the 16
// heads need no padding:
//   S^T [128 tokens x 16 heads]  = K [128 x 576] . Q^T          36 MMAs  M128 N16 K16 (kind::f16)
//   O^T [512 dims  x 16 heads]  += V^T [512 x 128 tokens] . P^T  32 MMAs  M128 N16 K16, 4 M blocks
// V is the ckv part of the very rows staged for K: a tile is kept in shared memory as nine blocks of
// [128 tokens x 64 features] (128-byte rows, 128-byte swizzle). As the A operand of S^T a block is
// K-major; two neighbouring blocks read "MN-major" are the A operand V^T of one 128-feature block
// of O^T. Nothing is staged twice and nothing is transposed by hand.
//
// Work split: the tiles of all query rows form one flat sequence; a persistent CTA per SM takes an
// equal contiguous share of it (+-1 tile whatever the mix of row lengths) and cuts its share at row
// boundaries into segments. A segment yields one partial (m, l, O) for its row, stored in slot
// row + CTA index (both only grow along the sequence, so the sum is unique and at most
// rows + CTAs - 1); a merge kernel combines the one to three partials a row typically has. The
// pipeline runs on across segments: barriers, TMEM and the rings are set up once per CTA, the next
// row's Q is staged into a second buffer while the current row is still being read.
//
// The gather: page size 1 means every token is a random 1152-byte row. Four producer warps copy
// rows with 16-byte cp.async straight to their swizzled place, 256 contiguous bytes of a row per
// half-warp (the piece size at which random gathers measured fastest on B200: 6.6 TB/s against
// 5.5 TB/s for 1 KB pieces and 4.6 TB/s for 128-byte pieces; 1 KB bulk copies: 5.4 TB/s). A tile
// is 144 KB, so the ring is kept per block pair (32 KB = one M block of O^T) rather than per tile:
// five pair slots and one kpe slot; a pair is released by the commit of the PV MMAs that read it,
// and the next tile's first blocks are in flight while this tile's softmax and PV run.
//
// Roles (16 warps = 4 warpgroups of 128 registers per thread, re-balanced with setmaxnreg):
//   warps 0-7   compute: warp = (TMEM lane quarter q, head half hh). As softmax, thread = token:
//               its 8 heads of the S^T row out of TMEM, per-head maximum over the 128 tokens by a
//               9-shuffle butterfly plus an exchange in shared memory, exp2, P^T as bf16 into a
//               K-major [16 heads x 128 tokens] B operand, per-thread partial row sums (reduced once
//               per segment). As fold, thread = output feature of M blocks 2hh, 2hh+1: PV of a tile
//               is a fresh accumulator, folded into registers as O * 2^(m_old - m_new) + PV, so
//               TMEM contents are never rescaled;
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
constexpr int NPAIR = 5;
constexpr int QCH = H * 128;                  // one 64-feature chunk of Q: 16 heads x 128 B
constexpr int Q_BYTES = 9 * QCH;
constexpr int P_BYTES = 2 * QCH;              // P^T: two chunks of 64 tokens
constexpr int OFF_KPE = NPAIR * PAIR;
constexpr int OFF_Q = OFF_KPE + BLK;          // two Q buffers (segment parity)
constexpr int OFF_P = OFF_Q + 2 * Q_BYTES;
constexpr int OFF_PREF = OFF_P + P_BYTES;     // decode: exclusive prefix of tiles per row
constexpr int MAX_ROWS = 1535;                // rows the prefix table holds (decode)
constexpr int SMEM = OFF_PREF + (MAX_ROWS + 1) * 4 + 1024;  // + slack for 1024-byte alignment
static_assert(SMEM <= 232448 - 2048, "shared memory per CTA (2 KB kept for the static part)");
constexpr int THREADS = 16 * 32;
constexpr int COMPUTE_WARPS = 8;
constexpr int PRODUCERS = 128;
constexpr int REGS_COMPUTE = 152, REGS_PRODUCER = 104, REGS_ISSUER = 104;  // 2 x 152 + 104 + 104 = 4 x 128
constexpr int TMEM_COLS = 128;                // S^T at column 0 (16), PV at column 32 (4 x 16)
constexpr uint32_t IDESC_S = ako::tc::idesc_bf16_f32(TOK, H);
constexpr uint32_t IDESC_PV = ako::tc::idesc_bf16_f32(128, H) | ako::tc::kIdescAMnMajor;

enum : int { kErrSoftmaxS = 31, kErrSoftmaxX = 32, kErrSoftmaxP = 33, kErrFold = 34, kErrFoldFin = 35,
             kErrProdPair = 36, kErrProdKpe = 37, kErrProdQ = 38, kErrMmaS = 39, kErrMmaPair = 40,
             kErrMmaKpe = 41, kErrMmaP = 42, kErrMmaPv = 43, kErrMmaQ = 44 };

// Reduction (max or sum) over the 32 lanes of 8 values each: after three halving exchanges a lane
// holds one value, after two more the result over the warp. 9 shuffles instead of 40. The index
// a lane ends up with is 4*bit4 + 2*bit3 + bit2 of its lane id.
template <bool SUM>
__device__ __forceinline__ float warp_reduce8(const float (&v)[8], int lane) {
  auto op = [](float a, float b) { return SUM ? a + b : fmaxf(a, b); };
  float a4[4], a2[2], a1;
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float send = b4 ? v[j] : v[4 + j];
    const float keep = b4 ? v[4 + j] : v[j];
    a4[j] = op(keep, __shfl_xor_sync(0xffffffffu, send, 16));
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float send = b3 ? a4[j] : a4[2 + j];
    const float keep = b3 ? a4[2 + j] : a4[j];
    a2[j] = op(keep, __shfl_xor_sync(0xffffffffu, send, 8));
  }
  {
    const float send = b2 ? a2[0] : a2[1];
    const float keep = b2 ? a2[1] : a2[0];
    a1 = op(keep, __shfl_xor_sync(0xffffffffu, send, 4));
  }
  a1 = op(a1, __shfl_xor_sync(0xffffffffu, a1, 2));
  return op(a1, __shfl_xor_sync(0xffffffffu, a1, 1));
}
__device__ __forceinline__ int reduce8_index(int lane) {
  return ((lane & 16) ? 4 : 0) + ((lane & 8) ? 2 : 0) + ((lane & 4) ? 1 : 0);
}

// 32 lanes x 8 consecutive fp32 columns of TMEM.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait_regs8(float (&v)[8]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile("tcgen05.wait::ld.sync.aligned;\n"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])
               :
               : "memory");
}

// Walks the segments (row, first tile, tile count) of one CTA's share of the flat tile sequence.
template <int MODE>
struct SegWalker {
  const Params& p;
  const int* pref;     // decode: prefix table in shared memory; sparse: unused
  int rows, tiles_per_row;
  int row, t0, nt;     // current segment
  int left;            // tiles of the share not yet handed out (current segment included)
  RowDesc rd;

  __device__ __forceinline__ int row_tiles(int r) const {
    return MODE == kSparse ? tiles_per_row : pref[r + 1] - pref[r];
  }
  // positions on the first segment; false when the share is empty
  __device__ __forceinline__ bool start(int g_begin, int g_end) {
    left = g_end - g_begin;
    if (left <= 0) return false;
    if (MODE == kSparse) {
      row = g_begin / tiles_per_row;
      t0 = g_begin - row * tiles_per_row;
    } else {
      int lo = 0, hi = rows;  // largest r with pref[r] <= g_begin
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (pref[mid] <= g_begin) lo = mid; else hi = mid;
      }
      row = lo;
      t0 = g_begin - pref[lo];
    }
    nt = min(row_tiles(row) - t0, left);
    rd = describe_row<MODE>(p, row);
    return true;
  }
  __device__ __forceinline__ bool next() {
    left -= nt;
    if (left <= 0) return false;
    do { ++row; } while (row_tiles(row) == 0);
    t0 = 0;
    nt = min(row_tiles(row), left);
    rd = describe_row<MODE>(p, row);
    return true;
  }
};

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1) mla_gather_tc_kernel(Params p, int rows, int* pref_out) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t b_pair_full[NPAIR], b_pair_empty[NPAIR];
  __shared__ __align__(8) uint64_t b_kpe_full, b_kpe_empty, b_q_full[2], b_q_empty[2];
  __shared__ __align__(8) uint64_t b_s_full, b_s_empty, b_p_full, b_p_empty, b_pv_full, b_pv_empty, b_x, b_fin[2];
  __shared__ uint32_t s_tmem;
  __shared__ int s_err;
  __shared__ __align__(16) float s_xm[4][H];       // tile maxima per lane quarter
  __shared__ __align__(16) float s_xs[4][H];       // row sums per lane quarter (segment end)
  __shared__ __align__(16) float s_alpha[2][H];    // 2^(m_old - m_new) of a tile, by tile parity
  __shared__ __align__(16) float s_ml[2][2][H];    // final (m, l) of a segment, by segment parity

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t base = (ako::smem_u32(smem_raw) + 1023u) & ~1023u;
  int* s_pref = reinterpret_cast<int*>(smem_raw + (base - ako::smem_u32(smem_raw)) + OFF_PREF);

  ako::pdl_trigger();
  // ---- the flat tile sequence and this CTA's share -----------------------------------------------
  const int tpr = (MODE == kSparse) ? (p.topk + TOK - 1) / TOK : 0;
  int total_tiles;
  if (MODE == kSparse) {
    total_tiles = rows * tpr;
  } else {
    for (int r = tid; r < rows; r += THREADS) {
      const int len = max(0, p.kv_indptr[r + 1] - p.kv_indptr[r]) * p.page_size;
      s_pref[r + 1] = (len + TOK - 1) / TOK;
    }
    if (tid == 0) s_pref[0] = 0;
    __syncthreads();
    if (warp == 0) {  // inclusive scan in chunks of 32
      int carry = 0;
      for (int r0 = 1; r0 <= rows; r0 += 32) {
        const int r = r0 + lane;
        int v = (r <= rows) ? s_pref[r] : 0;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const int y = __shfl_up_sync(0xffffffffu, v, off);
          if (lane >= off) v += y;
        }
        if (r <= rows) s_pref[r] = v + carry;
        carry += __shfl_sync(0xffffffffu, v, 31);
      }
    }
    __syncthreads();
    total_tiles = s_pref[rows];
    if (blockIdx.x == 0 && pref_out)
      for (int r = tid; r <= rows; r += THREADS) pref_out[r] = s_pref[r];
  }
  const int per = (total_tiles + (int)gridDim.x - 1) / (int)gridDim.x;
  const int g_begin = min(total_tiles, (int)blockIdx.x * per);
  const int g_end = min(total_tiles, g_begin + per);
  if (g_begin >= g_end) return;  // nothing for this CTA (uniform)

  if (tid == 0) {
    for (int s = 0; s < NPAIR; ++s) {
      ako::tc::mbar_init(ako::smem_u32(&b_pair_full[s]), PRODUCERS);
      ako::tc::mbar_init(ako::smem_u32(&b_pair_empty[s]), 1);
    }
    ako::tc::mbar_init(ako::smem_u32(&b_kpe_full), PRODUCERS);
    ako::tc::mbar_init(ako::smem_u32(&b_kpe_empty), 1);
    for (int s = 0; s < 2; ++s) {
      ako::tc::mbar_init(ako::smem_u32(&b_q_full[s]), PRODUCERS);
      ako::tc::mbar_init(ako::smem_u32(&b_q_empty[s]), 1);
      ako::tc::mbar_init(ako::smem_u32(&b_fin[s]), 2);
    }
    ako::tc::mbar_init(ako::smem_u32(&b_s_full), 1);
    ako::tc::mbar_init(ako::smem_u32(&b_s_empty), COMPUTE_WARPS);
    ako::tc::mbar_init(ako::smem_u32(&b_p_full), COMPUTE_WARPS);
    ako::tc::mbar_init(ako::smem_u32(&b_p_empty), 1);
    ako::tc::mbar_init(ako::smem_u32(&b_pv_full), 1);
    ako::tc::mbar_init(ako::smem_u32(&b_pv_empty), COMPUTE_WARPS);
    ako::tc::mbar_init(ako::smem_u32(&b_x), COMPUTE_WARPS);
    ako::tc::mbar_init_fence();
    s_err = 0;
  }
  if (warp == 12) ako::tc::tmem_alloc(ako::smem_u32(&s_tmem), TMEM_COLS);
  ako::tc::fence_before_thread_sync();
  __syncthreads();
  ako::tc::fence_after_thread_sync();
  const uint32_t tmem = s_tmem;
  int* err = &s_err;

  SegWalker<MODE> w{p, s_pref, rows, tpr};
  w.start(g_begin, g_end);

  if (warp < COMPUTE_WARPS) {
    // ============================ compute: softmax, then fold ==================================
    ako::tc::reg_inc<REGS_COMPUTE>();
    const int q = warp & 3, hh = warp >> 2;
    const int tok = 32 * q + lane;          // softmax: token of the tile; fold: feature of a block
    const int isel = reduce8_index(lane);
    const uint32_t p_dst = base + OFF_P + (tok >> 6) * QCH + (8 * hh) * 128 + (tok & 7) * 2;
    const int c16 = (tok & 63) >> 3;
    const uint32_t t_lane = (uint32_t)(32 * q) << 16;
    bool ok = true;
    uint32_t xph = 0;
    int gt = 0, seg = 0;
    do {
      float m_run[8], l_part[8], O[2][H];
#pragma unroll
      for (int h = 0; h < 8; ++h) { m_run[h] = -INFINITY; l_part[h] = 0.f; }
#pragma unroll
      for (int mb = 0; mb < 2; ++mb)
#pragma unroll
        for (int h = 0; h < H; ++h) O[mb][h] = 0.f;
      const int tok_end = w.rd.count;
      auto entry_at = [&](int tile) -> int32_t {
        const int pos = min(tile * TOK + tok, tok_end - 1);
        return __ldg(w.rd.idx + (p.page_size == 1 ? pos : pos / p.page_size));
      };
      int32_t ent_next = (MODE == kSparse) ? entry_at(w.t0) : 0;
      for (int it = 0; it < w.nt; ++it, ++gt) {
        const int tile = w.t0 + it;
        const int32_t ent = ent_next;
        if (MODE == kSparse && it + 1 < w.nt) ent_next = entry_at(tile + 1);
        const bool valid = (tile * TOK + tok < tok_end) && (MODE != kSparse || ent >= 0);
        // ---- softmax of this tile ----
        if (!ako::tc::mbar_wait_warp(ako::smem_u32(&b_s_full), (uint32_t)(gt & 1), err, kErrSoftmaxS)) { ok = false; break; }
        ako::tc::fence_after_thread_sync();
        float x[8];
        tmem_ld8(tmem + t_lane + 8 * hh, x);
        tmem_ld_wait_regs8(x);
        ako::tc::fence_before_thread_sync();
        __syncwarp();
        if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&b_s_empty));
#pragma unroll
        for (int h = 0; h < 8; ++h) x[h] = valid ? x[h] * p.scale_log2 : -INFINITY;
        const float wmax = warp_reduce8<false>(x, lane);
        if ((lane & 3) == 0) s_xm[q][8 * hh + isel] = wmax;
        __syncwarp();
        if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&b_x));
        if (!ako::tc::mbar_wait_warp(ako::smem_u32(&b_x), xph, err, kErrSoftmaxX)) { ok = false; break; }
        xph ^= 1u;
        float pr[8];
#pragma unroll
        for (int h4 = 0; h4 < 8; h4 += 4) {
          const float4 m0 = *reinterpret_cast<const float4*>(&s_xm[0][8 * hh + h4]);
          const float4 m1 = *reinterpret_cast<const float4*>(&s_xm[1][8 * hh + h4]);
          const float4 m2 = *reinterpret_cast<const float4*>(&s_xm[2][8 * hh + h4]);
          const float4 m3 = *reinterpret_cast<const float4*>(&s_xm[3][8 * hh + h4]);
          const float mt[4] = {fmaxf(fmaxf(m0.x, m1.x), fmaxf(m2.x, m3.x)), fmaxf(fmaxf(m0.y, m1.y), fmaxf(m2.y, m3.y)),
                               fmaxf(fmaxf(m0.z, m1.z), fmaxf(m2.z, m3.z)), fmaxf(fmaxf(m0.w, m1.w), fmaxf(m2.w, m3.w))};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int h = h4 + k;
            const float m_new = fmaxf(m_run[h], mt[k]);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            // the maximum is the same in every thread of the CTA, so this branch is uniform
            const float alpha = (m_new == m_run[h] && m_new != -INFINITY) ? 1.f : ako::fast_exp2(m_run[h] - m_use);
            pr[h] = ako::fast_exp2(x[h] - m_use);
            l_part[h] = fmaf(l_part[h], alpha, pr[h]);
            m_run[h] = m_new;
            if (q == 0 && lane == h) s_alpha[gt & 1][8 * hh + h] = alpha;
          }
        }
        // P^T may be overwritten once the PV MMAs of the previous tile have read it
        if (gt > 0 && !ako::tc::mbar_wait_warp(ako::smem_u32(&b_p_empty), (uint32_t)((gt - 1) & 1), err, kErrSoftmaxP)) { ok = false; break; }
#pragma unroll
        for (int h = 0; h < 8; ++h) {
          const __nv_bfloat16 pb = __float2bfloat16_rn(pr[h]);
          asm volatile("st.shared.b16 [%0], %1;\n" ::"r"(p_dst + h * 128 + ((c16 ^ h) << 4)),  // (8hh + h) & 7 == h
                       "h"(*reinterpret_cast<const unsigned short*>(&pb))
                       : "memory");
        }
        ako::tc::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&b_p_full));
        const bool last = (it + 1 == w.nt);
        if (last) {
          // segment end: row sums (per-thread partials -> warp -> CTA); m is the same in every thread
          const float wsum = warp_reduce8<true>(l_part, lane);
          if ((lane & 3) == 0) s_xs[q][8 * hh + isel] = wsum;
          __syncwarp();
          if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&b_x));
          if (!ako::tc::mbar_wait_warp(ako::smem_u32(&b_x), xph, err, kErrSoftmaxX)) { ok = false; break; }
          xph ^= 1u;
          if (q == 0) {
#pragma unroll
            for (int h = 0; h < 8; ++h) {
              if (lane == h) {
                s_ml[seg & 1][0][8 * hh + h] = m_run[h];
                s_ml[seg & 1][1][8 * hh + h] = s_xs[0][8 * hh + h] + s_xs[1][8 * hh + h] + s_xs[2][8 * hh + h] + s_xs[3][8 * hh + h];
              }
            }
            __syncwarp();
            if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&b_fin[seg & 1]));
          }
        }
        // ---- fold of this tile: M blocks 2hh and 2hh+1, all 16 heads ----
        if (!ako::tc::mbar_wait_warp(ako::smem_u32(&b_pv_full), (uint32_t)(gt & 1), err, kErrFold)) { ok = false; break; }
        ako::tc::fence_after_thread_sync();
        float v[2][H];
        ako::tc::tmem_ld16(tmem + t_lane + 32 + 16 * (2 * hh), v[0]);
        ako::tc::tmem_ld16(tmem + t_lane + 32 + 16 * (2 * hh + 1), v[1]);
        ako::tc::tmem_ld_wait_regs16(v[0]);
        ako::tc::tmem_ld_wait_regs16(v[1]);
        ako::tc::fence_before_thread_sync();
#pragma unroll
        for (int h4 = 0; h4 < H; h4 += 4) {
          const float4 a4 = *reinterpret_cast<const float4*>(&s_alpha[gt & 1][h4]);
          const float a[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            O[0][h4 + k] = fmaf(O[0][h4 + k], a[k], v[0][h4 + k]);
            O[1][h4 + k] = fmaf(O[1][h4 + k], a[k], v[1][h4 + k]);
          }
        }
        if (last) {
          // the segment's partial: slot = row + CTA index
          if (!ako::tc::mbar_wait_warp(ako::smem_u32(&b_fin[seg & 1]), (uint32_t)((seg >> 1) & 1), err, kErrFoldFin)) { ok = false; break; }
          const int64_t slot = (int64_t)w.row + blockIdx.x;
#pragma unroll
          for (int h = 0; h < H; ++h) {
            float* pa = p.part_acc + (slot * H + h) * DC + 128 * (2 * hh) + tok;
            pa[0] = O[0][h];
            pa[128] = O[1][h];
          }
          if (warp == 0 && lane < H) {
            float* ml = p.part_ml + (slot * H + lane) * 2;
            ml[0] = s_ml[seg & 1][0][lane];
            ml[1] = s_ml[seg & 1][1][lane];
          }
        }
        // the PV buffer (and, at a segment end, the (m, l) words) may be reused from here on
        __syncwarp();
        if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&b_pv_empty));
      }
      ++seg;
    } while (ok && w.next());
  } else if (warp < 12) {
    // ==================================== producers ============================================
    ako::tc::reg_dec<REGS_PRODUCER>();
    const int pw = warp - 8;
    const int t128 = tid - 256;
    const int half = lane >> 4, l16 = lane & 15;  // half-warp = one row's 256-byte piece
    const int fb = l16 >> 3, j = l16 & 7;
    const int kq = lane >> 3, kj = lane & 7;      // kpe: 8 lanes per row, 4 rows per instruction
    bool ok = true;
    int gt = 0, seg = 0;
    do {
      // Q of this row as the B operand of S^T: nine K-major chunks [16 heads x 64 features]
      if (!ako::tc::mbar_wait_warp(ako::smem_u32(&b_q_empty[seg & 1]), (uint32_t)(((seg >> 1) & 1) ^ 1), err, kErrProdQ)) { ok = false; break; }
      const uint32_t qdst = base + OFF_Q + (seg & 1) * Q_BYTES;
      for (int i = t128; i < H * 72; i += PRODUCERS) {
        const int h = i / 72, c = i % 72;         // 16-byte piece c of head h's 1152-byte row
        const int ch = c >> 3, jj = c & 7;
        const void* src = (ch < 8) ? (const void*)(p.q_nope + ((int64_t)w.row * H + h) * DC + c * 8)
                                   : (const void*)(p.q_pe + ((int64_t)w.row * H + h) * DP + jj * 8);
        ako::cp_async16(qdst + ch * QCH + h * 128 + ((jj ^ (h & 7)) << 4), src);
      }
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(ako::smem_u32(&b_q_full[seg & 1])) : "memory");
      const int tok_end = w.rd.count;
      auto entry_at = [&](int tile) -> int32_t {
        const int pos = min(tile * TOK + 32 * pw + lane, tok_end - 1);
        return __ldg(w.rd.idx + (p.page_size == 1 ? pos : pos / p.page_size));
      };
      int32_t ent_next = entry_at(w.t0);
      for (int it = 0; it < w.nt && ok; ++it, ++gt) {
        const int tile = w.t0 + it;
        const int32_t ent = ent_next;
        if (it + 1 < w.nt) ent_next = entry_at(tile + 1);
        // cache row (or -1) of this lane's token; rows of other lanes come by shuffle
        const int mypos = tile * TOK + 32 * pw + lane;
        int64_t myrow = -1;
        if (mypos < tok_end && (MODE != kSparse || ent >= 0))
          myrow = (p.page_size == 1) ? (int64_t)ent : (int64_t)ent * p.page_size + mypos % p.page_size;
        const int rlo = (int)(myrow & 0xffffffffLL), rhi = (int)(myrow >> 32);
        // kpe first: its slot is free as soon as the previous tile's S MMAs are done
        if (!ako::tc::mbar_wait_warp(ako::smem_u32(&b_kpe_empty), (uint32_t)((gt & 1) ^ 1), err, kErrProdKpe)) { ok = false; break; }
        const uint32_t kdst = base + OFF_KPE;
#pragma unroll 4
        for (int i = 0; i < 8; ++i) {
          const int src_lane = 4 * i + kq;
          const int64_t r = ((int64_t)__shfl_sync(0xffffffffu, rhi, src_lane) << 32) |
                            (uint32_t)__shfl_sync(0xffffffffu, rlo, src_lane);
          const int t = 32 * pw + src_lane;
          const bool valid = r >= 0;
          ako::cp_async16(kdst + t * 128 + ((kj ^ (t & 7)) << 4), p.kpe + (valid ? r : 0) * KPE_ROW + kj * 16, valid);
        }
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(ako::smem_u32(&b_kpe_full)) : "memory");
        for (int pr = 0; pr < 4; ++pr) {
          const int g = gt * 4 + pr, slot = g % NPAIR;
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
      }
      ++seg;
    } while (ok && w.next());
    ako::cp_async_wait<0>();  // nothing of this thread is in flight when the CTA leaves
  } else {
    ako::tc::reg_dec<REGS_ISSUER>();
    if (warp == 12 && lane == 0) {
      // =================================== MMA issuer ============================================
      const uint32_t p_lo = ako::tc::smem_desc_lo(base + OFF_P);
      const uint32_t k_lo = ako::tc::smem_desc_lo(base + OFF_KPE);
      const uint32_t d_s = tmem, d_pv = tmem + 32;
      bool ok = true;
      int gt = 0, seg = 0;
      do {
        if (!ako::tc::mbar_wait(ako::smem_u32(&b_q_full[seg & 1]), (uint32_t)((seg >> 1) & 1), err, kErrMmaQ)) { ok = false; break; }
        ako::tc::fence_proxy_async_smem();
        const uint32_t q_lo = ako::tc::smem_desc_lo(base + OFF_Q + (seg & 1) * Q_BYTES);
        for (int it = 0; it < w.nt && ok; ++it, ++gt) {
          // ---- S^T = K Q^T: the kpe chunk first (it was fetched ahead), then the four pairs ----
          if (gt > 0 && !ako::tc::mbar_wait(ako::smem_u32(&b_s_empty), (uint32_t)((gt - 1) & 1), err, kErrMmaS)) { ok = false; break; }
          if (!ako::tc::mbar_wait(ako::smem_u32(&b_kpe_full), (uint32_t)(gt & 1), err, kErrMmaKpe)) { ok = false; break; }
          ako::tc::fence_proxy_async_smem();  // cp.async wrote the block through the generic proxy
          ako::tc::fence_after_thread_sync();
#pragma unroll
          for (int k = 0; k < 4; ++k)
            ako::tc::mma_bf16_lohi(d_s, k_lo + 2 * k, q_lo + (uint32_t)(8 * (QCH >> 4)) + 2 * k, IDESC_S, k ? 1u : 0u);
          ako::tc::mma_commit(ako::smem_u32(&b_kpe_empty));
          for (int pr = 0; pr < 4 && ok; ++pr) {
            const int g = gt * 4 + pr, slot = g % NPAIR;
            if (!ako::tc::mbar_wait(ako::smem_u32(&b_pair_full[slot]), (uint32_t)((g / NPAIR) & 1), err, kErrMmaPair)) { ok = false; break; }
            ako::tc::fence_proxy_async_smem();
            ako::tc::fence_after_thread_sync();
#pragma unroll
            for (int fbk = 0; fbk < 8; ++fbk) {
              const int f2 = fbk >> 2, k = fbk & 3;
              const uint32_t a_lo = ako::tc::smem_desc_lo(base + slot * PAIR + f2 * BLK) + 2 * k;
              const uint32_t b_lo = q_lo + (uint32_t)((2 * pr + f2) * (QCH >> 4)) + 2 * k;
              ako::tc::mma_bf16_lohi(d_s, a_lo, b_lo, IDESC_S, 1u);
            }
          }
          if (!ok) break;
          ako::tc::mma_commit(ako::smem_u32(&b_s_full));
          if (it + 1 == w.nt) ako::tc::mma_commit(ako::smem_u32(&b_q_empty[seg & 1]));  // last S of this row
          // ---- O^T partial = V^T P^T ----
          if (!ako::tc::mbar_wait(ako::smem_u32(&b_p_full), (uint32_t)(gt & 1), err, kErrMmaP)) { ok = false; break; }
          if (gt > 0 && !ako::tc::mbar_wait(ako::smem_u32(&b_pv_empty), (uint32_t)((gt - 1) & 1), err, kErrMmaPv)) { ok = false; break; }
          ako::tc::fence_after_thread_sync();
          for (int mb = 0; mb < 4; ++mb) {
            const int g = gt * 4 + mb, slot = g % NPAIR;
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
        ++seg;
      } while (ok && w.next());
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

// Merge of the segment partials: one block per (row, head), 128 threads x 4 columns. The partials of
// row r are the slots r + c for the CTAs c whose share of the flat tile sequence touches the row.
template <int MODE>
__global__ void __launch_bounds__(DC / 4) mla_gather_tc_merge_kernel(
    const float* __restrict__ part_acc, const float* __restrict__ part_ml, const int* __restrict__ pref,
    int rows, int tiles_per_row, int ctas, __nv_bfloat16* __restrict__ o, float* __restrict__ lse) {
  ako::pdl_wait();
  const int r = blockIdx.x / H, h = blockIdx.x % H;
  int t0, t1, total;
  if (MODE == kSparse) {
    t0 = r * tiles_per_row; t1 = t0 + tiles_per_row; total = rows * tiles_per_row;
  } else {
    t0 = pref[r]; t1 = pref[r + 1]; total = pref[rows];
  }
  const int per = (total + ctas - 1) / ctas;
  float M = -INFINITY, L = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (t1 > t0) {
    const int c0 = t0 / per, c1 = (t1 - 1) / per;
    for (int c = c0; c <= c1; ++c) M = fmaxf(M, part_ml[((int64_t)(r + c) * H + h) * 2]);
    if (M > -INFINITY) {
      for (int c = c0; c <= c1; ++c) {
        const float* ml = part_ml + ((int64_t)(r + c) * H + h) * 2;
        if (ml[0] == -INFINITY) continue;
        const float wgt = exp2f(ml[0] - M);
        L = fmaf(ml[1], wgt, L);
        const float4 p4 = *reinterpret_cast<const float4*>(part_acc + ((int64_t)(r + c) * H + h) * DC + threadIdx.x * 4);
        acc.x = fmaf(p4.x, wgt, acc.x);
        acc.y = fmaf(p4.y, wgt, acc.y);
        acc.z = fmaf(p4.z, wgt, acc.z);
        acc.w = fmaf(p4.w, wgt, acc.w);
      }
    }
  }
  const float inv = (L > 0.f) ? 1.f / L : 0.f;
  uint2 pk;
  pk.x = ako::pack_bf16x2(acc.x * inv, acc.y * inv);
  pk.y = ako::pack_bf16x2(acc.z * inv, acc.w * inv);
  *reinterpret_cast<uint2*>(o + (int64_t)blockIdx.x * DC + threadIdx.x * 4) = pk;
  if (threadIdx.x == 0) lse[blockIdx.x] = (L > 0.f) ? M + log2f(L) : -INFINITY;
}

}  // namespace tcg
