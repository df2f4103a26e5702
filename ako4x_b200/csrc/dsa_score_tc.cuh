// DSA index scores on the 5th-generation tensor cores (tcgen05 + TMEM) fed by TMA; included by
// dsa_indexer.cu inside its anonymous namespace.
//
// score[r, t] = (sum_h w[r,h] * relu(q[r,h,:] . k[t,:])) * kscale[t]. Tokens are the M dimension of
// the MMA (128 tokens = two 64-token cache pages), the 64 heads of up to FOUR query rows the N
// dimension (N = 256), K = 128 e4m3 values (four tcgen05.mma K32 steps). With tokens on the TMEM
// lanes, relu, the head weights and the head reduction are plain per-thread arithmetic on the
// accumulator columns: no shuffles.
//
// A unit of work is (group of 4 consecutive query rows, pair of logical pages). When the four rows
// map that page pair to the same physical pages (consecutive tokens of one sequence, the prefill
// case) the key tile is loaded once and one N = 256 MMA sequence serves all four rows; otherwise
// the unit runs as four N = 64 sequences, one key tile each, into the four column blocks of the
// same accumulator. A persistent CTA takes a contiguous range of units, so the 32 KB query tile of
// a row group stays in shared memory while the CTA sweeps pages.
//   warp 9      one thread: TMA loads of query tiles (2 buffers) and key tiles (6-stage ring; a
//               page is a [64 x 128 B] box of a 3-D tensor map over the 8448-byte pages);
//   warp 8      one thread: MMAs into one of two 256-column TMEM accumulators; commits free the
//               key stage, the query buffer and publish the accumulator;
//   warps 0-7   epilogue: thread (w, l) owns token 32*(w%4)+l and the two rows (w/4)*2, +1.
// Every mbarrier wait is bounded; a timeout sets the status word and all roles unwind.

constexpr int TS_ROWS = 4;                      // query rows per unit
constexpr int TS_N = TS_ROWS * NH;              // 256 accumulator columns
constexpr int TS_A_BYTES = 2 * PS * HD;         // 16 KB: two pages of e4m3 keys
constexpr int TS_Q_BYTES = TS_N * HD;           // 32 KB: four rows of e4m3 queries
constexpr int TS_A_STAGES = 6;
constexpr int TS_SMEM = 2 * TS_Q_BYTES + TS_A_STAGES * TS_A_BYTES + 1024;
constexpr int TS_EPI_THREADS = 256;
constexpr int TS_THREADS = TS_EPI_THREADS + 64;

__device__ int g_dsa_status = 0;  // 0 = ok; set when a bounded wait gave up

struct ScoreParams {
  const float* weights;
  const int32_t* seq_lens;
  const int32_t* block_table;
  const unsigned char* cache;
  float* scores;
  int rows, max_pages;
  int64_t num_cache_pages;
  int skip_short;
};

struct ScoreUnit {
  int row0;          // first query row of the group
  int pp;            // page pair: logical pages 2*pp, 2*pp+1
  bool any;          // some row of the group needs this page pair
  bool shared;       // all needed rows map it to the same physical pages
  int pa[TS_ROWS], pb[TS_ROWS];  // physical pages per row (clamped into range)
};

__device__ __forceinline__ bool row_needs(const ScoreParams& p, int r, int pp) {
  if (r >= p.rows) return false;
  const int sl = p.seq_lens[r];
  if (sl <= 0 || (p.skip_short && sl <= TOPK)) return false;
  return 2 * pp * PS < min(sl, p.max_pages * PS);
}

__device__ __forceinline__ int phys_page(const ScoreParams& p, int r, int lp) {
  r = min(r, p.rows - 1);
  lp = min(lp, p.max_pages - 1);
  const int64_t pg = p.block_table[(int64_t)r * p.max_pages + lp];
  return (pg < 0 || pg >= p.num_cache_pages) ? 0 : (int)pg;  // out-of-range id: stay in bounds
}

__device__ __forceinline__ ScoreUnit describe_unit(const ScoreParams& p, int unit, int pairs) {
  ScoreUnit u;
  u.row0 = (unit / pairs) * TS_ROWS;
  u.pp = unit % pairs;
  u.any = false;
  u.shared = true;
  int fa = -1, fb = -1;
#pragma unroll
  for (int i = 0; i < TS_ROWS; ++i) {
    const bool need = row_needs(p, u.row0 + i, u.pp);
    u.pa[i] = phys_page(p, u.row0 + i, 2 * u.pp);
    u.pb[i] = phys_page(p, u.row0 + i, 2 * u.pp + 1);
    if (need) {
      if (!u.any) { fa = u.pa[i]; fb = u.pb[i]; }
      else if (u.pa[i] != fa || u.pb[i] != fb) u.shared = false;
      u.any = true;
    }
  }
  if (u.shared && u.any) {
#pragma unroll
    for (int i = 0; i < TS_ROWS; ++i) { u.pa[i] = fa; u.pb[i] = fb; }
  }
  return u;
}

__global__ void __launch_bounds__(TS_THREADS, 1)
dsa_score_tc_kernel(ScoreParams p, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t s_a_full[TS_A_STAGES];
  __shared__ __align__(8) uint64_t s_a_empty[TS_A_STAGES];
  __shared__ __align__(8) uint64_t s_q_full[2];
  __shared__ __align__(8) uint64_t s_q_empty[2];
  __shared__ __align__(8) uint64_t s_acc_full[2];
  __shared__ __align__(8) uint64_t s_acc_empty[2];
  __shared__ uint32_t s_tmem_base;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t smem_base = (ako::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_base = smem_base;
  const uint32_t a_base = smem_base + 2 * TS_Q_BYTES;

  if (tid == 0) {
    for (int s = 0; s < TS_A_STAGES; ++s) {
      ako::tc::mbar_init(ako::smem_u32(&s_a_full[s]), 1);
      ako::tc::mbar_init(ako::smem_u32(&s_a_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ako::tc::mbar_init(ako::smem_u32(&s_q_full[b]), 1);
      ako::tc::mbar_init(ako::smem_u32(&s_q_empty[b]), 1);
      ako::tc::mbar_init(ako::smem_u32(&s_acc_full[b]), 1);
      ako::tc::mbar_init(ako::smem_u32(&s_acc_empty[b]), TS_EPI_THREADS / 32);
    }
    ako::tc::mbar_init_fence();
  }
  if (warp == 8) ako::tc::tmem_alloc(ako::smem_u32(&s_tmem_base), 512);
  ako::tc::fence_before_thread_sync();
  __syncthreads();
  ako::tc::fence_after_thread_sync();
  const uint32_t tmem_base = s_tmem_base;

  const int pairs = (p.max_pages + 1) / 2;
  const int groups = (p.rows + TS_ROWS - 1) / TS_ROWS;
  const int64_t total = (int64_t)groups * pairs;
  const int u_begin = (int)(total * blockIdx.x / gridDim.x);
  const int u_end = (int)(total * (blockIdx.x + 1) / gridDim.x);

  if (warp == 9) {
    // ================================ TMA producer =============================================
    if (lane == 0) {
      ako::tc::tma_prefetch_desc(&tm_q);
      ako::tc::tma_prefetch_desc(&tm_k);
      int ac = 0, qc = 0, cur_group = -1;
      bool ok = true;
      for (int unit = u_begin; ok && unit < u_end; ++unit) {
        const ScoreUnit u = describe_unit(p, unit, pairs);
        if (!u.any) continue;
        if (u.row0 != cur_group) {
          cur_group = u.row0;
          const int qb = qc & 1;
          if (!ako::tc::mbar_wait(ako::smem_u32(&s_q_empty[qb]), (uint32_t)(((qc >> 1) & 1) ^ 1), &g_dsa_status, 1)) { ok = false; break; }
          const uint32_t bar = ako::smem_u32(&s_q_full[qb]);
          ako::tc::mbar_arrive_expect_tx(bar, TS_Q_BYTES);
#pragma unroll
          for (int i = 0; i < TS_ROWS; ++i)
            ako::tc::tma_load_2d(q_base + qb * TS_Q_BYTES + i * NH * HD, &tm_q, 0, min(u.row0 + i, p.rows - 1) * NH, bar);
          ++qc;
        }
        const int subs = u.shared ? 1 : TS_ROWS;
        for (int s = 0; s < subs; ++s, ++ac) {
          const int stage = ac % TS_A_STAGES;
          if (!ako::tc::mbar_wait(ako::smem_u32(&s_a_empty[stage]), (uint32_t)(((ac / TS_A_STAGES) & 1) ^ 1), &g_dsa_status, 2)) { ok = false; break; }
          const uint32_t bar = ako::smem_u32(&s_a_full[stage]);
          const uint32_t dst = a_base + stage * TS_A_BYTES;
          ako::tc::mbar_arrive_expect_tx(bar, TS_A_BYTES);
          ako::tc::tma_load_3d(dst, &tm_k, 0, 0, u.pa[s], bar);
          ako::tc::tma_load_3d(dst + PS * HD, &tm_k, 0, 0, u.pb[s], bar);
        }
      }
    }
  } else if (warp == 8) {
    // ================================ MMA issuer ===============================================
    if (lane == 0) {
      constexpr uint32_t IDESC_SHARED = ako::tc::idesc_e4m3_f32(128, TS_N);
      constexpr uint32_t IDESC_ROW = ako::tc::idesc_e4m3_f32(128, NH);
      int ac = 0, qc = 0, uc = 0, cur_group = -1;
      bool ok = true;
      for (int unit = u_begin; ok && unit < u_end; ++unit) {
        const ScoreUnit u = describe_unit(p, unit, pairs);
        if (!u.any) continue;
        if (u.row0 != cur_group) {
          if (cur_group >= 0) ako::tc::mma_commit(ako::smem_u32(&s_q_empty[(qc - 1) & 1]));  // previous tile is done with
          cur_group = u.row0;
          if (!ako::tc::mbar_wait(ako::smem_u32(&s_q_full[qc & 1]), (uint32_t)((qc >> 1) & 1), &g_dsa_status, 3)) { ok = false; break; }
          ++qc;
        }
        const uint32_t qs = q_base + ((qc - 1) & 1) * TS_Q_BYTES;
        const int buf = uc & 1;
        if (!ako::tc::mbar_wait(ako::smem_u32(&s_acc_empty[buf]), (uint32_t)(((uc >> 1) & 1) ^ 1), &g_dsa_status, 4)) { ok = false; break; }
        const int subs = u.shared ? 1 : TS_ROWS;
        for (int s = 0; s < subs; ++s, ++ac) {
          const int stage = ac % TS_A_STAGES;
          if (!ako::tc::mbar_wait(ako::smem_u32(&s_a_full[stage]), (uint32_t)((ac / TS_A_STAGES) & 1), &g_dsa_status, 5)) { ok = false; break; }
          ako::tc::fence_after_thread_sync();
          const uint32_t sa = a_base + stage * TS_A_BYTES;
          const uint32_t sb = qs + (u.shared ? 0 : s * NH * HD);
          const uint32_t d = tmem_base + buf * TS_N + (u.shared ? 0 : s * NH);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            ako::tc::mma_f8(d, ako::tc::smem_desc_k_sw128(sa + ks * 32), ako::tc::smem_desc_k_sw128(sb + ks * 32),
                            u.shared ? IDESC_SHARED : IDESC_ROW, ks > 0 ? 1u : 0u);
          ako::tc::mma_commit(ako::smem_u32(&s_a_empty[stage]));
        }
        if (!ok) break;
        ako::tc::mma_commit(ako::smem_u32(&s_acc_full[buf]));
        ++uc;
      }
    }
  } else {
    // ================================ epilogue ====================================================
    const int q = warp & 3;             // TMEM lane quarter
    const int rh = warp >> 2;           // which two rows of the group
    const int t = 32 * q + lane;        // token inside the unit
    int uc = 0;
    bool ok = true;
    for (int unit = u_begin; ok && unit < u_end; ++unit) {
      const ScoreUnit u = describe_unit(p, unit, pairs);
      if (!u.any) continue;
      const int buf = uc & 1;
      if (!ako::tc::mbar_wait(ako::smem_u32(&s_acc_full[buf]), (uint32_t)((uc >> 1) & 1), &g_dsa_status, 6)) { ok = false; break; }
      ako::tc::fence_after_thread_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + buf * TS_N + rh * 2 * NH;
      float sum[2] = {0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {  // 32 columns each: row (c>>1) of this thread's pair, heads 32*(c&1)..
        float v[32];
        ako::tc::tmem_ld32(taddr + 32 * c, v);
        const int r = min(u.row0 + rh * 2 + (c >> 1), p.rows - 1);
        const float4* wp = reinterpret_cast<const float4*>(p.weights + (int64_t)r * NH + 32 * (c & 1));
        float4 w4[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) w4[j] = __ldg(wp + j);
        ako::tc::tmem_ld_wait();
        if (c == 3) {  // the accumulator is in registers: release it
          ako::tc::fence_before_thread_sync();
          __syncwarp();
          if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&s_acc_empty[buf]));
        }
        float s = sum[c >> 1];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s = fmaf(fmaxf(v[4 * j + 0], 0.f), w4[j].x, s);
          s = fmaf(fmaxf(v[4 * j + 1], 0.f), w4[j].y, s);
          s = fmaf(fmaxf(v[4 * j + 2], 0.f), w4[j].z, s);
          s = fmaf(fmaxf(v[4 * j + 3], 0.f), w4[j].w, s);
        }
        sum[c >> 1] = s;
      }
      const int tok = u.pp * 2 * PS + t;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int ri = rh * 2 + i;
        const int r = u.row0 + ri;
        if (!row_needs(p, r, u.pp)) continue;
        const int sl = p.seq_lens[r];
        if (tok >= p.max_pages * PS) continue;
        const int page = (t < PS) ? u.pa[ri] : u.pb[ri];
        const float ksc = __ldg(reinterpret_cast<const float*>(p.cache + (int64_t)page * PAGE_BYTES + PS * HD) + (t & (PS - 1)));
        p.scores[(int64_t)r * p.max_pages * PS + tok] = (tok < sl) ? sum[i] * ksc : -INFINITY;
      }
      ++uc;
    }
  }

  ako::tc::fence_before_thread_sync();
  __syncthreads();
  if (warp == 8) {
    ako::tc::fence_after_thread_sync();
    ako::tc::tmem_dealloc(tmem_base, 512);
  }
}
