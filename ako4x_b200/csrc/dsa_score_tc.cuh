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
//   warp 9      producer: lanes 0-3 read the block table of the group's four rows; lane 0 issues
//               the TMA loads (query tile + head weights per group: 2 buffers; key tile: 6-stage
//               ring, a page is a [64 x 128 B] box of a 3-D tensor map over the 8448-byte pages)
//               and, per key tile, a slot of a 16-deep ring that carries the tile's 128 key scales
//               and the unit's descriptor, so that no other warp touches the block table;
//   warp 8      one thread: MMAs into one of two 256-column TMEM accumulators; commits free the
//               key stage, the query buffer and publish the accumulator;
//   warps 0-7   epilogue: thread (w, l) owns token 32*(w%4)+l and the two rows (w/4)*2, +1.
// Every reader of TMA-written shared memory waits on the mbarrier the copy completes on. Every
// wait is bounded; a timeout sets the status word and all roles unwind.

constexpr int TS_ROWS = 4;                      // query rows per unit
constexpr int TS_N = TS_ROWS * NH;              // 256 accumulator columns
constexpr int TS_A_BYTES = 2 * PS * HD;         // 16 KB: two pages of e4m3 keys
constexpr int TS_Q_BYTES = TS_N * HD;           // 32 KB: four rows of e4m3 queries
constexpr int TS_W_BYTES = TS_N * 4;            // 1 KB: their head weights
constexpr int TS_A_STAGES = 6;
constexpr int TS_SLOTS = 16;                    // descriptor + key-scale ring
constexpr int TS_SLOT_BYTES = 2 * PS * 4 + 64;  // 128 scales, then the descriptor
constexpr int TS_SMEM = 2 * TS_Q_BYTES + TS_A_STAGES * TS_A_BYTES + 2 * TS_W_BYTES + TS_SLOTS * TS_SLOT_BYTES + 1024;
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

// Unit descriptor, written by the producer into the unit's first ring slot.
struct ScoreDesc {
  int row0;           // first query row of the group
  int pp;             // page pair: logical pages 2*pp, 2*pp+1
  int flags;          // TS_F_*
  int sl[TS_ROWS];    // row's sequence length, or -1 when the row takes nothing from this unit
  int pad;
};
constexpr int TS_F_SHARED = 1, TS_F_NEWGROUP = 2, TS_F_END = 4;

__device__ __forceinline__ int phys_page(const ScoreParams& p, int r, int lp) {
  r = min(r, p.rows - 1);
  lp = min(lp, p.max_pages - 1);
  const int64_t pg = __ldg(p.block_table + (int64_t)r * p.max_pages + lp);
  return (pg < 0 || pg >= p.num_cache_pages) ? 0 : (int)pg;  // out-of-range id: stay in bounds
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
  __shared__ __align__(8) uint64_t s_slot_full[TS_SLOTS];
  __shared__ __align__(8) uint64_t s_slot_empty[TS_SLOTS];
  __shared__ uint32_t s_tmem_base;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned char* smem_al = smem_raw + ((1024u - (ako::smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t q_base = ako::smem_u32(smem_al);
  const uint32_t a_base = q_base + 2 * TS_Q_BYTES;
  unsigned char* w_ptr = smem_al + 2 * TS_Q_BYTES + TS_A_STAGES * TS_A_BYTES;
  unsigned char* slot_ptr = w_ptr + 2 * TS_W_BYTES;
  const uint32_t w_base = ako::smem_u32(w_ptr);
  const uint32_t slot_base = ako::smem_u32(slot_ptr);

  if (tid == 0) {
    for (int s = 0; s < TS_A_STAGES; ++s) {
      ako::tc::mbar_init(ako::smem_u32(&s_a_full[s]), 1);
      ako::tc::mbar_init(ako::smem_u32(&s_a_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ako::tc::mbar_init(ako::smem_u32(&s_q_full[b]), 1);
      ako::tc::mbar_init(ako::smem_u32(&s_q_empty[b]), 1 + TS_EPI_THREADS / 32);
      ako::tc::mbar_init(ako::smem_u32(&s_acc_full[b]), 1);
      ako::tc::mbar_init(ako::smem_u32(&s_acc_empty[b]), TS_EPI_THREADS / 32);
    }
    for (int s = 0; s < TS_SLOTS; ++s) {
      ako::tc::mbar_init(ako::smem_u32(&s_slot_full[s]), 1);
      ako::tc::mbar_init(ako::smem_u32(&s_slot_empty[s]), TS_EPI_THREADS / 32);
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
    // ================================ producer (whole warp) ====================================
    if (lane == 0) {
      ako::tc::tma_prefetch_desc(&tm_q);
      ako::tc::tma_prefetch_desc(&tm_k);
    }
    int ac = 0, qc = 0, loaded_group = -1, issued_group = -1;
    int my_sl = -1, my_lim = 0;  // lanes 0-3: this lane's row of the group
    int ok = 1;
    for (int unit = u_begin; ok && unit <= u_end; ++unit) {
      const bool end = unit == u_end;
      const int row0 = end ? 0 : (unit / pairs) * TS_ROWS;
      const int pp = end ? 0 : unit % pairs;
      int pa = 0, pb = 0;
      bool shared = true;
      if (!end) {
        if (row0 != loaded_group) {
          loaded_group = row0;
          my_sl = -1;
          my_lim = 0;
          if (lane < TS_ROWS && row0 + lane < p.rows) {
            const int sl = __ldg(p.seq_lens + row0 + lane);
            if (sl > 0 && !(p.skip_short && sl <= TOPK)) {
              my_sl = sl;
              my_lim = min(sl, p.max_pages * PS);
            }
          }
        }
        const bool need = lane < TS_ROWS && 2 * pp * PS < my_lim;
        if (lane < TS_ROWS) {
          pa = phys_page(p, row0 + lane, 2 * pp);
          pb = phys_page(p, row0 + lane, 2 * pp + 1);
        }
        const unsigned needmask = __ballot_sync(0xffffffffu, need);
        if (needmask == 0u) continue;
        const int first = __ffs(needmask) - 1;
        const int fa = __shfl_sync(0xffffffffu, pa, first), fb = __shfl_sync(0xffffffffu, pb, first);
        shared = __ballot_sync(0xffffffffu, need && (pa != fa || pb != fb)) == 0u;
        if (shared) { pa = fa; pb = fb; }
      }
      const int sl_unit = (!end && lane < TS_ROWS && 2 * pp * PS < my_lim) ? my_sl : -1;
      int sl4[TS_ROWS];
#pragma unroll
      for (int i = 0; i < TS_ROWS; ++i) sl4[i] = __shfl_sync(0xffffffffu, sl_unit, i);
      const bool newgroup = !end && row0 != issued_group;
      if (newgroup) {
        issued_group = row0;
        if (lane == 0) {
          const int qb = qc & 1;
          if (ako::tc::mbar_wait(ako::smem_u32(&s_q_empty[qb]), (uint32_t)(((qc >> 1) & 1) ^ 1), &g_dsa_status, 1)) {
            const uint32_t bar = ako::smem_u32(&s_q_full[qb]);
            ako::tc::mbar_arrive_expect_tx(bar, TS_Q_BYTES + TS_W_BYTES);
#pragma unroll
            for (int i = 0; i < TS_ROWS; ++i) {
              const int r = min(row0 + i, p.rows - 1);
              ako::tc::tma_load_2d(q_base + qb * TS_Q_BYTES + i * NH * HD, &tm_q, 0, r * NH, bar);
              ako::tc::bulk_load_1d(w_base + qb * TS_W_BYTES + i * NH * 4, p.weights + (int64_t)r * NH, NH * 4, bar);
            }
          } else {
            ok = 0;
          }
        }
        ++qc;
      }
      const int subs = (end || shared) ? 1 : TS_ROWS;
      for (int s = 0; s < subs; ++s, ++ac) {
        const int pas = __shfl_sync(0xffffffffu, pa, shared ? 0 : s);
        const int pbs = __shfl_sync(0xffffffffu, pb, shared ? 0 : s);
        if (lane == 0 && ok) {
          const int slot = ac % TS_SLOTS, stage = ac % TS_A_STAGES;
          if (!ako::tc::mbar_wait(ako::smem_u32(&s_slot_empty[slot]), (uint32_t)(((ac / TS_SLOTS) & 1) ^ 1), &g_dsa_status, 2)) {
            ok = 0;
          } else {
            unsigned char* sp = slot_ptr + slot * TS_SLOT_BYTES;
            const uint32_t sbar = ako::smem_u32(&s_slot_full[slot]);
            if (s == 0) {
              ScoreDesc* d = reinterpret_cast<ScoreDesc*>(sp + 2 * PS * 4);
              d->row0 = row0;
              d->pp = pp;
              d->flags = (shared ? TS_F_SHARED : 0) | (newgroup ? TS_F_NEWGROUP : 0) | (end ? TS_F_END : 0);
#pragma unroll
              for (int i = 0; i < TS_ROWS; ++i) d->sl[i] = sl4[i];
            }
            if (end) {
              ako::tc::mbar_arrive(sbar);
            } else {
              ako::tc::mbar_arrive_expect_tx(sbar, 2 * PS * 4);
              const uint32_t sdst = slot_base + slot * TS_SLOT_BYTES;
              ako::tc::bulk_load_1d(sdst, p.cache + (int64_t)pas * PAGE_BYTES + PS * HD, PS * 4, sbar);
              ako::tc::bulk_load_1d(sdst + PS * 4, p.cache + (int64_t)pbs * PAGE_BYTES + PS * HD, PS * 4, sbar);
              if (!ako::tc::mbar_wait(ako::smem_u32(&s_a_empty[stage]), (uint32_t)(((ac / TS_A_STAGES) & 1) ^ 1), &g_dsa_status, 3)) {
                ok = 0;
              } else {
                const uint32_t bar = ako::smem_u32(&s_a_full[stage]);
                const uint32_t dst = a_base + stage * TS_A_BYTES;
                ako::tc::mbar_arrive_expect_tx(bar, TS_A_BYTES);
                ako::tc::tma_load_3d(dst, &tm_k, 0, 0, pas, bar);
                ako::tc::tma_load_3d(dst + PS * HD, &tm_k, 0, 0, pbs, bar);
              }
            }
          }
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
    }
  } else if (warp == 8) {
    // ================================ MMA issuer ===============================================
    if (lane == 0) {
      constexpr uint32_t IDESC_SHARED = ako::tc::idesc_e4m3_f32(128, TS_N);
      constexpr uint32_t IDESC_ROW = ako::tc::idesc_e4m3_f32(128, NH);
      int ac = 0, qc = 0, uc = 0;
      while (true) {
        const int slot = ac % TS_SLOTS;
        if (!ako::tc::mbar_wait(ako::smem_u32(&s_slot_full[slot]), (uint32_t)((ac / TS_SLOTS) & 1), &g_dsa_status, 4)) break;
        const int flags = reinterpret_cast<const volatile ScoreDesc*>(slot_ptr + slot * TS_SLOT_BYTES + 2 * PS * 4)->flags;
        if (flags & TS_F_END) break;
        if (flags & TS_F_NEWGROUP) {
          if (qc > 0) ako::tc::mma_commit(ako::smem_u32(&s_q_empty[(qc - 1) & 1]));  // previous tile is done with
          if (!ako::tc::mbar_wait(ako::smem_u32(&s_q_full[qc & 1]), (uint32_t)((qc >> 1) & 1), &g_dsa_status, 5)) break;
          ++qc;
        }
        const bool shared = flags & TS_F_SHARED;
        const uint32_t qs = q_base + ((qc - 1) & 1) * TS_Q_BYTES;
        const int buf = uc & 1;
        if (!ako::tc::mbar_wait(ako::smem_u32(&s_acc_empty[buf]), (uint32_t)(((uc >> 1) & 1) ^ 1), &g_dsa_status, 6)) break;
        const int subs = shared ? 1 : TS_ROWS;
        bool ok = true;
        for (int s = 0; s < subs; ++s, ++ac) {
          const int stage = ac % TS_A_STAGES;
          if (!ako::tc::mbar_wait(ako::smem_u32(&s_a_full[stage]), (uint32_t)((ac / TS_A_STAGES) & 1), &g_dsa_status, 7)) { ok = false; break; }
          ako::tc::fence_after_thread_sync();
          const uint32_t sa = a_base + stage * TS_A_BYTES;
          const uint32_t sb = qs + (shared ? 0 : s * NH * HD);
          const uint32_t d = tmem_base + buf * TS_N + (shared ? 0 : s * NH);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            ako::tc::mma_f8(d, ako::tc::smem_desc_k_sw128(sa + ks * 32), ako::tc::smem_desc_k_sw128(sb + ks * 32),
                            shared ? IDESC_SHARED : IDESC_ROW, ks > 0 ? 1u : 0u);
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
    int ac = 0, qc = 0, uc = 0;
    while (true) {
      const int slot0 = ac % TS_SLOTS;
      if (!ako::tc::mbar_wait(ako::smem_u32(&s_slot_full[slot0]), (uint32_t)((ac / TS_SLOTS) & 1), &g_dsa_status, 8)) break;
      const ScoreDesc d = *reinterpret_cast<const ScoreDesc*>(slot_ptr + slot0 * TS_SLOT_BYTES + 2 * PS * 4);
      if (d.flags & TS_F_END) break;
      const bool shared = d.flags & TS_F_SHARED;
      const int subs = shared ? 1 : TS_ROWS;
      if (d.flags & TS_F_NEWGROUP) {
        if (qc > 0) {  // this warp has read the previous group's weights for the last time
          __syncwarp();
          if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&s_q_empty[(qc - 1) & 1]));
        }
        if (!ako::tc::mbar_wait(ako::smem_u32(&s_q_full[qc & 1]), (uint32_t)((qc >> 1) & 1), &g_dsa_status, 9)) break;
        ++qc;
      }
      const float* wrow = reinterpret_cast<const float*>(w_ptr + ((qc - 1) & 1) * TS_W_BYTES) + rh * 2 * NH;
      // key scales of this thread's token for its two rows
      float ksc[2];
      bool ok = true;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int a2 = ac + (shared ? 0 : rh * 2 + i);
        const int sl2 = a2 % TS_SLOTS;
        if (!shared && !ako::tc::mbar_wait(ako::smem_u32(&s_slot_full[sl2]), (uint32_t)((a2 / TS_SLOTS) & 1), &g_dsa_status, 10)) { ok = false; break; }
        ksc[i] = reinterpret_cast<const float*>(slot_ptr + sl2 * TS_SLOT_BYTES)[t];
      }
      if (!ok) break;
      if (!shared) {  // the other rows' slots are released by every warp as well: wait for them first
#pragma unroll
        for (int s = 0; s < TS_ROWS; ++s) {
          const int a2 = ac + s;
          if (!ako::tc::mbar_wait(ako::smem_u32(&s_slot_full[a2 % TS_SLOTS]), (uint32_t)((a2 / TS_SLOTS) & 1), &g_dsa_status, 11)) { ok = false; break; }
        }
        if (!ok) break;
      }
      __syncwarp();
      if (lane == 0) {
        for (int s = 0; s < subs; ++s) ako::tc::mbar_arrive(ako::smem_u32(&s_slot_empty[(ac + s) % TS_SLOTS]));
      }
      ac += subs;

      const int buf = uc & 1;
      if (!ako::tc::mbar_wait(ako::smem_u32(&s_acc_full[buf]), (uint32_t)((uc >> 1) & 1), &g_dsa_status, 12)) break;
      ako::tc::fence_after_thread_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + buf * TS_N + rh * 2 * NH;
      float sum[2] = {0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {  // 32 columns each: row (c>>1) of this thread's pair, heads 32*(c&1)..
        float v[32];
        ako::tc::tmem_ld32(taddr + 32 * c, v);
        const float4* wp = reinterpret_cast<const float4*>(wrow + 32 * c);
        float4 w4[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) w4[j] = wp[j];
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
      const int tok = d.pp * 2 * PS + t;
      if (tok < p.max_pages * PS) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int sl = d.sl[rh * 2 + i];
          if (sl < 0) continue;
          p.scores[(int64_t)(d.row0 + rh * 2 + i) * p.max_pages * PS + tok] = (tok < sl) ? sum[i] * ksc[i] : -INFINITY;
        }
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
