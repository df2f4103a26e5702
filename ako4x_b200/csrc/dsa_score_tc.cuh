// DSA index scores on the 5th-generation tensor cores (tcgen05 + TMEM) fed by TMA; included by
// dsa_indexer.cu inside its anonymous namespace.
//
// score[r, t] = (sum_h w[r,h] * relu(q[r,h,:] . k[t,:])) * kscale[t]. Tokens are the M dimension of
// the MMA (128 tokens = two 64-token cache pages), the 64 heads of up to EIGHT query rows the N
// dimension (N = 512 = all of TMEM, as four accumulators of 128 columns = two rows each), K = 128
// e4m3 values (four tcgen05.mma K32 steps). With tokens on the TMEM lanes, relu, the head weights
// and the head reduction are plain per-thread arithmetic on the accumulator columns: no shuffles.
// That arithmetic (two CUDA-core instructions per accumulator element) costs about as much as the
// MMA, so it gets sixteen warps.
//
// A unit of work is (group of 8 consecutive query rows, pair of logical pages). When the rows map
// that page pair to the same physical pages (consecutive tokens of one sequence, the prefill case)
// the key tile is loaded ONCE for all eight rows -- every key byte brought into shared memory feeds
// 8 x 64 dot products -- and runs as four N = 128 MMA sequences; otherwise the unit runs as eight
// N = 64 sequences, one key tile each. A persistent CTA takes a contiguous range of units, so the
// 64 KB query tile of a row group stays in shared memory while the CTA sweeps pages (one buffer: a
// group is ~256 units, the refill bubble is small).
//   warp 20     producer. Describe step: each of 16 lanes reads the block table and sequence
//               lengths of one of the next 16 units and writes one record per key tile into shared
//               memory. Issue step: up to six lanes at a time take one record each and issue its
//               copies (key tile: 6-stage ring, a page is a [64 x 128 B] box of a 3-D tensor map
//               over the 8448-byte pages; per unit a slot of an 8-deep ring that carries the key
//               scales and the unit's descriptor, so that no other warp touches the block table;
//               query tile + head weights per row group). A record that starts a row group always
//               opens an issue step, so every wait of a step depends only on earlier steps;
//   warps 16-19 MMA issuers, one thread each; warps 0-15 epilogue, four teams of four warps.
//               Accumulator a (rows 2a, 2a+1 of the group) has its own issuer and its own team: the
//               issuer runs the N = 128 MMAs of its rows for every unit, the team reads the result
//               (thread (w, l): token 32*(w%4)+l, both rows). The chain MMA -> commit -> team's
//               TMEM loads -> release -> next MMA is about a thousand cycles of latency per
//               accumulator (commit -> waiter ~300 cycles, arrive -> waiter ~170, every step of an
//               issuer 50-100); four chains in flight cover the tensor pipe's time for a unit.
// Every reader of TMA-written shared memory waits on the mbarrier the copy completes on. Every
// wait is bounded; a timeout sets the status word and all roles unwind.

constexpr int TS_ROWS = 8;                      // query rows per unit
constexpr int TS_N = TS_ROWS * NH;              // 512 accumulator columns
constexpr int TS_A_BYTES = 2 * PS * HD;         // 16 KB: two pages of e4m3 keys
constexpr int TS_Q_BYTES = TS_N * HD;           // 64 KB: eight rows of e4m3 queries
constexpr int TS_W_BYTES = TS_N * 4;            // 2 KB: their head weights
constexpr int TS_A_STAGES = 6;
constexpr int TS_SLOTS = 8;                     // per-unit ring: key scales + descriptor
constexpr int TS_SCALE_BYTES = 2 * PS * 4;      // 128 key scales of one key tile
constexpr int TS_SLOT_BYTES = TS_ROWS * TS_SCALE_BYTES + 64;
constexpr int TS_DESCRIBE = 16;                 // units described per producer round (one per lane)
constexpr int TS_RECS = TS_DESCRIBE * TS_ROWS + 1;
constexpr int TS_REC_BYTES = 80;
constexpr int TS_SMEM = TS_Q_BYTES + TS_A_STAGES * TS_A_BYTES + TS_W_BYTES + TS_SLOTS * TS_SLOT_BYTES +
                        TS_RECS * TS_REC_BYTES + 1024;
constexpr int TS_ACCS = 4;                      // accumulators = teams = issuers
constexpr int TS_ACC_COLS = TS_N / TS_ACCS;     // 128 columns: two query rows
constexpr int TS_TEAM_WARPS = 4;
constexpr int TS_EPI_WARPS = TS_ACCS * TS_TEAM_WARPS;
constexpr int TS_MMA_WARP = TS_EPI_WARPS, TS_PRODUCER_WARP = TS_EPI_WARPS + TS_ACCS;  // issuers: warps 16-19
constexpr int TS_THREADS = (TS_EPI_WARPS + TS_ACCS + 1) * 32;

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

// Unit descriptor, written by the producer into the unit's ring slot.
struct ScoreDesc {
  int row0;           // first query row of the group
  int pp;             // page pair: logical pages 2*pp, 2*pp+1
  int flags;          // TS_F_*
  int qc;             // ordinal of the row group inside this CTA (phase of the query buffer)
  int sl[TS_ROWS];    // row's sequence length, or -1 when the row takes nothing from this unit
  int ac0;            // ordinal of the unit's first key tile inside this CTA (key stage = ordinal % stages)
  int pad[3];
};
// NEWGROUP: first unit of its row group in this CTA; LASTGROUP: last one (the query buffer is
// handed back after it).
constexpr int TS_F_SHARED = 1, TS_F_NEWGROUP = 2, TS_F_END = 4, TS_F_LASTGROUP = 8;

// One key tile to load: the producer's describe step writes these, its issue step reads them.
struct ScoreRec {
  int pa, pb;         // physical pages
  int uo;             // ordinal of the unit inside this CTA (ring slot = uo % TS_SLOTS)
  int sub;            // which key tile of the unit (0 for a shared one, else the row)
  ScoreDesc d;
};
static_assert(sizeof(ScoreDesc) == 64 && sizeof(ScoreRec) == TS_REC_BYTES, "record size");

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
  __shared__ __align__(8) uint64_t s_q_full, s_q_empty;
  __shared__ __align__(8) uint64_t s_acc_full[TS_ACCS];
  __shared__ __align__(8) uint64_t s_acc_empty[TS_ACCS];
  __shared__ __align__(8) uint64_t s_slot_full[TS_SLOTS];
  __shared__ __align__(8) uint64_t s_slot_empty[TS_SLOTS];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_err;  // code of a wait of this CTA that gave up (0 = none), published on exit

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned char* smem_al = smem_raw + ((1024u - (ako::smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t q_base = ako::smem_u32(smem_al);
  const uint32_t a_base = q_base + TS_Q_BYTES;
  unsigned char* w_ptr = smem_al + TS_Q_BYTES + TS_A_STAGES * TS_A_BYTES;
  unsigned char* slot_ptr = w_ptr + TS_W_BYTES;
  const uint32_t w_base = ako::smem_u32(w_ptr);
  const uint32_t slot_base = ako::smem_u32(slot_ptr);

  if (tid == 0) {
    s_err = 0;
    for (int s = 0; s < TS_A_STAGES; ++s) {
      ako::tc::mbar_init(ako::smem_u32(&s_a_full[s]), 1);
      ako::tc::mbar_init(ako::smem_u32(&s_a_empty[s]), TS_ACCS);  // every issuer passes every key tile
    }
    ako::tc::mbar_init(ako::smem_u32(&s_q_full), 1);
    ako::tc::mbar_init(ako::smem_u32(&s_q_empty), TS_ACCS + TS_EPI_WARPS);   // every issuer + every epilogue warp
    for (int a = 0; a < TS_ACCS; ++a) {
      ako::tc::mbar_init(ako::smem_u32(&s_acc_full[a]), 1);
      ako::tc::mbar_init(ako::smem_u32(&s_acc_empty[a]), TS_TEAM_WARPS);
    }
    for (int s = 0; s < TS_SLOTS; ++s) {
      ako::tc::mbar_init(ako::smem_u32(&s_slot_full[s]), 1);
      ako::tc::mbar_init(ako::smem_u32(&s_slot_empty[s]), TS_ACCS + TS_EPI_WARPS);  // every issuer and warp reads every slot
    }
    ako::tc::mbar_init_fence();
  }
  if (warp == TS_MMA_WARP) ako::tc::tmem_alloc(ako::smem_u32(&s_tmem_base), 512);
  ako::tc::fence_before_thread_sync();
  __syncthreads();
  ako::tc::fence_after_thread_sync();
  const uint32_t tmem_base = s_tmem_base;

  const int pairs = (p.max_pages + 1) / 2;
  const int groups = (p.rows + TS_ROWS - 1) / TS_ROWS;
  const int64_t total = (int64_t)groups * pairs;
  const int u_begin = (int)(total * blockIdx.x / gridDim.x);
  const int u_end = (int)(total * (blockIdx.x + 1) / gridDim.x);

  if (warp == TS_PRODUCER_WARP) {
    // ================================ producer (whole warp) ====================================
    if (lane == 0) {
      ako::tc::tma_prefetch_desc(&tm_q);
      ako::tc::tma_prefetch_desc(&tm_k);
    }
    ScoreRec* recs = reinterpret_cast<ScoreRec*>(slot_ptr + TS_SLOTS * TS_SLOT_BYTES);
    const unsigned lt_mask = (1u << lane) - 1u;
    int ac = 0, qc_base = 0, uo_base = 0;
    bool done = false;
    for (int ubase = u_begin; !done; ubase += TS_DESCRIBE) {
      // ---- describe: lane l < 16 takes unit ubase + l; the END record follows the last unit in the
      // first round that has a lane to spare.
      const int unit = ubase + lane;
      int nsubs = 0, flags = 0, row0 = 0, pp = 0;
      int pa[TS_ROWS], pb[TS_ROWS], sl[TS_ROWS];
#pragma unroll
      for (int i = 0; i < TS_ROWS; ++i) { pa[i] = 0; pb[i] = 0; sl[i] = -1; }
      const int n_left = max(0, u_end - ubase);
      const bool last_round = n_left <= TS_DESCRIBE - 1;
      if (lane < TS_DESCRIBE && unit < u_end) {
        row0 = (unit / pairs) * TS_ROWS;
        pp = unit % pairs;
        bool any = false, shared = true;
        int fa = 0, fb = 0, maxlim = 0;
#pragma unroll
        for (int i = 0; i < TS_ROWS; ++i) {
          const int r = row0 + i;
          int s0 = (r < p.rows) ? __ldg(p.seq_lens + r) : 0;
          if (s0 <= 0 || (p.skip_short && s0 <= TOPK)) s0 = 0;
          const int lim = min(s0, p.max_pages * PS);
          maxlim = max(maxlim, lim);
          const bool need = 2 * pp * PS < lim;
          pa[i] = phys_page(p, r, 2 * pp);
          pb[i] = phys_page(p, r, 2 * pp + 1);
          if (need) {
            sl[i] = s0;
            if (!any) { fa = pa[i]; fb = pb[i]; }
            else if (pa[i] != fa || pb[i] != fb) shared = false;
            any = true;
          }
        }
        if (any) {
          nsubs = shared ? 1 : TS_ROWS;
          // A group's needed page pairs are a prefix [0, last_pp]: its first unit in this CTA's
          // range opens it, and the unit at last_pp (or the end of the range) closes it.
          const int last_pp = (maxlim - 1) / (2 * PS);
          flags = (shared ? TS_F_SHARED : 0) | ((pp == 0 || unit == u_begin) ? TS_F_NEWGROUP : 0) |
                  ((pp == last_pp || unit == u_end - 1) ? TS_F_LASTGROUP : 0);
          if (shared) {
#pragma unroll
            for (int i = 0; i < TS_ROWS; ++i) { pa[i] = fa; pb[i] = fb; }
          }
        }
      } else if (last_round && lane == n_left) {
        nsubs = 1;
        flags = TS_F_END;
      }
      if (last_round) done = true;
      int off = nsubs;  // exclusive prefix sum of nsubs over the warp
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, off, o);
        if (lane >= o) off += y;
      }
      const int nrec = __shfl_sync(0xffffffffu, off, 31);
      off -= nsubs;
      const unsigned ngmask = __ballot_sync(0xffffffffu, (flags & TS_F_NEWGROUP) != 0);
      // the group ordinal of a unit = groups opened before it or by it, minus one
      const int qc = qc_base + __popc(ngmask & (lt_mask | (1u << lane))) - 1;
      qc_base += __popc(ngmask);
      const unsigned umask = __ballot_sync(0xffffffffu, nsubs > 0);
      const int uo = uo_base + __popc(umask & lt_mask);
      uo_base += __popc(umask);
      for (int sidx = 0; sidx < nsubs; ++sidx) {
        ScoreRec& rc = recs[off + sidx];
        int a = pa[0], b = pb[0];
#pragma unroll
        for (int i = 1; i < TS_ROWS; ++i)
          if (i == sidx) { a = pa[i]; b = pb[i]; }
        rc.pa = a;
        rc.pb = b;
        rc.uo = uo;
        rc.sub = sidx;
        rc.d.row0 = row0;
        rc.d.pp = pp;
        rc.d.flags = (sidx == 0) ? flags : (flags & ~TS_F_NEWGROUP);
        rc.d.qc = qc;
        rc.d.ac0 = ac + off;  // every record of earlier rounds has been issued: ac counts them
#pragma unroll
        for (int i = 0; i < TS_ROWS; ++i) rc.d.sl[i] = sl[i];
      }
      __syncwarp();

      // ---- issue: up to TS_A_STAGES records per step, one per lane
      int k = 0;
      while (k < nrec) {
        const bool have = lane < TS_A_STAGES && k + lane < nrec;
        ScoreRec rc;
        rc.d.flags = 0;
        if (have) rc = recs[k + lane];
        const unsigned cut = __ballot_sync(0xffffffffu, have && lane > 0 && (rc.d.flags & TS_F_NEWGROUP));
        int nb = min(TS_A_STAGES, nrec - k);
        if (cut) nb = min(nb, __ffs(cut) - 1);
        bool ok = true;
        if (lane < nb) {
          const int a = ac + lane;
          const int slot = rc.uo % TS_SLOTS, stage = a % TS_A_STAGES;
          if (rc.d.flags & TS_F_NEWGROUP) {
            // one query buffer: group qc is loaded once everybody has handed back group qc-1
            ok = ako::tc::mbar_wait(ako::smem_u32(&s_q_empty), (uint32_t)((rc.d.qc & 1) ^ 1), &s_err, 1);
            if (ok) {
              const uint32_t bar = ako::smem_u32(&s_q_full);
              ako::tc::mbar_arrive_expect_tx(bar, TS_Q_BYTES + TS_W_BYTES);
#pragma unroll
              for (int i = 0; i < TS_ROWS; ++i) {
                const int r = min(rc.d.row0 + i, p.rows - 1);
                ako::tc::tma_load_2d(q_base + i * NH * HD, &tm_q, 0, r * NH, bar);
                ako::tc::bulk_load_1d(w_base + i * NH * 4, p.weights + (int64_t)r * NH, NH * 4, bar);
              }
            }
          }
          // every key tile of the unit waits for the slot: the tiles of one unit may be issued together
          ok = ok && ako::tc::mbar_wait(ako::smem_u32(&s_slot_empty[slot]), (uint32_t)(((rc.uo / TS_SLOTS) & 1) ^ 1), &s_err, 2);
          if (ok) {
            const uint32_t sbar = ako::smem_u32(&s_slot_full[slot]);
            if (rc.sub == 0) {
              *reinterpret_cast<ScoreDesc*>(slot_ptr + slot * TS_SLOT_BYTES + TS_ROWS * TS_SCALE_BYTES) = rc.d;
              if (rc.d.flags & TS_F_END) ako::tc::mbar_arrive(sbar);
              else ako::tc::mbar_arrive_expect_tx(sbar, ((rc.d.flags & TS_F_SHARED) ? 1 : TS_ROWS) * TS_SCALE_BYTES);
            }
            if (!(rc.d.flags & TS_F_END)) {
              const uint32_t sdst = slot_base + slot * TS_SLOT_BYTES + rc.sub * TS_SCALE_BYTES;
              ako::tc::bulk_load_1d(sdst, p.cache + (int64_t)rc.pa * PAGE_BYTES + PS * HD, PS * 4, sbar);
              ako::tc::bulk_load_1d(sdst + PS * 4, p.cache + (int64_t)rc.pb * PAGE_BYTES + PS * HD, PS * 4, sbar);
              ok = ako::tc::mbar_wait(ako::smem_u32(&s_a_empty[stage]), (uint32_t)(((a / TS_A_STAGES) & 1) ^ 1), &s_err, 3);
              if (ok) {
                const uint32_t bar = ako::smem_u32(&s_a_full[stage]);
                const uint32_t dst = a_base + stage * TS_A_BYTES;
                ako::tc::mbar_arrive_expect_tx(bar, TS_A_BYTES);
                ako::tc::tma_load_3d(dst, &tm_k, 0, 0, rc.pa, bar);
                ako::tc::tma_load_3d(dst + PS * HD, &tm_k, 0, 0, rc.pb, bar);
              }
            }
          }
        }
        ac += nb;
        k += nb;
        if (__ballot_sync(0xffffffffu, !ok) != 0u) { done = true; break; }
      }
      __syncwarp();  // the records are rewritten by the next describe step
    }
  } else if (warp >= TS_MMA_WARP && warp < TS_MMA_WARP + TS_ACCS) {
    // ================================ MMA issuers ==============================================
    // The barrier waits and the descriptor read for the issuer's NEXT key tile are done between
    // the second and third MMA of the current one.
    if (lane == 0) {
      constexpr uint32_t IDESC_SHARED = ako::tc::idesc_e4m3_f32(128, TS_ACC_COLS);
      constexpr uint32_t IDESC_ROW = ako::tc::idesc_e4m3_f32(128, NH);
      // a_lo, b_lo: descriptor low words; mma: this issuer's rows take part in the tile;
      // q_done: the tile is the unit's last and the unit the group's last
      struct Tile { uint32_t a_lo, b_lo, d, idesc; int stage, acc_wait; bool last, mma, q_done; };
      const int me = warp - TS_MMA_WARP;    // accumulator = row pair (rows 2*me, 2*me+1 of the group)
      const uint32_t a_lo0 = ako::tc::smem_desc_lo(a_base);
      const uint32_t q_lo = ako::tc::smem_desc_lo(q_base) + me * ((2 * NH * HD) >> 4);  // this pair's rows
      const uint32_t acc = tmem_base + me * TS_ACC_COLS;
      int n = 0;                            // units taken so far
      int ac = 0, subs = 0, sub = 0;        // current unit: next key tile ordinal, tiles, tiles issued
      bool shared = true, last_unit = false;
      int acc_wait = 1;
      // 1: tile ready, 0: END record, -1: a wait gave up
      auto prepare = [&](Tile& t) -> int {
        if (sub == subs) {  // next unit
          const int slot = n % TS_SLOTS;
          if (!ako::tc::mbar_wait(ako::smem_u32(&s_slot_full[slot]), (uint32_t)((n / TS_SLOTS) & 1), &s_err, 4)) return -1;
          const volatile ScoreDesc* dp = reinterpret_cast<const volatile ScoreDesc*>(slot_ptr + slot * TS_SLOT_BYTES + TS_ROWS * TS_SCALE_BYTES);
          const int flags = dp->flags, qc = dp->qc;
          ac = dp->ac0;
          ako::tc::mbar_arrive(ako::smem_u32(&s_slot_empty[slot]));
          if (flags & TS_F_END) return 0;
          if ((flags & TS_F_NEWGROUP) &&
              !ako::tc::mbar_wait(ako::smem_u32(&s_q_full), (uint32_t)(qc & 1), &s_err, 5)) return -1;
          shared = flags & TS_F_SHARED;
          last_unit = flags & TS_F_LASTGROUP;
          subs = shared ? 1 : TS_ROWS;
          sub = 0;
          acc_wait = (n & 1) ^ 1;  // parity to wait for before the unit's first MMA
          ++n;
        }
        // Tiles of the other row pairs are waited for as well: the stage's release counts all
        // issuers, and this keeps an issuer from arriving for the stage's next use too early.
        const int stage = ac % TS_A_STAGES;
        if (!ako::tc::mbar_wait(ako::smem_u32(&s_a_full[stage]), (uint32_t)((ac / TS_A_STAGES) & 1), &s_err, 7)) return -1;
        ako::tc::fence_after_thread_sync();
        t.mma = shared || (sub >> 1) == me;
        t.a_lo = a_lo0 + stage * (TS_A_BYTES >> 4);
        t.b_lo = q_lo + (shared ? 0 : (sub & 1) * ((NH * HD) >> 4));
        t.d = acc + (shared ? 0 : (sub & 1) * NH);
        t.idesc = shared ? IDESC_SHARED : IDESC_ROW;
        t.stage = stage;
        t.acc_wait = (shared || sub == 2 * me) ? acc_wait : -1;  // first tile that writes the accumulator
        t.last = shared || sub == 2 * me + 1;                    // last tile that writes it
        t.q_done = last_unit && sub == subs - 1;
        ++sub;
        ++ac;
        return 1;
      };
      Tile cur, nxt;
      int r = prepare(cur);
      while (r == 1) {
        if (cur.mma) {
          // This issuer's units share one accumulator: the team must have read the previous result.
          if (cur.acc_wait >= 0 &&
              !ako::tc::mbar_wait(ako::smem_u32(&s_acc_empty[me]), (uint32_t)cur.acc_wait, &s_err, 6)) break;
          ako::tc::mma_f8_lohi<false>(cur.d, cur.a_lo, cur.b_lo, cur.idesc);  // K = 32 slices: +32 B = +2
          ako::tc::mma_f8_lohi<true>(cur.d, cur.a_lo + 2, cur.b_lo + 2, cur.idesc);
          if (!cur.q_done) r = prepare(nxt);
          ako::tc::mma_f8_lohi<true>(cur.d, cur.a_lo + 4, cur.b_lo + 4, cur.idesc);
          ako::tc::mma_f8_lohi<true>(cur.d, cur.a_lo + 6, cur.b_lo + 6, cur.idesc);
          ako::tc::mma_commit(ako::smem_u32(&s_a_empty[cur.stage]));
          if (cur.last) ako::tc::mma_commit(ako::smem_u32(&s_acc_full[me]));
        } else {
          ako::tc::mbar_arrive(ako::smem_u32(&s_a_empty[cur.stage]));
          if (!cur.q_done) r = prepare(nxt);
        }
        if (cur.q_done) {
          // The group's last tile: hand the query buffer back once this issuer's MMAs are done,
          // and only then look at the next unit (its group cannot be loaded before).
          ako::tc::mma_commit(ako::smem_u32(&s_q_empty));
          r = prepare(nxt);
        }
        cur = nxt;
      }
    }
  } else {
    // ================================ epilogue (four teams) =======================================
    const int team = warp / TS_TEAM_WARPS;  // accumulator = row pair
    const int q = warp & 3;             // TMEM lane quarter
    const int t = 32 * q + lane;        // token inside the unit
    const uint32_t tmem_team = tmem_base + ((uint32_t)(32 * q) << 16) + team * TS_ACC_COLS;
    const float* wrow = reinterpret_cast<const float*>(w_ptr) + team * 2 * NH;
    float* orow[2] = {nullptr, nullptr};
    for (int n = 0;; ++n) {
      const int slot = n % TS_SLOTS;
      const unsigned char* sp = slot_ptr + slot * TS_SLOT_BYTES;
      if (!ako::tc::mbar_wait(ako::smem_u32(&s_slot_full[slot]), (uint32_t)((n / TS_SLOTS) & 1), &s_err, 8)) break;
      const int4 d0 = *reinterpret_cast<const int4*>(sp + TS_ROWS * TS_SCALE_BYTES);  // row0, pp, flags, qc
      const int row0 = d0.x, pp = d0.y, flags = d0.z, qc = d0.w;
      if (flags & TS_F_END) break;
      const int2 sl2 = *reinterpret_cast<const int2*>(sp + TS_ROWS * TS_SCALE_BYTES + 16 + team * 8);  // sl[2*team], +1
      if (flags & TS_F_NEWGROUP) {
        if (!ako::tc::mbar_wait(ako::smem_u32(&s_q_full), (uint32_t)(qc & 1), &s_err, 9)) break;
#pragma unroll
        for (int i = 0; i < 2; ++i)
          orow[i] = p.scores + (int64_t)min(row0 + team * 2 + i, p.rows - 1) * p.max_pages * PS;
      }
      // key scales of this thread's token for its two rows
      const bool shared = flags & TS_F_SHARED;
      float ksc[2];
#pragma unroll
      for (int i = 0; i < 2; ++i)
        ksc[i] = reinterpret_cast<const float*>(sp + (shared ? 0 : team * 2 + i) * TS_SCALE_BYTES)[t];
      __syncwarp();
      if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&s_slot_empty[slot]));

      if (!ako::tc::mbar_wait(ako::smem_u32(&s_acc_full[team]), (uint32_t)(n & 1), &s_err, 10)) break;
      ako::tc::fence_after_thread_sync();
      // 32 accumulator columns per step: row (c>>1) of this thread's pair, heads 32*(c&1)...
      // relu is one instruction per element; the weighted sums go two elements per instruction
      // (fma.rn.f32x2): this loop is bound by instruction issue, not by the tensor pipe.
      float2 part[2][2] = {{{0.f, 0.f}, {0.f, 0.f}}, {{0.f, 0.f}, {0.f, 0.f}}};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float v[32];
        ako::tc::tmem_ld32(tmem_team + 32 * c, v);
        ako::tc::tmem_ld_wait_regs(v);
        if (c == 3) {  // the accumulator is in registers: release it
          ako::tc::fence_before_thread_sync();
          __syncwarp();
          if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&s_acc_empty[team]));
        }
        const float4* wp = reinterpret_cast<const float4*>(wrow + 32 * c);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 w4 = wp[j];
          part[c >> 1][0] = __ffma2_rn(make_float2(fmaxf(v[4 * j + 0], 0.f), fmaxf(v[4 * j + 1], 0.f)),
                                       make_float2(w4.x, w4.y), part[c >> 1][0]);
          part[c >> 1][1] = __ffma2_rn(make_float2(fmaxf(v[4 * j + 2], 0.f), fmaxf(v[4 * j + 3], 0.f)),
                                       make_float2(w4.z, w4.w), part[c >> 1][1]);
        }
      }
      if (flags & TS_F_LASTGROUP) {  // this warp has read the group's weights for the last time
        __syncwarp();
        if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&s_q_empty));
      }
      const int tok = pp * 2 * PS + t;
      if (tok < p.max_pages * PS) {
        const int sls[2] = {sl2.x, sl2.y};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          if (sls[i] < 0) continue;
          const float sum = (part[i][0].x + part[i][0].y) + (part[i][1].x + part[i][1].y);
          orow[i][tok] = (tok < sls[i]) ? sum * ksc[i] : -INFINITY;
        }
      }
    }
  }

  ako::tc::fence_before_thread_sync();
  __syncthreads();
  if (tid == 0 && s_err != 0) atomicCAS(&g_dsa_status, 0, s_err);
  if (warp == TS_MMA_WARP) {
    ako::tc::fence_after_thread_sync();
    ako::tc::tmem_dealloc(tmem_base, 512);
  }
}
