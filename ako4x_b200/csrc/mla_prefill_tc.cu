// Causal paged MLA prefill on the 5th-generation tensor cores (tcgen05 + TMEM) fed by TMA.
//
// Two launches. (1) gather: the keys of all sequences are copied from the paged caches into a
// contiguous [tokens, 576] matrix Kc (ckv | kpe) and, transposed, into Vt [512, columns] (every
// sequence starts at a multiple of 8 columns so a TMA box may start there). (2) attention: a CTA
// owns a tile of 8 consecutive query tokens of one sequence (128 rows: token x head) and ONE half of
// the 512 output columns; the O tile would fill all of TMEM, so the two halves are separate CTAs that
// both compute S. Per tile of 128 keys:
//   S  = Q Kc^T        128 x 128, reduction 576 streamed in nine 64-column chunks of Q and Kc through
//                      a 5-stage TMA ring; 36 tcgen05.mma (bf16, N = 128, K = 16) into one of two
//                      128-column TMEM buffers;
//   P  = softmax step  four warps, one thread per row: two sweeps over the S buffer (row maximum,
//                      then exp2), causal mask, running (m, l); P is written back with tcgen05.st as
//                      packed bf16 pairs over the first 64 columns of the S buffer it was read from,
//                      alpha = 2^(m_old-m_new) goes to shared memory;
//   PV = P Vt^T        128 x 256, 8 MMAs (N = 256) with the A operand (P) taken from TMEM, into a
//                      256-column TMEM buffer, NOT accumulated; their commit frees the S buffer;
//   O  = O alpha + PV  eight warps hold the 128 x 256 fp32 O tile in registers (128 per thread) and
//                      fold every PV tile in -- no rescaling of TMEM contents.
// S of tile j+1 streams in while the softmax works on tile j; PV of tile j is issued by a thread of
// its own as soon as P is complete. The kernel is bound by the bytes that cross shared memory (TMA
// writes + MMA operand reads, 128 B/clk per SM), which is why P stays in TMEM.
// Warps: 0-7 O accumulation (setmaxnreg 184), 8-11 softmax (104), 12 Q/K producer, 13 S issuer,
// 14 V producer, 15 PV issuer (40). Rows of a partial last tile and keys past the causal limit are
// masked; every mbarrier wait is bounded and a timeout sets the status word. Shared memory: ring
// 160 KB + Vt tile 64 KB + 3 KB (alpha, l, mbarriers) = the whole 227 KB, none of it static.
#include "mla_prefill_tc.h"

#include <cuda_bf16.h>

#include "ako4x_b200.h"
#include "common.cuh"
#include "tcgen05.cuh"
#include "tma_host.cuh"

namespace {

constexpr int H = 16, DC = 512, DP = 64, DQK = DC + DP;
constexpr int QT = 8;                     // query tokens per tile
constexpr int BM = QT * H;                // 128 rows
constexpr int BK = 128;                   // keys per tile
constexpr int NCH = DQK / 64;             // nine reduction chunks of 64 columns
constexpr int CH_BYTES = BM * 128;        // one 128-row x 64-column bf16 chunk: 16 KB
constexpr int ST_BYTES = 2 * CH_BYTES;    // Q chunk + K chunk
constexpr int NST = 5;
constexpr int V_BYTES = 2 * 256 * 128;    // two boxes of 256 rows x 64 keys
constexpr int AUX_BYTES = 3072;           // alpha[4][128], final l[128], mbarriers, TMEM address, work item
// exactly the 227 KB a CTA may have: no static shared memory in this kernel, so that the dynamic
// region starts on a 1024-byte boundary (checked at entry) and needs no alignment slack
constexpr int SMEM = NST * ST_BYTES + V_BYTES + AUX_BYTES;
static_assert(SMEM <= 232448, "shared memory per CTA");
static_assert(2560 + (2 * NST + 11) * 8 + 8 + 16 <= AUX_BYTES, "aux region");
constexpr int THREADS = 512;
constexpr int REGS_O = 184, REGS_SOFTMAX = 104, REGS_OTHER = 40;  // 2*184 + 104 + 40 = 4*128
constexpr float NEG = -1.0e30f;           // finite stand-in for -inf

// Wait status of the CURRENT call (cleared by the gather kernel that starts every call, so a code
// left by an earlier call cannot make this call's waits give up early) and the sticky word that
// ako_mla_prefill_tc_status() reports. The per-call word stays in global memory on purpose: with
// the word in shared memory, as in the other kernels, this kernel measured 18 % slower (1 463 ->
// 1 725 us at the benchmark shape; the roles that run on 40 registers do not take the extra pointer
// well).
__device__ int g_pf_status = 0;
__device__ int g_pf_sticky = 0;

struct PfParams {
  const int32_t* qo_indptr;
  const int32_t* kv_indptr;
  __nv_bfloat16* o;
  float* lse;
  float scale_log2;
  int batch, page_size;
};

// ---------------------------------------------------------------------------------------------
// gather: 32 key tokens per CTA
// ---------------------------------------------------------------------------------------------
constexpr int G_TOK = 32, G_PITCH = 520;  // bf16 elements per staged row (1040 B: 16-byte aligned)

__host__ __device__ inline int64_t vt_start(int64_t first_token, int b) {
  return ((first_token + 7) / 8) * 8 + 8 * (int64_t)b;  // non-overlapping and a multiple of 8 columns
}

__global__ void __launch_bounds__(256) mla_prefill_gather_kernel(
    const uint4* __restrict__ ckv, const uint4* __restrict__ kpe, const int32_t* __restrict__ kv_indices,
    const int32_t* __restrict__ kv_indptr, int batch, int page_size, int64_t ntok, uint4* __restrict__ kc,
    __nv_bfloat16* __restrict__ vt, int64_t vt_cols) {
  __shared__ __align__(16) __nv_bfloat16 s_v[G_TOK * G_PITCH];
  __shared__ int64_t s_row[G_TOK];
  __shared__ int64_t s_col[G_TOK];
  const int tid = threadIdx.x;
  const int64_t g0 = (int64_t)blockIdx.x * G_TOK;
  if (blockIdx.x == 0 && tid == 0) g_pf_status = 0;  // this call's wait status starts clean
  if (tid < G_TOK) {
    const int64_t g = g0 + tid;
    int64_t row = 0, col = -1;
    if (g < ntok) {
      const int64_t pg = kv_indices[g / page_size];
      row = pg * page_size + g % page_size;
      // sequence of this token: kv_indptr counts pages
      int b = 0;
      const int64_t page_slot = g / page_size;
      while (b + 1 < batch && (int64_t)kv_indptr[b + 1] <= page_slot) ++b;
      const int64_t first = (int64_t)kv_indptr[b] * page_size;
      col = vt_start(first, b) + (g - first);
    }
    s_row[tid] = row;
    s_col[tid] = col;
  }
  __syncthreads();
  for (int i = tid; i < G_TOK * 72; i += 256) {
    const int t = i / 72, c = i % 72;
    if (g0 + t >= ntok) continue;
    const int64_t row = s_row[t];
    const uint4 v = (c < 64) ? __ldg(ckv + row * 64 + c) : __ldg(kpe + row * 8 + (c - 64));
    kc[(g0 + t) * 72 + c] = v;
    if (c < 64) *reinterpret_cast<uint4*>(s_v + t * G_PITCH + c * 8) = v;
  }
  __syncthreads();
  for (int i = tid; i < DC * G_TOK; i += 256) {
    const int d = i / G_TOK, t = i % G_TOK;
    const int64_t col = s_col[t];
    if (col >= 0) vt[(int64_t)d * vt_cols + col] = s_v[t * G_PITCH + d];
  }
}

// ---------------------------------------------------------------------------------------------
// attention
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS, 1)
mla_prefill_tc_kernel(PfParams p, const __grid_constant__ CUtensorMap tm_qn, const __grid_constant__ CUtensorMap tm_qp,
                      const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int half = blockIdx.y;  // which 256 output columns
  unsigned char* smem_al = smem_raw;
  if (ako::smem_u32(smem_raw) & 1023u) {  // the swizzled operand tiles need this; nothing is started yet
    if (tid == 0) atomicCAS(&g_pf_sticky, 0, 13);
    return;
  }
  const uint32_t st_base = ako::smem_u32(smem_al);
  const uint32_t v_base = st_base + NST * ST_BYTES;
  float* alpha_s = reinterpret_cast<float*>(smem_al + NST * ST_BYTES + V_BYTES);  // [4][128]
  float* fin_l = alpha_s + 4 * BM;                                                // [128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(fin_l + BM);
  uint64_t* st_full = bars;
  uint64_t* st_empty = bars + NST;
  uint64_t* s_full = bars + 2 * NST;
  uint64_t* s_empty = bars + 2 * NST + 2;
  uint64_t& p_full = bars[2 * NST + 4];
  uint64_t& v_full = bars[2 * NST + 5];
  uint64_t& v_empty = bars[2 * NST + 6];
  uint64_t& pv_full = bars[2 * NST + 7];
  uint64_t& pv_empty = bars[2 * NST + 8];
  uint64_t& fin = bars[2 * NST + 9];
  uint32_t& s_tmem = *reinterpret_cast<uint32_t*>(bars + 2 * NST + 10);
  int* s_work = reinterpret_cast<int*>(bars + 2 * NST + 11);  // sequence, tile inside the sequence (or -1)

  if (tid == 0) {
    // reversed: within a sequence the later query tiles see more keys, so the long CTAs start
    // first and the short ones fill the end of the grid
    int t = (int)(gridDim.x - 1 - blockIdx.x), b = 0;
    for (; b < p.batch; ++b) {
      const int nt = (p.qo_indptr[b + 1] - p.qo_indptr[b] + QT - 1) / QT;
      if (t < nt) break;
      t -= nt;
    }
    s_work[0] = b;
    s_work[1] = (b < p.batch) ? t : -1;
    for (int s = 0; s < NST; ++s) {
      ako::tc::mbar_init(ako::smem_u32(&st_full[s]), 1);
      ako::tc::mbar_init(ako::smem_u32(&st_empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      ako::tc::mbar_init(ako::smem_u32(&s_full[s]), 1);
      ako::tc::mbar_init(ako::smem_u32(&s_empty[s]), 1);
    }
    ako::tc::mbar_init(ako::smem_u32(&p_full), 4);
    ako::tc::mbar_init(ako::smem_u32(&v_full), 1);
    ako::tc::mbar_init(ako::smem_u32(&v_empty), 1);
    ako::tc::mbar_init(ako::smem_u32(&pv_full), 1);
    ako::tc::mbar_init(ako::smem_u32(&pv_empty), 8);
    ako::tc::mbar_init(ako::smem_u32(&fin), 4);
    ako::tc::mbar_init_fence();
  }
  if (warp == 13) ako::tc::tmem_alloc(ako::smem_u32(&s_tmem), 512);
  ako::tc::fence_before_thread_sync();
  __syncthreads();
  ako::tc::fence_after_thread_sync();
  const uint32_t tmem = s_tmem;

  const int b = s_work[0], tile = s_work[1];
  // geometry of this tile (every thread computes the same values)
  int q0 = 0, nq = 0, kv_len = 0, q_len = 0, ntk = 0;
  int64_t kbase = 0, vbase = 0;
  if (tile >= 0) {
    const int qb = p.qo_indptr[b];
    q_len = p.qo_indptr[b + 1] - qb;
    q0 = qb + tile * QT;
    nq = min(QT, q_len - tile * QT);
    kbase = (int64_t)p.kv_indptr[b] * p.page_size;
    kv_len = (p.kv_indptr[b + 1] - p.kv_indptr[b]) * p.page_size;
    vbase = vt_start(kbase, b);
    // keys visible to the tile's last token: [0, kv_len - q_len + last + 1)
    const int kv_end = max(0, min(kv_len, kv_len - q_len + tile * QT + nq));
    ntk = (kv_end + BK - 1) / BK;
  }

  if (warp < 8) {
    // ================================ O accumulation ============================================
    ako::tc::reg_inc<REGS_O>();
    const int r = 32 * (warp & 3) + lane;
    const int ch = warp >> 2;  // which 128 of this CTA's 256 columns
    const uint32_t taddr = tmem + ((uint32_t)(32 * (warp & 3)) << 16) + 256 + ch * 128;
    float o[128];
#pragma unroll
    for (int i = 0; i < 128; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < ntk; ++j) {
      if (!ako::tc::mbar_wait(ako::smem_u32(&pv_full), (uint32_t)(j & 1), &g_pf_status, 1)) { ok = false; break; }
      ako::tc::fence_after_thread_sync();
      const float a = alpha_s[(j & 3) * BM + r];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float v[32];
        ako::tc::tmem_ld32(taddr + 32 * c, v);
        ako::tc::tmem_ld_wait_regs(v);
        if (c == 3) {  // PV buffer and alpha slot are free again
          ako::tc::fence_before_thread_sync();
          __syncwarp();
          if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&pv_empty));
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) o[32 * c + i] = fmaf(o[32 * c + i], a, v[i]);
      }
    }
    if (ok && tile >= 0 && ako::tc::mbar_wait(ako::smem_u32(&fin), 0u, &g_pf_status, 2)) {
      const int qtok = r >> 4;
      if (qtok < nq) {
        const float l = fin_l[r];
        const float inv = (l > 0.f) ? 1.0f / l : 0.f;
        __nv_bfloat16* dst = p.o + ((int64_t)(q0 + qtok) * H + (r & 15)) * DC + half * 256 + ch * 128;
#pragma unroll
        for (int i = 0; i < 128; i += 8) {
          uint4 w;
          w.x = ako::pack_bf16x2(o[i] * inv, o[i + 1] * inv);
          w.y = ako::pack_bf16x2(o[i + 2] * inv, o[i + 3] * inv);
          w.z = ako::pack_bf16x2(o[i + 4] * inv, o[i + 5] * inv);
          w.w = ako::pack_bf16x2(o[i + 6] * inv, o[i + 7] * inv);
          *reinterpret_cast<uint4*>(dst + i) = w;
        }
      }
    }
  } else if (warp < 12) {
    // ================================ softmax ====================================================
    ako::tc::reg_dec<REGS_SOFTMAX>();
    const int r = 32 * (warp & 3) + lane;
    const int qtok = r >> 4;
    const bool row_ok = tile >= 0 && qtok < nq;
    const int kv_lim = row_ok ? max(0, min(kv_len, kv_len - q_len + tile * QT + qtok + 1)) : 0;
    const uint32_t tq = tmem + ((uint32_t)(32 * (warp & 3)) << 16);
    float m = NEG, l = 0.f;
    bool ok = true;
    for (int j = 0; j < ntk; ++j) {
      const int buf = j & 1;
      if (!ako::tc::mbar_wait(ako::smem_u32(&s_full[buf]), (uint32_t)((j >> 1) & 1), &g_pf_status, 3)) { ok = false; break; }
      ako::tc::fence_after_thread_sync();
      const uint32_t ts = tq + buf * BK;
      const int nvis = kv_lim - j * BK;  // visible keys of this tile for this row (may be <= 0 or > 128)
      // no masked key for any row of this warp in this tile; warp-uniform, because the aligned TMEM
      // loads and stores below must be reached by the whole warp together
      const bool fast = __all_sync(0xffffffffu, nvis >= BK) && p.scale_log2 > 0.f;
      float tmax = NEG;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float v[32];
        ako::tc::tmem_ld32(ts + 32 * c, v);
        ako::tc::tmem_ld_wait_regs(v);
        if (fast) {  // four independent chains, the (positive) scale applied once
          float t0 = v[0], t1 = v[1], t2 = v[2], t3 = v[3];
#pragma unroll
          for (int i = 4; i < 32; i += 4) {
            t0 = fmaxf(t0, v[i]);
            t1 = fmaxf(t1, v[i + 1]);
            t2 = fmaxf(t2, v[i + 2]);
            t3 = fmaxf(t3, v[i + 3]);
          }
          tmax = fmaxf(tmax, fmaxf(fmaxf(t0, t1), fmaxf(t2, t3)) * p.scale_log2);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) tmax = fmaxf(tmax, (32 * c + i < nvis) ? v[i] * p.scale_log2 : NEG);
        }
      }
      const float m_new = fmaxf(m, tmax);
      const float alpha = ako::fast_exp2(m - m_new);
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float v[32];
        ako::tc::tmem_ld32(ts + 32 * c, v);
        ako::tc::tmem_ld_wait_regs(v);
        // P overwrites the S buffer it came from, as bf16 pairs: the 32 columns just read become
        // columns [16c, 16c+16), all of them read already; the PV MMAs take P from there (A operand
        // in TMEM), so P never crosses shared memory
        uint32_t w[16];
        if (fast) {
          float s0 = 0.f, s1 = 0.f;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float e0 = ako::fast_exp2(v[i] * p.scale_log2 - m_new);
            const float e1 = ako::fast_exp2(v[i + 1] * p.scale_log2 - m_new);
            s0 += e0;
            s1 += e1;
            w[i >> 1] = ako::pack_bf16x2(e0, e1);
          }
          sum += s0 + s1;
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float e0 = (32 * c + i < nvis) ? ako::fast_exp2(v[i] * p.scale_log2 - m_new) : 0.f;
            const float e1 = (32 * c + i + 1 < nvis) ? ako::fast_exp2(v[i + 1] * p.scale_log2 - m_new) : 0.f;
            sum += e0 + e1;
            w[i >> 1] = ako::pack_bf16x2(e0, e1);
          }
        }
        ako::tc::tmem_st16(ts + 16 * c, w);
      }
      ako::tc::tmem_st_wait();
      l = l * alpha + sum;
      m = m_new;
      alpha_s[(j & 3) * BM + r] = alpha;
      ako::tc::fence_before_thread_sync();
      // Nothing else holds a fast warp back (tiles without masked keys take the short path, a warp
      // with masked rows does not), so it may finish tile j before a slow warp has finished tile
      // j-1; its arrival would then complete the phase of tile j-1 in the slow warp's place. Wait
      // until all four warps have arrived for tile j-1 before arriving for tile j.
      if (j > 0 && !ako::tc::mbar_wait(ako::smem_u32(&p_full), (uint32_t)((j - 1) & 1), &g_pf_status, 4)) { ok = false; break; }
      __syncwarp();
      if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&p_full));
    }
    if (ok && tile >= 0) {
      fin_l[r] = (kv_lim > 0) ? l : 0.f;
      if (half == 0 && row_ok)
        p.lse[(int64_t)(q0 + qtok) * H + (r & 15)] = (kv_lim > 0 && l > 0.f) ? m + log2f(l) : -INFINITY;
      __syncwarp();
      if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&fin));
    }
  } else {
    ako::tc::reg_dec<REGS_OTHER>();
    if (warp == 12 && lane == 0 && ntk > 0) {
      // ================================ Q / K producer =========================================
      ako::tc::tma_prefetch_desc(&tm_qn);
      ako::tc::tma_prefetch_desc(&tm_qp);
      ako::tc::tma_prefetch_desc(&tm_k);
      int g = 0;
      for (int j = 0; j < ntk; ++j) {
        bool ok = true;
        for (int c = 0; c < NCH; ++c, ++g) {
          const int stage = g % NST;
          if (!ako::tc::mbar_wait(ako::smem_u32(&st_empty[stage]), (uint32_t)(((g / NST) & 1) ^ 1), &g_pf_status, 5)) { ok = false; break; }
          const uint32_t bar = ako::smem_u32(&st_full[stage]);
          const uint32_t dst = st_base + stage * ST_BYTES;
          ako::tc::mbar_arrive_expect_tx(bar, ST_BYTES);
          if (c < DC / 64) ako::tc::tma_load_2d(dst, &tm_qn, c * 64, q0 * H, bar);
          else ako::tc::tma_load_2d(dst, &tm_qp, 0, q0 * H, bar);
          ako::tc::tma_load_2d(dst + CH_BYTES, &tm_k, c * 64, (int)(kbase + (int64_t)j * BK), bar);
        }
        if (!ok) break;
      }
    } else if (warp == 14 && lane == 0 && ntk > 0) {
      // ================================ V producer ==============================================
      ako::tc::tma_prefetch_desc(&tm_v);
      for (int j = 0; j < ntk; ++j) {
        if (!ako::tc::mbar_wait(ako::smem_u32(&v_empty), (uint32_t)((j & 1) ^ 1), &g_pf_status, 6)) break;
        const uint32_t bar = ako::smem_u32(&v_full);
        ako::tc::mbar_arrive_expect_tx(bar, V_BYTES);
        const int x = (int)(vbase + (int64_t)j * BK);
        ako::tc::tma_load_2d(v_base, &tm_v, x, half * 256, bar);
        ako::tc::tma_load_2d(v_base + V_BYTES / 2, &tm_v, x + 64, half * 256, bar);
      }
    } else if (warp == 13 && lane == 0 && ntk > 0) {
      // ================================ S issuer ================================================
      constexpr uint32_t IDESC_S = ako::tc::idesc_bf16_f32(BM, BK);
      const uint32_t st_lo0 = ako::tc::smem_desc_lo(st_base);
      int g = 0;
      for (int j = 0; j < ntk; ++j) {
        const int buf = j & 1;
        // the PV MMAs of tile j-2 have read P out of this buffer
        if (!ako::tc::mbar_wait(ako::smem_u32(&s_empty[buf]), (uint32_t)(((j >> 1) & 1) ^ 1), &g_pf_status, 7)) break;
        const uint32_t d = tmem + buf * BK;
        bool ok = true;
        for (int c = 0; c < NCH; ++c, ++g) {
          const int stage = g % NST;
          if (!ako::tc::mbar_wait(ako::smem_u32(&st_full[stage]), (uint32_t)((g / NST) & 1), &g_pf_status, 8)) { ok = false; break; }
          ako::tc::fence_after_thread_sync();
          const uint32_t a_lo = st_lo0 + stage * (ST_BYTES >> 4);
          const uint32_t b_lo = a_lo + (CH_BYTES >> 4);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            ako::tc::mma_bf16_lohi(d, a_lo + 2 * ks, b_lo + 2 * ks, IDESC_S, (c > 0 || ks > 0) ? 1u : 0u);
          ako::tc::mma_commit(ako::smem_u32(&st_empty[stage]));
        }
        if (!ok) break;
        ako::tc::mma_commit(ako::smem_u32(&s_full[buf]));
      }
    } else if (warp == 15 && lane == 0 && ntk > 0) {
      // ================================ PV issuer ===============================================
      // a thread of its own: PV of tile j goes to the tensor pipe the moment P is written, while
      // the S issuer is still waiting on the operand stream of a later tile
      constexpr uint32_t IDESC_PV = ako::tc::idesc_bf16_f32(BM, 256);
      const uint32_t v_lo0 = ako::tc::smem_desc_lo(v_base);
      for (int j = 0; j < ntk; ++j) {
        if (!ako::tc::mbar_wait(ako::smem_u32(&p_full), (uint32_t)(j & 1), &g_pf_status, 9)) break;
        if (!ako::tc::mbar_wait(ako::smem_u32(&v_full), (uint32_t)(j & 1), &g_pf_status, 10)) break;
        if (!ako::tc::mbar_wait(ako::smem_u32(&pv_empty), (uint32_t)((j & 1) ^ 1), &g_pf_status, 11)) break;
        ako::tc::fence_after_thread_sync();
        const uint32_t d = tmem + 256;
#pragma unroll
        for (int at = 0; at < 2; ++at)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            ako::tc::mma_bf16_tmem_a(d, tmem + (j & 1) * BK + 8 * (4 * at + ks), v_lo0 + at * ((V_BYTES / 2) >> 4) + 2 * ks,
                                     IDESC_PV, (at > 0 || ks > 0) ? 1u : 0u);
        ako::tc::mma_commit(ako::smem_u32(&pv_full));
        ako::tc::mma_commit(ako::smem_u32(&v_empty));
        ako::tc::mma_commit(ako::smem_u32(&s_empty[j & 1]));  // P (inside the S buffer) has been read
      }
    }
  }

  ako::tc::fence_before_thread_sync();
  __syncthreads();
  if (tid == 0) {
    const int code = *reinterpret_cast<volatile int*>(&g_pf_status);
    if (code != 0) atomicCAS(&g_pf_sticky, 0, code);
  }
  if (warp == 13) {
    ako::tc::fence_after_thread_sync();
    ako::tc::tmem_dealloc(tmem, 512);
  }
}

int64_t vt_columns(int64_t ntok, int64_t batch) { return ((ntok + 8 * batch + 8 + 7) / 8) * 8; }

}  // namespace

size_t ako_mla_prefill_tc_workspace_bytes(int64_t batch, int64_t num_kv_indices, int64_t page_size) {
  const int64_t ntok = num_kv_indices * page_size;
  if (ntok <= 0 || batch <= 0) return 0;
  const size_t kc = ((size_t)ntok * DQK * 2 + 255) / 256 * 256;
  const size_t vt = (size_t)DC * vt_columns(ntok, batch) * 2;
  return kc + vt;
}

int ako_mla_prefill_tc_launch(const void* q_nope, const void* q_pe, const void* ckv_cache, const void* kpe_cache,
                              const int32_t* qo_indptr, const int32_t* kv_indptr, const int32_t* kv_indices,
                              float sm_scale, void* o, float* lse, int64_t total_q, int64_t batch,
                              int64_t num_kv_indices, int64_t page_size, void* workspace, size_t workspace_bytes,
                              cudaStream_t st) {
  const int64_t ntok = num_kv_indices * page_size;
  if (ntok <= 0 || ntok > 0x7fffffffLL || total_q * H > 0x7fffffffLL) return AKO4X_EUNSUPPORTED_SHAPE;
  const size_t need = ako_mla_prefill_tc_workspace_bytes(batch, num_kv_indices, page_size);
  if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255)) return AKO4X_EWORKSPACE;
  const int64_t W = vt_columns(ntok, batch);
  unsigned char* kc = (unsigned char*)workspace;
  unsigned char* vt = kc + ((size_t)ntok * DQK * 2 + 255) / 256 * 256;
  // the gaps between sequences in Vt are multiplied by P = 0: they must hold finite values
  if (cudaMemsetAsync(vt, 0, (size_t)DC * W * 2, st) != cudaSuccess) return AKO4X_ELAUNCH;
  mla_prefill_gather_kernel<<<(unsigned)ako::cdiv(ntok, G_TOK), 256, 0, st>>>(
      (const uint4*)ckv_cache, (const uint4*)kpe_cache, kv_indices, kv_indptr, (int)batch, (int)page_size, ntok,
      (uint4*)kc, (__nv_bfloat16*)vt, W);
  AKO_CHECK_LAUNCH();

  CUtensorMap tm_qn, tm_qp, tm_k, tm_v;
  if (!ako::tma::bf16_matrix_map(&tm_qn, q_nope, (uint64_t)total_q * H, DC, DC * 2, BM) ||
      !ako::tma::bf16_matrix_map(&tm_qp, q_pe, (uint64_t)total_q * H, DP, DP * 2, BM) ||
      !ako::tma::bf16_matrix_map(&tm_k, kc, (uint64_t)ntok, DQK, DQK * 2, BK) ||
      !ako::tma::bf16_matrix_map(&tm_v, vt, DC, (uint64_t)W, (uint64_t)W * 2, 256))
    return AKO4X_ELAUNCH;
  if (!ako::ensure_dynamic_smem<mla_prefill_tc_kernel>(SMEM)) return AKO4X_ELAUNCH;
  PfParams p;
  p.qo_indptr = qo_indptr;
  p.kv_indptr = kv_indptr;
  p.o = (__nv_bfloat16*)o;
  p.lse = lse;
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  p.batch = (int)batch;
  p.page_size = (int)page_size;
  const dim3 grid((unsigned)(ako::cdiv(total_q, QT) + batch), 2);
  mla_prefill_tc_kernel<<<grid, THREADS, SMEM, st>>>(p, tm_qn, tm_qp, tm_k, tm_v);
  AKO_CHECK_LAUNCH();
  return AKO4X_OK;
}

int ako_mla_prefill_tc_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_pf_sticky, sizeof(int)) != cudaSuccess) return AKO4X_ELAUNCH;
  return v;
}
