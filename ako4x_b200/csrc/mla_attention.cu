// MLA attention core shared by paged MLA decode, DSA sparse attention and causal MLA prefill:
// 16 heads, ckv dim 512 (keys and values), kpe dim 64, bf16, fp32 accumulation.
//
// A "row" is one query token (16 heads = one m16 tile of mma.sync). Its keys are a list of cache
// rows: the paged KV list of its sequence (decode), its sparse index list with -1 holes (DSA), or
// the causally visible prefix of its sequence's KV list (prefill). One CTA of 8 warps owns
// (row, KV split) and streams 64-token tiles through a 2-stage ring. A token is gathered with TWO
// bulk copies (cp.async.bulk: 1024 B of ckv, 128 B of kpe; completion counted in bytes on the
// stage's mbarrier) issued by the 64 lanes of warps 0-1, one token per lane; the lane loads its
// gather index one tile earlier and nothing depends on that load until the copy is issued.
// Rows sit in shared memory with 1040 / 144-byte pitches, which keeps ldmatrix bank-conflict free
// without a swizzle.
//   S phase : warp w computes logits of tokens 16*(w&3).. over one half of the 576-wide
//             reduction (w>>2) with its Q fragments held in registers; halves meet in shared memory.
//   PV phase: every warp rebuilds P (softmax is recomputed per warp, which removes two barriers)
//             and accumulates its own 64 of the 512 output columns.
// Each token costs 1152 bytes of HBM traffic and 34816 flop, so the kernel is gather-bandwidth
// bound; shared-memory traffic per token (about 4.4 KB) is the second limit. Waits on the
// mbarriers are bounded: a wait that exceeds its cycle limit records a code in a device status word
// and the CTA stops consuming.
#include "lse_merge.cuh"
#include "mla_prefill_tc.h"
#include "tcgen05.cuh"

namespace {

constexpr int H = 16, DC = 512, DP = 64;
constexpr int TILE = 64;
constexpr int THREADS = 256;
constexpr int CKV_ROW = DC * 2;                 // 1024 bytes
constexpr int KPE_ROW = DP * 2;                 // 128 bytes
constexpr int CKV_PITCH = CKV_ROW + 16;
constexpr int KPE_PITCH = KPE_ROW + 16;
constexpr int CKV_TILE_BYTES = TILE * CKV_PITCH;
constexpr int KPE_TILE_BYTES = TILE * KPE_PITCH;
constexpr int STAGE_BYTES = CKV_TILE_BYTES + KPE_TILE_BYTES;  // 75776
constexpr int STAGES = 2;
constexpr int SROW = 72;  // padded fp32 row stride of the logit exchange buffer
constexpr int SBUF_FLOATS = 2 * H * SROW;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + SBUF_FLOATS * 4;
constexpr int MAX_SPLITS = 64;

__device__ int g_mla_status = 0;  // 0 = ok; set when a bounded wait gave up

enum Mode { kDecode = 0, kSparse = 1, kPrefill = 2 };
constexpr int64_t kPrefillTcMinQueries = 48;

struct Params {
  const __nv_bfloat16* q_nope;
  const __nv_bfloat16* q_pe;
  const unsigned char* ckv;
  const unsigned char* kpe;
  const int32_t* qo_indptr;   // prefill only
  const int32_t* kv_indptr;   // decode / prefill
  const int32_t* indices;     // kv_indices or sparse_indices
  __nv_bfloat16* o;
  float* lse;
  float* part_acc;            // [rows*16][splits][512]
  float* part_ml;             // [rows*16][splits][2]
  float scale_log2;
  int page_size;
  int num_splits;
  int topk;                   // sparse only
  int batch;                  // prefill only (number of sequences)
};

struct RowDesc {
  const int32_t* idx;  // index list of the row
  int count;           // number of key positions (holes included)
};

template <int MODE>
__device__ __forceinline__ RowDesc describe_row(const Params& p, int64_t row) {
  RowDesc d;
  if (MODE == kDecode) {
    const int s = p.kv_indptr[row], e = p.kv_indptr[row + 1];
    d.idx = p.indices + s;
    d.count = max(0, e - s) * p.page_size;
  } else if (MODE == kSparse) {
    d.idx = p.indices + row * p.topk;
    d.count = p.topk;
  } else {
    // binary search: largest b with qo_indptr[b] <= row
    int lo = 0, hi = p.batch;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (p.qo_indptr[mid] <= row) lo = mid; else hi = mid;
    }
    const int qs = p.qo_indptr[lo], qe = p.qo_indptr[lo + 1];
    const int ks = p.kv_indptr[lo], ke = p.kv_indptr[lo + 1];
    const int kv_len = max(0, ke - ks) * p.page_size;
    const int q_len = qe - qs;
    const int visible = (kv_len - q_len) + (int)(row - qs) + 1;
    d.idx = p.indices + ks;
    d.count = min(kv_len, max(0, visible));
  }
  return d;
}

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1) mla_attention_kernel(Params p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t s_full[STAGES];
  __shared__ uint32_t s_valid[STAGES][2];  // per stage: which of the 64 tokens were copied
  __shared__ int s_err;  // code of a wait of this CTA that gave up (0 = none), published on exit
  float* sbuf = reinterpret_cast<float*>(smem_raw + STAGES * STAGE_BYTES);
  const uint32_t smem_base = ako::smem_u32(smem_raw);

  const int split = blockIdx.x % p.num_splits;
  const int64_t row = blockIdx.x / p.num_splits;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int pw = warp & 3;   // token group of the S phase
  const int kh = warp >> 2;  // reduction half of the S phase

  ako::pdl_trigger();
  const RowDesc rd = describe_row<MODE>(p, row);
  int chunk = (int)ako::round_up(ako::cdiv(rd.count, p.num_splits), TILE);
  if (chunk < TILE) chunk = TILE;
  const int tok_begin = min(rd.count, split * chunk);
  const int tok_end = min(rd.count, tok_begin + chunk);
  const int ntiles = (tok_end - tok_begin + TILE - 1) / TILE;

  // Shared memory starts finite: rows of holes / tokens past the end are never copied, and
  // 0 * stale must not be NaN in the PV product.
  for (int i = threadIdx.x; i < STAGES * STAGE_BYTES / 16; i += THREADS)
    reinterpret_cast<uint4*>(smem_raw)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    // arrivals per phase: warps 0 and 1 (bulk copies, with byte counts) + one deferred arrival per
    // thread that fires when its kpe cp.async copies have landed
    for (int s = 0; s < STAGES; ++s) ako::tc::mbar_init(ako::smem_u32(&s_full[s]), 2 + THREADS);
    ako::tc::mbar_init_fence();
    s_err = 0;
  }
  ako::tc::fence_proxy_async_smem();
  __syncthreads();

  // ---- producer state (warps 0-1: lane = one token of a tile) -----------------------------------
  const int my_tok = warp * 32 + lane;  // meaningful for warps 0, 1
  int32_t entry_next = 0;               // raw index entry for the next tile to be issued
  // kpe rows (128 B) go through 16-byte cp.async instead: a bulk copy costs the copy engine the
  // same whatever its size, and one per token (the 1 KB ckv row) is what it sustains. Thread t
  // copies chunk t&7 of tokens t>>3 and (t>>3)+32 of the tile.
  int32_t kentry_next[2] = {0, 0};
  auto fetch_entry = [&](int tile) {
    if (rd.count <= 0) return;
    const int last = max(tok_end - 1, 0);
    if (warp < 2) {
      const int pos = min(tok_begin + tile * TILE + my_tok, last);
      entry_next = __ldg(rd.idx + (p.page_size == 1 ? pos : pos / p.page_size));
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int pos = min(tok_begin + tile * TILE + (int)(threadIdx.x >> 3) + 32 * j, last);
      kentry_next[j] = __ldg(rd.idx + (p.page_size == 1 ? pos : pos / p.page_size));
    }
  };
  auto issue_kpe = [&](int tile) {  // every thread; uses kentry_next fetched for `tile`
    const int stage = tile % STAGES;
    const int c = threadIdx.x & 7;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int tk = (int)(threadIdx.x >> 3) + 32 * j;
      const int pos = tok_begin + tile * TILE + tk;
      const bool valid = pos < tok_end && kentry_next[j] >= 0;
      const int64_t crow = !valid ? 0
                           : (p.page_size == 1) ? (int64_t)kentry_next[j]
                                                : (int64_t)kentry_next[j] * p.page_size + pos % p.page_size;
      ako::cp_async16(smem_base + stage * STAGE_BYTES + CKV_TILE_BYTES + tk * KPE_PITCH + c * 16,
                      p.kpe + crow * KPE_ROW + c * 16, valid);
    }
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(ako::smem_u32(&s_full[stage]))
                 : "memory");
  };
  auto issue_tile = [&](int tile) {  // uses entry_next fetched for `tile`
    const int stage = tile % STAGES;
    const uint32_t bar = ako::smem_u32(&s_full[stage]);
    const int pos = tok_begin + tile * TILE + my_tok;
    const bool valid = pos < tok_end && entry_next >= 0;
    const int64_t crow = (p.page_size == 1) ? (int64_t)entry_next
                                            : (int64_t)entry_next * p.page_size + pos % p.page_size;
    const unsigned m = __ballot_sync(0xffffffffu, valid);
    if (lane == 0) {
      s_valid[stage][warp] = m;
      ako::tc::mbar_arrive_expect_tx(bar, (uint32_t)__popc(m) * CKV_ROW);
    }
    __syncwarp();
    if (valid) {
      const uint32_t dst = smem_base + stage * STAGE_BYTES;
      ako::tc::bulk_load_1d(dst + my_tok * CKV_PITCH, p.ckv + crow * CKV_ROW, CKV_ROW, bar);
    }
  };
  if (ntiles > 0) {
    fetch_entry(0);
    if (warp < 2) issue_tile(0);
    issue_kpe(0);
  }
  fetch_entry(1);

  // Q fragments of this warp's reduction half: 18 k-steps of 16.
  uint32_t qa[18][4];
  {
    const __nv_bfloat16* qn0 = p.q_nope + (row * H + g) * DC;
    const __nv_bfloat16* qn1 = qn0 + 8 * DC;
    const __nv_bfloat16* qp0 = p.q_pe + (row * H + g) * DP;
    const __nv_bfloat16* qp1 = qp0 + 8 * DP;
#pragma unroll
    for (int ks = 0; ks < 18; ++ks) {
      const __nv_bfloat16 *r0, *r1;
      int k0;
      if (kh == 0) { r0 = qn0; r1 = qn1; k0 = ks * 16; }
      else if (ks < 14) { r0 = qn0; r1 = qn1; k0 = 288 + ks * 16; }
      else { r0 = qp0; r1 = qp1; k0 = (ks - 14) * 16; }
      qa[ks][0] = *reinterpret_cast<const uint32_t*>(r0 + k0 + 2 * t);
      qa[ks][1] = *reinterpret_cast<const uint32_t*>(r1 + k0 + 2 * t);
      qa[ks][2] = *reinterpret_cast<const uint32_t*>(r0 + k0 + 8 + 2 * t);
      qa[ks][3] = *reinterpret_cast<const uint32_t*>(r1 + k0 + 8 + 2 * t);
    }
  }

  float oacc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  for (int it = 0; it < ntiles; ++it) {
    const int stage = it & 1;
    const bool landed = ako::tc::mbar_wait(ako::smem_u32(&s_full[stage]), (uint32_t)((it >> 1) & 1),
                                           &s_err, 1);
    // every warp has finished tile it-1: its stage (and s_valid entry) is free for tile it+1
    if (!__syncthreads_and(landed)) break;
    if (it + 1 < ntiles) {
      if (warp < 2) {
        ako::tc::fence_proxy_async_smem();  // generic reads of the freed stage before async writes
        issue_tile(it + 1);
      }
      issue_kpe(it + 1);
    }
    fetch_entry(it + 2);
    const uint32_t Cs = smem_base + stage * STAGE_BYTES;
    const uint32_t Ps = Cs + CKV_TILE_BYTES;

    // ---- S phase: 16 tokens x half of the reduction --------------------------------------
    {
      float sacc[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
      const int tok = 16 * pw + ((lane >> 4) << 3) + (lane & 7);
      const int csel = (lane >> 3) & 1;
#pragma unroll
      for (int ks = 0; ks < 18; ++ks) {
        uint32_t b00, b01, b10, b11;
        uint32_t addr;
        if (kh == 0 || ks < 14) {
          const int c = (kh == 0 ? 0 : 36) + 2 * ks + csel;  // 16-byte chunk of the 512-wide row
          addr = Cs + tok * CKV_PITCH + (c << 4);
        } else {
          const int c = 2 * (ks - 14) + csel;
          addr = Ps + tok * KPE_PITCH + (c << 4);
        }
        ako::ldmatrix_x4(b00, b01, b10, b11, addr);
        ako::mma_bf16_16816(sacc[0], qa[ks], b00, b01);
        ako::mma_bf16_16816(sacc[1], qa[ks], b10, b11);
      }
      float* sb = sbuf + kh * H * SROW;
      const uint32_t vmask = s_valid[stage][pw >> 1];  // tokens 32*(pw>>1) ..
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int c0 = 16 * pw + 8 * nt + 2 * t;
        float v0 = sacc[nt][0], v1 = sacc[nt][1], v2 = sacc[nt][2], v3 = sacc[nt][3];
        if (kh == 0) {  // the first half carries the validity mask
          const bool ok0 = (vmask >> (c0 & 31)) & 1u;
          const bool ok1 = (vmask >> ((c0 + 1) & 31)) & 1u;
          if (!ok0) { v0 = -INFINITY; v2 = -INFINITY; }
          if (!ok1) { v1 = -INFINITY; v3 = -INFINITY; }
        }
        *reinterpret_cast<float2*>(sb + g * SROW + c0) = make_float2(v0, v1);
        *reinterpret_cast<float2*>(sb + (g + 8) * SROW + c0) = make_float2(v2, v3);
      }
    }
    __syncthreads();

    // ---- softmax (per warp, rows g and g+8 over the 64 tokens) ----------------------------
    float sv[2][16];
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float* s0 = sbuf + (g + 8 * r) * SROW + 2 * t;
      const float* s1 = s0 + H * SROW;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 a = *reinterpret_cast<const float2*>(s0 + 8 * i);
        const float2 b = *reinterpret_cast<const float2*>(s1 + 8 * i);
        const float x0 = (a.x + b.x) * p.scale_log2, x1 = (a.y + b.y) * p.scale_log2;
        sv[r][2 * i] = x0;
        sv[r][2 * i + 1] = x1;
        mx[r] = fmaxf(mx[r], fmaxf(x0, x1));
      }
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    uint32_t pa[4][4];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float m_new = fmaxf(m_run[r], mx[r]);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = ako::fast_exp2(m_run[r] - m_use);
      float psum = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float p0 = ako::fast_exp2(sv[r][2 * i] - m_use);
        const float p1 = ako::fast_exp2(sv[r][2 * i + 1] - m_use);
        psum += p0 + p1;
        // tokens 8i+2t, 8i+2t+1 -> k-step i/2, low (i even) or high (i odd) half
        pa[i >> 1][(i & 1) * 2 + r] = ako::pack_bf16x2(p0, p1);
      }
      psum += __shfl_xor_sync(0xffffffffu, psum, 1);
      psum += __shfl_xor_sync(0xffffffffu, psum, 2);
      l_run[r] = l_run[r] * corr + psum;
      m_run[r] = m_new;
#pragma unroll
      for (int nd = 0; nd < 8; ++nd) {
        oacc[nd][2 * r] *= corr;
        oacc[nd][2 * r + 1] *= corr;
      }
    }

    // ---- PV phase: this warp's 64 output columns ---------------------------------------------
    {
      const int trow = (((lane >> 3) & 1) << 3) + (lane & 7);
      const int csel = lane >> 4;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int tok = 16 * j + trow;
#pragma unroll
        for (int nd = 0; nd < 8; nd += 2) {
          uint32_t v00, v01, v10, v11;
          const int c = 8 * warp + nd + csel;
          ako::ldmatrix_x4_trans(v00, v01, v10, v11, Cs + tok * CKV_PITCH + (c << 4));
          ako::mma_bf16_16816(oacc[nd], pa[j], v00, v01);
          ako::mma_bf16_16816(oacc[nd + 1], pa[j], v10, v11);
        }
      }
    }
  }

  // ---- epilogue ---------------------------------------------------------------------------------
  if (threadIdx.x == 0 && s_err != 0) atomicCAS(&g_mla_status, 0, s_err);
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int64_t rh = row * H + g + 8 * r;
    if (p.num_splits == 1) {
      const float inv = (l_run[r] > 0.f) ? 1.f / l_run[r] : 0.f;
      __nv_bfloat16* op = p.o + rh * DC + 64 * warp + 2 * t;
#pragma unroll
      for (int nd = 0; nd < 8; ++nd)
        *reinterpret_cast<uint32_t*>(op + nd * 8) =
            ako::pack_bf16x2(oacc[nd][2 * r] * inv, oacc[nd][2 * r + 1] * inv);
      if (warp == 0 && t == 0)
        p.lse[rh] = (l_run[r] > 0.f) ? m_run[r] + log2f(l_run[r]) : -INFINITY;
    } else {
      float* pa_out = p.part_acc + (rh * p.num_splits + split) * DC + 64 * warp + 2 * t;
#pragma unroll
      for (int nd = 0; nd < 8; ++nd)
        *reinterpret_cast<float2*>(pa_out + nd * 8) = make_float2(oacc[nd][2 * r], oacc[nd][2 * r + 1]);
      if (warp == 0 && t == 0) {
        float* ml = p.part_ml + (rh * p.num_splits + split) * 2;
        ml[0] = m_run[r];
        ml[1] = l_run[r];
      }
    }
  }
}

// The tensor-core form of the decode / sparse kernels (128-token tiles, tcgen05 + TMEM).
#include "mla_gather_tc.cuh"

// Calls with fewer 128-token tiles than this keep the 64-token mma.sync kernel: its CTAs are half
// the size, so a call that cannot fill the GPU twice spreads over more SMs and has a shorter tail.
constexpr int64_t kTcMinTiles = 296;

// `ragged`: rows have their own lengths (decode), which needs the per-row tile table in shared memory.
bool use_tc(int64_t rows, int64_t avg_keys, bool ragged) {
  if (ragged && rows > tcg::MAX_ROWS) return false;
  return rows <= 0x7fffffffLL / 4096 && rows * ako::cdiv(avg_keys > 0 ? avg_keys : 1, tcg::TOK) >= kTcMinTiles;
}

// Workspace of the tensor-core path: the tile prefix table (rows + 1 ints, padded), then one partial
// slot per (row + CTA) sum: fp32 O [16][512] and (m, l) [16][2].
struct TcWorkspace {
  int* pref;
  float* part_acc;
  float* part_ml;
  size_t total;
};
TcWorkspace tc_carve(void* base, int64_t rows, int ctas) {
  const size_t slots = (size_t)rows + (size_t)ctas;
  const size_t pref_bytes = (((size_t)rows + 1) * sizeof(int) + 255) & ~(size_t)255;
  TcWorkspace w;
  w.pref = (int*)base;
  w.part_acc = (float*)((unsigned char*)base + pref_bytes);
  w.part_ml = w.part_acc + slots * H * DC;
  w.total = pref_bytes + slots * H * (DC + 2) * sizeof(float);
  return w;
}

template <int MODE>
int launch_tc(Params& p, int64_t rows, void* workspace, cudaStream_t st) {
  const int ctas = ako::sm_count();
  const TcWorkspace w = tc_carve(workspace, rows, ctas);
  p.part_acc = w.part_acc;
  p.part_ml = w.part_ml;
  p.num_splits = 0;
  if (!ako::ensure_dynamic_smem<tcg::mla_gather_tc_kernel<MODE>>(tcg::SMEM)) return AKO4X_ELAUNCH;
  tcg::mla_gather_tc_kernel<MODE><<<ctas, tcg::THREADS, tcg::SMEM, st>>>(p, (int)rows, w.pref);
  AKO_CHECK_LAUNCH();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(rows * H));
  cfg.blockDim = dim3(DC / 4);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const float* pacc = w.part_acc;
  const float* pml = w.part_ml;
  const int* pref = w.pref;
  int nrows = (int)rows, tpr = (MODE == kSparse) ? (p.topk + tcg::TOK - 1) / tcg::TOK : 0, nctas = ctas;
  __nv_bfloat16* op = p.o;
  float* lp = p.lse;
  if (cudaLaunchKernelEx(&cfg, tcg::mla_gather_tc_merge_kernel<MODE>, pacc, pml, pref, nrows, tpr, nctas, op, lp) !=
      cudaSuccess)
    return AKO4X_ELAUNCH;
  return AKO4X_OK;
}

int pick_splits(int64_t rows, int64_t avg_keys) {
  if (rows <= 0) return 1;
  int64_t want = ako::cdiv(592, rows);       // ~4 waves of 148 single-CTA SMs
  int64_t cap = avg_keys / 128;               // at least two tiles per CTA on average
  if (cap < 1) cap = 1;
  // Few rows leave SMs idle at that grain and the call's latency is the chunk length: one tile per CTA,
  // up to one wave of CTAs.
  if (rows * cap < 148) {
    const int64_t fine = avg_keys / TILE > 1 ? avg_keys / TILE : 1;
    const int64_t one_wave = 148 / rows > 1 ? 148 / rows : 1;
    cap = fine < one_wave ? fine : one_wave;
  }
  int64_t s = want < cap ? want : cap;
  if (s < 1) s = 1;
  if (s > MAX_SPLITS) s = MAX_SPLITS;
  // Around that value, prefer the split count whose grid fills its last wave of CTAs (one per SM) best.
  int64_t best = s;
  double best_eff = 0.0;
  for (int64_t c = (s + 1) / 2; c <= 2 * s && c <= cap && c <= MAX_SPLITS; ++c) {
    const int64_t n = rows * c;
    const double eff = (double)n / (double)(ako::cdiv(n, 148) * 148);
    if (eff > best_eff + 0.02 || (eff > best_eff - 0.02 && c == s)) { best_eff = eff; best = c; }
  }
  return (int)best;
}

size_t workspace_for(int64_t rows, int splits) {
  if (splits == 1) return 0;
  return (size_t)rows * H * splits * (DC + 2) * sizeof(float);
}

template <int MODE>
int launch(Params& p, int64_t rows, int splits, void* workspace, cudaStream_t st) {
  p.num_splits = splits;
  p.part_acc = (float*)workspace;
  p.part_ml = workspace ? p.part_acc + (size_t)rows * H * splits * DC : nullptr;
  const int64_t grid = rows * splits;
  if (grid > 0x7fffffffLL) return AKO4X_EINVAL;
  if (!ako::ensure_dynamic_smem<mla_attention_kernel<MODE>>(SMEM_BYTES)) return AKO4X_ELAUNCH;
  mla_attention_kernel<MODE><<<(unsigned)grid, THREADS, SMEM_BYTES, st>>>(p);
  AKO_CHECK_LAUNCH();
  if (splits > 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(rows * H));
    cfg.blockDim = dim3(DC / 4);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const float* pacc = p.part_acc;
    const float* pml = p.part_ml;
    __nv_bfloat16* op = p.o;
    float* lp = p.lse;
    int ns = splits;
    if (cudaLaunchKernelEx(&cfg, ako::lse_merge_kernel<DC, 4>, pacc, pml, op, lp, ns) != cudaSuccess)
      return AKO4X_ELAUNCH;
  }
  return AKO4X_OK;
}

bool misaligned(const void* a, const void* b, const void* c, const void* d, const void* e) {
  return (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)d | (uintptr_t)e) & 15) != 0;
}

void fill_common(Params& p, const void* q_nope, const void* q_pe, const void* ckv_cache,
                 const void* kpe_cache, void* o, float* lse, float sm_scale) {
  p.q_nope = (const __nv_bfloat16*)q_nope;
  p.q_pe = (const __nv_bfloat16*)q_pe;
  p.ckv = (const unsigned char*)ckv_cache;
  p.kpe = (const unsigned char*)kpe_cache;
  p.o = (__nv_bfloat16*)o;
  p.lse = lse;
  p.scale_log2 = sm_scale * AKO_LOG2E;
}

}  // namespace

// ---- paged MLA decode ----------------------------------------------------------------------------
extern "C" size_t ako4x_mla_paged_decode_workspace_bytes(int64_t batch, int64_t num_kv_indices,
                                                         int64_t page_size) {
  if (batch <= 0) return 0;
  const int64_t avg = num_kv_indices * page_size / batch;
  if (use_tc(batch, avg, true)) return tc_carve(nullptr, batch, ako::sm_count()).total;
  return workspace_for(batch, pick_splits(batch, avg));
}

extern "C" int ako4x_mla_paged_decode(const void* q_nope, const void* q_pe, const void* ckv_cache,
                                      const void* kpe_cache, const int32_t* kv_indptr,
                                      const int32_t* kv_indices, float sm_scale, void* o, float* lse,
                                      int64_t batch, int64_t num_kv_indices, int64_t page_size,
                                      void* workspace, size_t workspace_bytes, void* stream) {
  if (batch < 0 || num_kv_indices < 0 || page_size < 1) return AKO4X_EINVAL;
  if (batch == 0) return AKO4X_OK;
  if (!q_nope || !q_pe || !ckv_cache || !kpe_cache || !kv_indptr || !o || !lse) return AKO4X_EINVAL;
  if (num_kv_indices > 0 && !kv_indices) return AKO4X_EINVAL;
  if (misaligned(q_nope, q_pe, ckv_cache, kpe_cache, o)) return AKO4X_EINVAL;
  const int64_t avg = num_kv_indices * page_size / batch;
  const bool tc = use_tc(batch, avg, true);
  const int splits = tc ? 0 : pick_splits(batch, avg);
  const size_t need = tc ? tc_carve(nullptr, batch, ako::sm_count()).total : workspace_for(batch, splits);
  if (need > 0 && (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 15))) return AKO4X_EWORKSPACE;
  Params p = {};
  fill_common(p, q_nope, q_pe, ckv_cache, kpe_cache, o, lse, sm_scale);
  p.kv_indptr = kv_indptr;
  p.indices = kv_indices;
  p.page_size = (int)page_size;
  if (tc) return launch_tc<kDecode>(p, batch, workspace, (cudaStream_t)stream);
  return launch<kDecode>(p, batch, splits, workspace, (cudaStream_t)stream);
}

// ---- DSA sparse attention ------------------------------------------------------------------------
extern "C" size_t ako4x_dsa_sparse_attention_workspace_bytes(int64_t tokens, int64_t topk) {
  if (tokens <= 0) return 0;
  if (use_tc(tokens, topk, false)) return tc_carve(nullptr, tokens, ako::sm_count()).total;
  return workspace_for(tokens, pick_splits(tokens, topk));
}

extern "C" int ako4x_dsa_sparse_attention(const void* q_nope, const void* q_pe, const void* ckv_cache,
                                          const void* kpe_cache, const int32_t* sparse_indices,
                                          float sm_scale, void* o, float* lse, int64_t tokens,
                                          int64_t topk, int64_t num_cache_rows, void* workspace,
                                          size_t workspace_bytes, void* stream) {
  (void)num_cache_rows;
  if (tokens < 0 || topk < 0 || topk > 0x7fffffffLL) return AKO4X_EINVAL;
  if (tokens == 0) return AKO4X_OK;
  if (!q_nope || !q_pe || !ckv_cache || !kpe_cache || !o || !lse) return AKO4X_EINVAL;
  if (topk > 0 && !sparse_indices) return AKO4X_EINVAL;
  if (misaligned(q_nope, q_pe, ckv_cache, kpe_cache, o)) return AKO4X_EINVAL;
  const bool tc = use_tc(tokens, topk, false);
  const int splits = tc ? 0 : pick_splits(tokens, topk);
  const size_t need = tc ? tc_carve(nullptr, tokens, ako::sm_count()).total : workspace_for(tokens, splits);
  if (need > 0 && (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 15))) return AKO4X_EWORKSPACE;
  Params p = {};
  fill_common(p, q_nope, q_pe, ckv_cache, kpe_cache, o, lse, sm_scale);
  p.indices = sparse_indices;
  p.page_size = 1;
  p.topk = (int)topk;
  if (tc) return launch_tc<kSparse>(p, tokens, workspace, (cudaStream_t)stream);
  return launch<kSparse>(p, tokens, splits, workspace, (cudaStream_t)stream);
}

// ---- DSA indexer followed by sparse attention, the top-k list staying on the device ---------------
extern "C" size_t ako4x_dsa_indexer_attention_workspace_bytes(int64_t rows, int64_t max_pages) {
  const size_t a = (ako4x_dsa_topk_indexer_workspace_bytes(rows, max_pages) + 255) & ~(size_t)255;
  return a + ako4x_dsa_sparse_attention_workspace_bytes(rows, 2048);
}

extern "C" int ako4x_dsa_indexer_attention(const void* q_index_fp8, const void* k_index_cache,
                                           const float* weights, const int32_t* seq_lens,
                                           const int32_t* block_table, const void* q_nope, const void* q_pe,
                                           const void* ckv_cache, const void* kpe_cache, float sm_scale,
                                           int32_t* topk_indices, void* o, float* lse, int64_t rows,
                                           int64_t max_pages, int64_t num_cache_pages, void* workspace,
                                           size_t workspace_bytes, void* stream) {
  if (rows < 0 || max_pages < 0 || num_cache_pages < 0) return AKO4X_EINVAL;
  if (rows == 0) return AKO4X_OK;
  const size_t a = (ako4x_dsa_topk_indexer_workspace_bytes(rows, max_pages) + 255) & ~(size_t)255;
  const size_t b = ako4x_dsa_sparse_attention_workspace_bytes(rows, 2048);
  if (a + b > 0 && (!workspace || workspace_bytes < a + b || ((uintptr_t)workspace & 255))) return AKO4X_EWORKSPACE;
  int rc = ako4x_dsa_topk_indexer(q_index_fp8, k_index_cache, weights, seq_lens, block_table, topk_indices, rows,
                                  max_pages, num_cache_pages, workspace, a, stream);
  if (rc != AKO4X_OK) return rc;
  // the index space of the top-k list is the flattened cache: num_cache_pages * 64 rows
  return ako4x_dsa_sparse_attention(q_nope, q_pe, ckv_cache, kpe_cache, topk_indices, sm_scale, o, lse, rows, 2048,
                                    num_cache_pages * 64, (unsigned char*)workspace + a, b, stream);
}

// ---- causal paged MLA prefill --------------------------------------------------------------------
extern "C" size_t ako4x_mla_paged_prefill_workspace_bytes(int64_t total_q, int64_t batch,
                                                          int64_t num_kv_indices, int64_t page_size) {
  if (total_q < kPrefillTcMinQueries) return 0;
  return ako_mla_prefill_tc_workspace_bytes(batch, num_kv_indices, page_size);
}

extern "C" int ako4x_mla_paged_prefill(const void* q_nope, const void* q_pe, const void* ckv_cache,
                                       const void* kpe_cache, const int32_t* qo_indptr,
                                       const int32_t* kv_indptr, const int32_t* kv_indices,
                                       float sm_scale, void* o, float* lse, int64_t total_q,
                                       int64_t batch, int64_t num_kv_indices, int64_t page_size,
                                       void* workspace, size_t workspace_bytes, void* stream) {
  if (total_q < 0 || batch < 0 || num_kv_indices < 0 || page_size < 1) return AKO4X_EINVAL;
  if (total_q == 0) return AKO4X_OK;
  if (batch == 0) return AKO4X_EINVAL;
  if (!q_nope || !q_pe || !ckv_cache || !kpe_cache || !qo_indptr || !kv_indptr || !o || !lse)
    return AKO4X_EINVAL;
  if (num_kv_indices > 0 && !kv_indices) return AKO4X_EINVAL;
  if (misaligned(q_nope, q_pe, ckv_cache, kpe_cache, o)) return AKO4X_EINVAL;
  // From a few query tiles on, the tensor-core path (mla_prefill_tc.cu): 4x faster at the benchmark
  // shape. Below that its fixed cost (gather of all keys, two launches) outweighs it and the
  // one-query-token-per-CTA kernel below answers in a third of the time.
  if (num_kv_indices > 0 && total_q >= kPrefillTcMinQueries)
    return ako_mla_prefill_tc_launch(q_nope, q_pe, ckv_cache, kpe_cache, qo_indptr, kv_indptr, kv_indices,
                                     sm_scale, o, lse, total_q, batch, num_kv_indices, page_size, workspace,
                                     workspace_bytes, (cudaStream_t)stream);
  Params p = {};
  fill_common(p, q_nope, q_pe, ckv_cache, kpe_cache, o, lse, sm_scale);
  p.qo_indptr = qo_indptr;
  p.kv_indptr = kv_indptr;
  p.indices = kv_indices;
  p.page_size = (int)page_size;
  p.batch = (int)batch;
  return launch<kPrefill>(p, total_q, 1, nullptr, (cudaStream_t)stream);
}

// Status word of the attention kernels of this file: 0, or the code of a bounded wait that gave
// up. Synchronises the device; meant for tests and post-mortems.
extern "C" int ako4x_mla_attention_device_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_mla_status, sizeof(int)) != cudaSuccess) return AKO4X_ELAUNCH;
  if (v == 0) v = ako_mla_prefill_tc_status();
  return v;
}
