// DSA top-k indexer: FP8 index scores + exact top-2048 selection.
//
// Score kernel: for query row r and token t, score = (sum_h w[r,h] * relu(q[r,h,:] . k[t,:])) *
// kscale[t]. Tokens are the M dimension of mma.sync.m16n8k32 (e4m3 x e4m3 -> fp32), the 64 index
// heads the N dimension, so relu, the head weights and the head reduction all happen in the
// accumulator registers of the thread that owns the token (two shuffles finish the sum). A warp
// owns one 64-token cache page at a time: the 8 KB of e4m3 values are copied with cp.async into a
// private double-buffered shared-memory slot (16-byte chunks XOR-swizzled by token) and read back
// with ldmatrix; Q fragments and head weights stay in registers. Scores are written as fp32.
//
// Select kernel: one CTA per row. Keys are the order-preserving unsigned image of the fp32 scores;
// a 4 x 8-bit most-significant-digit radix select (warp-aggregated shared-memory histograms)
// finds the 2048-th largest key, then a stable compaction in token order emits every token above
// the threshold plus the first tokens equal to it (ties: lower position wins), translated to
// global cache slots through the block table.
#include "common.cuh"

namespace {

constexpr int NH = 64, HD = 128, PS = 64, TOPK = 2048;
constexpr int PAGE_BYTES = PS * HD + PS * 4;  // 8448

// ---------------------------------------------------------------------------------------------
// score kernel
// ---------------------------------------------------------------------------------------------
constexpr int SC_WARPS = 4;
constexpr int SC_THREADS = SC_WARPS * 32;
constexpr int SC_MAX_PAGES_PER_WARP = 8;  // pages a warp walks; fewer when the grid would be small
constexpr int SC_SMEM = SC_WARPS * 2 * PS * HD;  // 64 KB

__device__ __forceinline__ void load_page(unsigned char* slot, const unsigned char* page, int lane) {
  // 64 rows x 8 chunks of 16 B; a warp pass covers 4 rows.
#pragma unroll
  for (int pass = 0; pass < 16; ++pass) {
    const int row = pass * 4 + (lane >> 3);
    const int c = lane & 7;
    ako::cp_async16(ako::smem_u32(slot + row * HD + ((c ^ (row & 7)) << 4)), page + row * HD + c * 16);
  }
}

__global__ void __launch_bounds__(SC_THREADS) dsa_score_kernel(
    const unsigned char* __restrict__ q, const unsigned char* __restrict__ cache,
    const float* __restrict__ weights, const int32_t* __restrict__ seq_lens,
    const int32_t* __restrict__ block_table, float* __restrict__ scores, int max_pages,
    int64_t num_cache_pages, int skip_short, int pages_per_warp) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int r = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  ako::pdl_trigger();
  const int sl = seq_lens[r];
  float* out = scores + (int64_t)r * max_pages * PS;
  const int page_lo = blockIdx.y * SC_WARPS * pages_per_warp;
  if (sl <= 0 || (skip_short && sl <= TOPK)) return;
  const int npages = min(max_pages, (sl + PS - 1) / PS);

  // B fragments: Q[head][k] for 8 n-tiles x 4 k-steps, and this thread's head weights.
  uint32_t qb[8][4][2];
  float wv[8][2];
  {
    const unsigned char* qr = q + (int64_t)r * NH * HD;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const unsigned char* qh = qr + (nt * 8 + g) * HD;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        qb[nt][ks][0] = *reinterpret_cast<const uint32_t*>(qh + ks * 32 + 4 * t);
        qb[nt][ks][1] = *reinterpret_cast<const uint32_t*>(qh + ks * 32 + 16 + 4 * t);
      }
      const float2 w2 = *reinterpret_cast<const float2*>(weights + (int64_t)r * NH + nt * 8 + 2 * t);
      wv[nt][0] = w2.x;
      wv[nt][1] = w2.y;
    }
  }

  unsigned char* slot0 = smem + warp * 2 * PS * HD;
  const int32_t* bt = block_table + (int64_t)r * max_pages;
  // pages of this warp: page_lo + warp + SC_WARPS * j
  int pg_next = page_lo + warp;
  int64_t phys_cur = -1, phys_next = -1;
  if (pg_next < npages) {
    phys_next = bt[pg_next];
    if (phys_next < 0 || phys_next >= num_cache_pages) phys_next = 0;  // out-of-range id: stay in bounds
    load_page(slot0, cache + phys_next * PAGE_BYTES, lane);
  }
  ako::cp_async_commit();

  for (int j = 0; j < pages_per_warp; ++j) {
    const int pg = page_lo + warp + SC_WARPS * j;
    if (pg >= npages) break;
    phys_cur = phys_next;
    pg_next = pg + SC_WARPS;
    if (j + 1 < pages_per_warp && pg_next < npages) {
      phys_next = bt[pg_next];
      if (phys_next < 0 || phys_next >= num_cache_pages) phys_next = 0;
      load_page(slot0 + ((j + 1) & 1) * PS * HD, cache + phys_next * PAGE_BYTES, lane);
    }
    ako::cp_async_commit();
    ako::cp_async_wait<1>();
    __syncwarp();
    const unsigned char* ks_smem = slot0 + (j & 1) * PS * HD;
    const float* kscale = reinterpret_cast<const float*>(cache + phys_cur * PAGE_BYTES + PS * HD);

#pragma unroll 1
    for (int mt = 0; mt < 4; ++mt) {  // 16 tokens per m-tile
      uint32_t a[4][4];
      {
        const int row = mt * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const int c = 2 * ks + (lane >> 4);
          ako::ldmatrix_x4(a[ks][0], a[ks][1], a[ks][2], a[ks][3],
                           ako::smem_u32(ks_smem + row * HD + ((c ^ (row & 7)) << 4)));
        }
      }
      float s0 = 0.f, s1 = 0.f;  // tokens g and g+8 of the m-tile
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) ako::mma_e4m3_16832(c, a[ks], qb[nt][ks][0], qb[nt][ks][1]);
        s0 = fmaf(fmaxf(c[0], 0.f), wv[nt][0], s0);
        s0 = fmaf(fmaxf(c[1], 0.f), wv[nt][1], s0);
        s1 = fmaf(fmaxf(c[2], 0.f), wv[nt][0], s1);
        s1 = fmaf(fmaxf(c[3], 0.f), wv[nt][1], s1);
      }
      s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
      s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
      s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
      s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
      if (t < 2) {
        const int tok_in_page = mt * 16 + g + 8 * t;
        const int tok = pg * PS + tok_in_page;
        const float v = (t == 0 ? s0 : s1) * __ldg(kscale + tok_in_page);
        out[tok] = (tok < sl) ? v : -INFINITY;
      }
    }
    __syncwarp();  // the slot is overwritten two iterations later; keep the warp together
  }
  ako::cp_async_wait<0>();
}

// ---------------------------------------------------------------------------------------------
// select kernel
// ---------------------------------------------------------------------------------------------
constexpr int SEL_THREADS = 1024;

__device__ __forceinline__ uint32_t order_key(float s) {
  const uint32_t b = __float_as_uint(s + 0.0f);  // -0 -> +0
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__global__ void __launch_bounds__(SEL_THREADS) dsa_select_kernel(
    const float* __restrict__ scores, const int32_t* __restrict__ seq_lens,
    const int32_t* __restrict__ block_table, int32_t* __restrict__ out, int max_pages) {
  __shared__ int hist[256];
  __shared__ int scan_buf[SEL_THREADS / 32];
  __shared__ uint32_t s_prefix;
  __shared__ int s_krem;
  __shared__ int s_gt_base, s_eq_base;

  const int r = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int32_t* bt = block_table + (int64_t)r * max_pages;
  int32_t* o = out + (int64_t)r * TOPK;
  int sl = seq_lens[r];
  if (sl > max_pages * PS) sl = max_pages * PS;

  if (sl <= TOPK) {  // every token, in order, then -1; needs no scores
    for (int k = tid; k < TOPK; k += SEL_THREADS)
      o[k] = (k < sl) ? bt[k >> 6] * PS + (k & 63) : -1;
    return;
  }
  ako::pdl_wait();
  const float* s = scores + (int64_t)r * max_pages * PS;

  if (tid == 0) { s_prefix = 0u; s_krem = TOPK; }
  const int n_iter = (sl + SEL_THREADS - 1) / SEL_THREADS;

  for (int d = 3; d >= 0; --d) {
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const int krem_in = s_krem;  // read before anyone updates it at the end of this pass
    const int shift = 8 * d;
    const uint32_t hi_mask = (d == 3) ? 0u : (0xffffffffu << (shift + 8));
    for (int it = 0; it < n_iter; ++it) {
      const int i = it * SEL_THREADS + tid;
      uint32_t digit = 0x100u | lane;  // sentinel: groups with nobody
      if (i < sl) {
        const uint32_t key = order_key(s[i]);
        if ((key & hi_mask) == prefix) digit = (key >> shift) & 0xffu;
      }
      const unsigned peers = __match_any_sync(0xffffffffu, digit);
      if (digit < 0x100u && lane == (__ffs(peers) - 1)) atomicAdd(&hist[digit], __popc(peers));
    }
    __syncthreads();
    // inclusive suffix sums over the 256 bins (Hillis-Steele, 8 steps)
    int v = (tid < 256) ? hist[tid] : 0;
    const int own = v;
    for (int off = 1; off < 256; off <<= 1) {
      int add = 0;
      if (tid < 256 && tid + off < 256) add = hist[tid + off];
      __syncthreads();
      if (tid < 256) { v += add; hist[tid] = v; }
      __syncthreads();
    }
    // v = count(digit >= tid); pick the bin where the k-th largest lives
    if (tid < 256) {
      const int gt = v - own;
      if (gt < krem_in && krem_in <= v) {
        s_prefix = prefix | ((uint32_t)tid << shift);
        s_krem = krem_in - gt;
      }
    }
    __syncthreads();
  }
  const uint32_t thr = s_prefix;
  const int krem = s_krem;  // how many keys equal to thr are taken (lowest positions first)
  if (tid == 0) { s_gt_base = 0; s_eq_base = 0; }
  __syncthreads();

  for (int it = 0; it < n_iter; ++it) {
    const int i = it * SEL_THREADS + tid;
    uint32_t key = 0u;
    const bool in = i < sl;
    if (in) key = order_key(s[i]);
    const bool is_gt = in && key > thr;
    const bool is_eq = in && key == thr;
    // block-wide exclusive scan of (gt, eq) packed as eq<<16 | gt
    const unsigned bg = __ballot_sync(0xffffffffu, is_gt);
    const unsigned be = __ballot_sync(0xffffffffu, is_eq);
    const unsigned lt_mask = (1u << lane) - 1u;
    int my = __popc(bg & lt_mask) | (__popc(be & lt_mask) << 16);
    if (lane == 0) scan_buf[warp] = __popc(bg) | (__popc(be) << 16);
    __syncthreads();
    if (warp == 0) {
      int x = scan_buf[lane];
      int incl = x;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += y;
      }
      scan_buf[lane] = incl - x;  // exclusive
      if (lane == 31) hist[0] = incl;  // chunk total (hist is free now)
    }
    __syncthreads();
    my += scan_buf[warp];
    const int G = s_gt_base + (my & 0xffff);
    const int E = s_eq_base + (my >> 16);
    if (is_gt || (is_eq && E < krem)) {
      const int pos = G + min(E, krem);
      o[pos] = bt[i >> 6] * PS + (i & 63);
    }
    __syncthreads();
    if (tid == 0) {
      const int tot = hist[0];
      s_gt_base += tot & 0xffff;
      s_eq_base += tot >> 16;
    }
    __syncthreads();
  }
}

int launch_scores(const void* q, const void* cache, const float* weights, const int32_t* seq_lens,
                  const int32_t* block_table, float* scores, int64_t rows, int64_t max_pages,
                  int64_t num_cache_pages, int skip_short, cudaStream_t st) {
  if (!ako::ensure_dynamic_smem<dsa_score_kernel>(SC_SMEM)) return AKO4X_ELAUNCH;
  // enough CTAs for ~4 waves of 148 SMs x 3 resident CTAs, at most 8 pages per warp
  int64_t ppw = rows * max_pages / (SC_WARPS * 1776);
  if (ppw < 1) ppw = 1;
  if (ppw > SC_MAX_PAGES_PER_WARP) ppw = SC_MAX_PAGES_PER_WARP;
  dim3 grid((unsigned)rows, (unsigned)ako::cdiv(max_pages, SC_WARPS * ppw));
  dsa_score_kernel<<<grid, SC_THREADS, SC_SMEM, st>>>(
      (const unsigned char*)q, (const unsigned char*)cache, weights, seq_lens, block_table, scores,
      (int)max_pages, num_cache_pages, skip_short, (int)ppw);
  AKO_CHECK_LAUNCH();
  return AKO4X_OK;
}

int launch_select(const float* scores, const int32_t* seq_lens, const int32_t* block_table,
                  int32_t* out, int64_t rows, int64_t max_pages, bool pdl, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)rows);
  cfg.blockDim = dim3(SEL_THREADS);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  int mp = (int)max_pages;
  if (cudaLaunchKernelEx(&cfg, dsa_select_kernel, scores, seq_lens, block_table, out, mp) != cudaSuccess)
    return AKO4X_ELAUNCH;
  return AKO4X_OK;
}

bool bad_dims(int64_t rows, int64_t max_pages) {
  return rows < 0 || max_pages < 0 || rows > 0x7fffffffLL || max_pages > (0x7fffffffLL / PS);
}

}  // namespace

extern "C" size_t ako4x_dsa_topk_indexer_workspace_bytes(int64_t rows, int64_t max_pages) {
  if (rows <= 0 || max_pages <= 0) return 0;
  return (size_t)rows * max_pages * PS * sizeof(float);
}

extern "C" int ako4x_dsa_index_scores(const void* q_index_fp8, const void* k_index_cache,
                                      const float* weights, const int32_t* seq_lens,
                                      const int32_t* block_table, float* scores, int64_t rows,
                                      int64_t max_pages, int64_t num_cache_pages, void* stream) {
  if (bad_dims(rows, max_pages) || num_cache_pages < 0) return AKO4X_EINVAL;
  if (rows == 0 || max_pages == 0) return AKO4X_OK;
  if (!q_index_fp8 || !k_index_cache || !weights || !seq_lens || !block_table || !scores)
    return AKO4X_EINVAL;
  if (((uintptr_t)q_index_fp8 | (uintptr_t)k_index_cache) & 15) return AKO4X_EINVAL;
  return launch_scores(q_index_fp8, k_index_cache, weights, seq_lens, block_table, scores, rows,
                       max_pages, num_cache_pages, 0, (cudaStream_t)stream);
}

extern "C" int ako4x_dsa_topk_select(const float* scores, const int32_t* seq_lens,
                                     const int32_t* block_table, int32_t* topk_indices, int64_t rows,
                                     int64_t max_pages, void* stream) {
  if (bad_dims(rows, max_pages)) return AKO4X_EINVAL;
  if (rows == 0) return AKO4X_OK;
  if (!scores || !seq_lens || !block_table || !topk_indices) return AKO4X_EINVAL;
  return launch_select(scores, seq_lens, block_table, topk_indices, rows, max_pages, false,
                       (cudaStream_t)stream);
}

extern "C" int ako4x_dsa_topk_indexer(const void* q_index_fp8, const void* k_index_cache,
                                      const float* weights, const int32_t* seq_lens,
                                      const int32_t* block_table, int32_t* topk_indices, int64_t rows,
                                      int64_t max_pages, int64_t num_cache_pages, void* workspace,
                                      size_t workspace_bytes, void* stream) {
  if (bad_dims(rows, max_pages) || num_cache_pages < 0) return AKO4X_EINVAL;
  if (rows == 0) return AKO4X_OK;
  if (!q_index_fp8 || !k_index_cache || !weights || !seq_lens || !block_table || !topk_indices)
    return AKO4X_EINVAL;
  if (((uintptr_t)q_index_fp8 | (uintptr_t)k_index_cache) & 15) return AKO4X_EINVAL;
  const size_t need = ako4x_dsa_topk_indexer_workspace_bytes(rows, max_pages);
  if (need > 0 && (!workspace || workspace_bytes < need)) return AKO4X_EWORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  float* scores = (float*)workspace;
  bool pdl = false;
  // With at most 32 pages no row can exceed 2048 tokens: selection lists every token.
  if (max_pages * PS > TOPK) {
    int rc = launch_scores(q_index_fp8, k_index_cache, weights, seq_lens, block_table, scores, rows,
                           max_pages, num_cache_pages, 1, st);
    if (rc != AKO4X_OK) return rc;
    pdl = true;
  }
  return launch_select(scores, seq_lens, block_table, topk_indices, rows, max_pages, pdl, st);
}
