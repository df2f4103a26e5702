// DSA top-k indexer: FP8 index scores + exact top-2048 selection.
//
// Score kernel: score = (sum_h w[r,h] * relu(q[r,h,:] . k[t,:])) * kscale[t] on the tcgen05 tensor
// cores (dsa_score_tc.cuh): tokens on the M dimension / TMEM lanes, heads of up to four query rows
// on the N dimension, TMA-fed, relu + head weights + head sum as per-thread arithmetic on the
// accumulator. Scores are written as fp32.
//
// Select kernel: one CTA per row. Keys are the order-preserving unsigned image of the fp32 scores;
// a 4 x 8-bit most-significant-digit radix select (warp-aggregated shared-memory histograms)
// finds the 2048-th largest key, then a stable compaction in token order emits every token above
// the threshold plus the first tokens equal to it (ties: lower position wins), translated to
// global cache slots through the block table.
#include "common.cuh"
#include "tcgen05.cuh"
#include "tma_host.cuh"

namespace {

constexpr int NH = 64, HD = 128, PS = 64, TOPK = 2048;
constexpr int PAGE_BYTES = PS * HD + PS * 4;  // 8448

// ---------------------------------------------------------------------------------------------
// score kernel (tensor cores)
// ---------------------------------------------------------------------------------------------
#include "dsa_score_tc.cuh"

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

int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int launch_scores(const void* q, const void* cache, const float* weights, const int32_t* seq_lens,
                  const int32_t* block_table, float* scores, int64_t rows, int64_t max_pages,
                  int64_t num_cache_pages, int skip_short, cudaStream_t st) {
  if (num_cache_pages < 1) return AKO4X_EINVAL;
  if (!ako::ensure_dynamic_smem<dsa_score_tc_kernel>(TS_SMEM)) return AKO4X_ELAUNCH;
  CUtensorMap tm_q, tm_k;
  if (!ako::tma::byte_matrix_map(&tm_q, q, (uint64_t)rows * NH, HD, NH) ||
      !ako::tma::paged_byte_matrix_map(&tm_k, cache, (uint64_t)num_cache_pages, PAGE_BYTES, PS))
    return AKO4X_ELAUNCH;
  ScoreParams p;
  p.weights = weights;
  p.seq_lens = seq_lens;
  p.block_table = block_table;
  p.cache = (const unsigned char*)cache;
  p.scores = scores;
  p.rows = (int)rows;
  p.max_pages = (int)max_pages;
  p.num_cache_pages = num_cache_pages;
  p.skip_short = skip_short;
  const int64_t units = ako::cdiv(rows, TS_ROWS) * ako::cdiv(max_pages, 2);
  const int grid = (int)(units < sm_count() ? units : sm_count());
  dsa_score_tc_kernel<<<grid, TS_THREADS, TS_SMEM, st>>>(p, tm_q, tm_k);
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

// Status word of the score kernel: 0, or the code of a bounded wait that gave up. Synchronises
// the device; meant for tests and post-mortems.
extern "C" int ako4x_dsa_indexer_device_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_dsa_status, sizeof(int)) != cudaSuccess) return AKO4X_ELAUNCH;
  return v;
}
