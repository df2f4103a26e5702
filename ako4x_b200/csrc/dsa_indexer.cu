// DSA top-k indexer: FP8 index scores + exact top-2048 selection.
//
// Score kernel: score = (sum_h w[r,h] * relu(q[r,h,:] . k[t,:])) * kscale[t] on the tcgen05 tensor
// cores (dsa_score_tc.cuh): tokens on the M dimension / TMEM lanes, heads of up to four query rows
// on the N dimension, TMA-fed, relu + head weights + head sum as per-thread arithmetic on the
// accumulator. Scores are written as fp32.
//
// Select kernel: one CTA per row. Keys are the order-preserving unsigned image of the fp32 scores,
// read once into shared memory; a three-pass most-significant-digit radix select (11, 11 and 10
// bits; the heavily repeated leading digit is warp-aggregated) finds the 2048-th largest key, then
// a stable compaction in token order emits every token above the threshold plus the first tokens
// equal to it (ties: lower position wins), translated to global cache slots through the block
// table.
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
constexpr int SEL_PER = 32;                          // tokens per thread and chunk
constexpr int SEL_CHUNK = SEL_THREADS * SEL_PER;     // 32768 tokens: one shared-memory resident chunk
constexpr int SEL_BINS = 2048;                       // widest digit: 11 bits
constexpr int SEL_SMEM = SEL_CHUNK * 4;              // 128 KB of keys

__device__ __forceinline__ uint32_t order_key(float s) {
  const uint32_t b = __float_as_uint(s + 0.0f);  // -0 -> +0
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Keys live in shared memory as 16-byte slots of four consecutive tokens. Slot f is stored at
// f ^ ((f >> 3) & 7): conflict-free both for the coalesced fill (lane = slot) and for the
// compaction, where a thread reads its own eight consecutive slots.
__device__ __forceinline__ int sel_slot(int f) { return f ^ ((f >> 3) & 7); }

// Fills the chunk's keys; tokens at or past `sl` get key 0 (below every finite score).
__device__ __forceinline__ void sel_fill(uint4* skeys, const float* __restrict__ s, int chunk, int sl, int tid) {
  const int nslots = (min(sl - chunk * SEL_CHUNK, SEL_CHUNK) + 3) >> 2;  // slots that hold a token
#pragma unroll
  for (int it = 0; it < SEL_PER / 4; ++it) {
    if (it * SEL_THREADS >= nslots) break;  // short rows: the passes below stop at the same slot
    const int f = it * SEL_THREADS + tid;
    const int i = chunk * SEL_CHUNK + 4 * f;  // a row is a whole number of 64-token pages: no overrun
    uint4 k = make_uint4(0u, 0u, 0u, 0u);
    if (i < sl) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(s + i));
      k.x = order_key(v.x);
      k.y = (i + 1 < sl) ? order_key(v.y) : 0u;
      k.z = (i + 2 < sl) ? order_key(v.z) : 0u;
      k.w = (i + 3 < sl) ? order_key(v.w) : 0u;
    }
    skeys[sel_slot(f)] = k;
  }
}

// Inclusive suffix sum over the block of one int per thread (thread 0 gets the block total).
// `buf` holds one int per warp. Two barriers.
__device__ __forceinline__ int block_suffix_sum(int x, int* buf, int lane, int warp) {
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int y = __shfl_down_sync(0xffffffffu, x, off);
    if (lane + off < 32) x += y;
  }
  if (lane == 0) buf[warp] = x;
  __syncthreads();
  int w = buf[lane];  // SEL_THREADS / 32 == 32 warps
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int y = __shfl_down_sync(0xffffffffu, w, off);
    if (lane + off < 32) w += y;
  }
  const int after = __shfl_sync(0xffffffffu, w, (warp + 1) & 31);
  __syncthreads();
  return x + ((warp < 31) ? after : 0);
}

template <int PASS>
__device__ __forceinline__ void sel_count(int* hist, uint32_t key, uint32_t prefix, int lane) {
  constexpr int shift = (PASS == 0) ? 21 : (PASS == 1) ? 10 : 0;
  constexpr uint32_t dmask = (PASS == 2) ? 0x3ffu : 0x7ffu;
  constexpr uint32_t hi_mask = (PASS == 0) ? 0u : (PASS == 1) ? 0xffe00000u : 0xfffffc00u;
  if (PASS == 0) {
    // the leading digit (sign, exponent, two mantissa bits) repeats heavily: one atomic per
    // distinct digit per warp
    const uint32_t digit = key >> shift;
    const unsigned peers = __match_any_sync(0xffffffffu, digit);
    if (lane == (__ffs(peers) - 1)) atomicAdd(&hist[digit], __popc(peers));
  } else if ((key & hi_mask) == prefix) {
    atomicAdd(&hist[(key >> shift) & dmask], 1);
  }
}

template <int PASS>
__device__ __forceinline__ void sel_pass(int* hist, const uint4* skeys, uint32_t prefix, int tid, int lane, int nslots) {
#pragma unroll
  for (int it = 0; it < SEL_PER / 4; ++it) {
    if (it * SEL_THREADS >= nslots) break;  // whole-block decision: the slots past the row were never filled
    const uint4 k = skeys[it * SEL_THREADS + tid];  // histogram: any order will do
    sel_count<PASS>(hist, k.x, prefix, lane);
    sel_count<PASS>(hist, k.y, prefix, lane);
    sel_count<PASS>(hist, k.z, prefix, lane);
    sel_count<PASS>(hist, k.w, prefix, lane);
  }
}

__global__ void __launch_bounds__(SEL_THREADS, 1) dsa_select_kernel(
    const float* __restrict__ scores, const int32_t* __restrict__ seq_lens,
    const int32_t* __restrict__ block_table, int32_t* __restrict__ out, int max_pages) {
  extern __shared__ __align__(16) unsigned char sel_smem[];
  __shared__ int hist[SEL_BINS];
  __shared__ int scan_buf[SEL_THREADS / 32];
  __shared__ int scan_buf2[SEL_THREADS / 32];
  __shared__ uint32_t s_prefix;
  __shared__ int s_krem;
  uint4* skeys = reinterpret_cast<uint4*>(sel_smem);

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
  // Up to 32768 tokens the keys are read from global memory once and stay in shared memory;
  // longer rows are swept chunk by chunk in every pass.
  const int chunks = (sl + SEL_CHUNK - 1) / SEL_CHUNK;
  sel_fill(skeys, s, 0, sl, tid);

  // ---- threshold: most-significant-digit radix select, digits of 11, 11 and 10 bits ------------
  // Padding keys (0) only ever land in the lowest bin, below the 2048-th largest real key.
  uint32_t prefix = 0u;
  int krem = TOPK;
#pragma unroll 1
  for (int pass = 0; pass < 3; ++pass) {
    const int shift = (pass == 0) ? 21 : (pass == 1) ? 10 : 0;
    hist[tid] = 0;
    hist[tid + SEL_THREADS] = 0;
    __syncthreads();  // also: the keys are in place
#pragma unroll 1
    for (int c = 0; c < chunks; ++c) {
      if (chunks > 1) {
        __syncthreads();
        sel_fill(skeys, s, c, sl, tid);
        __syncthreads();
      }
      const int nslots = (min(sl - c * SEL_CHUNK, SEL_CHUNK) + 3) >> 2;
      if (pass == 0) sel_pass<0>(hist, skeys, prefix, tid, lane, nslots);
      else if (pass == 1) sel_pass<1>(hist, skeys, prefix, tid, lane, nslots);
      else sel_pass<2>(hist, skeys, prefix, tid, lane, nslots);
    }
    __syncthreads();
    // thread t owns bins 2t and 2t+1; suffix sums give count(digit >= bin)
    const int h0 = hist[2 * tid], h1 = hist[2 * tid + 1];
    const int incl = block_suffix_sum(h0 + h1, scan_buf, lane, warp);
    const int gt1 = incl - (h0 + h1);  // keys with a larger digit than bin 2t+1
    const int gt0 = gt1 + h1;
    if (gt1 < krem && krem <= gt1 + h1) {
      s_prefix = prefix | ((uint32_t)(2 * tid + 1) << shift);
      s_krem = krem - gt1;
    } else if (gt0 < krem && krem <= gt0 + h0) {
      s_prefix = prefix | ((uint32_t)(2 * tid) << shift);
      s_krem = krem - gt0;
    }
    __syncthreads();
    prefix = s_prefix;
    krem = s_krem;  // how many keys of the chosen bin are still to be taken
  }
  const uint32_t thr = prefix;

  // ---- stable compaction in token order: keys above thr, plus the first `krem` equal to it ----
  // Thread t owns the 32 consecutive tokens of its eight slots.
  int g_base = 0, e_base = 0;
#pragma unroll 1
  for (int c = 0; c < chunks; ++c) {
    if (chunks > 1) {
      __syncthreads();
      sel_fill(skeys, s, c, sl, tid);
      __syncthreads();
    }
    const int tok0 = c * SEL_CHUNK + tid * SEL_PER;
    const int nvalid = max(0, min(SEL_PER, sl - tok0));
    uint32_t gmask = 0u, emask = 0u;  // bit j: token tok0 + j is above / equal to the threshold
#pragma unroll
    for (int q = 0; q < SEL_PER / 4; ++q) {
      const uint4 k = skeys[sel_slot(tid * (SEL_PER / 4) + q)];
      gmask |= ((k.x > thr) ? 1u : 0u) << (4 * q) | ((k.y > thr) ? 2u : 0u) << (4 * q) |
               ((k.z > thr) ? 4u : 0u) << (4 * q) | ((k.w > thr) ? 8u : 0u) << (4 * q);
      emask |= ((k.x == thr) ? 1u : 0u) << (4 * q) | ((k.y == thr) ? 2u : 0u) << (4 * q) |
               ((k.z == thr) ? 4u : 0u) << (4 * q) | ((k.w == thr) ? 8u : 0u) << (4 * q);
    }
    const uint32_t vmask = (nvalid >= 32) ? 0xffffffffu : ((1u << nvalid) - 1u);
    gmask &= vmask;
    emask &= vmask;
    const int ng = __popc(gmask), ne = __popc(emask);
    const int sg = block_suffix_sum(ng, scan_buf, lane, warp);
    const int se = block_suffix_sum(ne, scan_buf2, lane, warp);
    if (tid == 0) { scan_buf[0] = sg; scan_buf2[0] = se; }  // thread 0's suffix sum is the total
    __syncthreads();
    const int block_g = scan_buf[0], block_e = scan_buf2[0];
    int G = g_base + block_g - sg;  // above-threshold tokens before this thread's
    int E = e_base + block_e - se;  // threshold-valued tokens before this thread's
    uint32_t m = gmask | emask;
    while (m) {
      const int j = __ffs(m) - 1;
      m &= m - 1;
      const int i = tok0 + j;
      int pos;
      if (gmask >> j & 1u) {
        pos = G + min(E, krem);
        ++G;
      } else {
        pos = (E < krem) ? G + E : TOPK;
        ++E;
      }
      if (pos < TOPK) o[pos] = bt[i >> 6] * PS + (i & 63);
    }
    g_base += block_g;
    e_base += block_e;
    __syncthreads();
  }
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
  const int grid = (int)(units < ako::sm_count() ? units : ako::sm_count());
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
  cfg.dynamicSmemBytes = SEL_SMEM;
  if (!ako::ensure_dynamic_smem<dsa_select_kernel>(SEL_SMEM)) return AKO4X_ELAUNCH;
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
  if (((uintptr_t)q_index_fp8 | (uintptr_t)k_index_cache | (uintptr_t)weights) & 15) return AKO4X_EINVAL;
  return launch_scores(q_index_fp8, k_index_cache, weights, seq_lens, block_table, scores, rows,
                       max_pages, num_cache_pages, 0, (cudaStream_t)stream);
}

extern "C" int ako4x_dsa_topk_select(const float* scores, const int32_t* seq_lens,
                                     const int32_t* block_table, int32_t* topk_indices, int64_t rows,
                                     int64_t max_pages, void* stream) {
  if (bad_dims(rows, max_pages)) return AKO4X_EINVAL;
  if (rows == 0) return AKO4X_OK;
  if (!scores || !seq_lens || !block_table || !topk_indices) return AKO4X_EINVAL;
  if ((uintptr_t)scores & 15) return AKO4X_EINVAL;  // rows are read as float4
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
  if (((uintptr_t)q_index_fp8 | (uintptr_t)k_index_cache | (uintptr_t)weights) & 15) return AKO4X_EINVAL;
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
