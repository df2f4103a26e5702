// Paged GQA decode: 32 query heads, 8 KV heads, head_dim 128, bf16.
//
// HBM-bound: every KV token costs 4096 bytes (8 heads x 128 x bf16 for K and again for V) and
// only 4 query rows reuse it. One CTA owns (sequence, KV split, half of the KV heads): its 4
// warps each run flash-decoding for one KV head (the 4 query heads of that group padded to an
// m16 tile of mma.sync) over a 3-stage ring of 16-token tiles. A token's four K heads are 1 KB
// contiguous in the cache, so the gather is ONE 1 KB bulk copy (cp.async.bulk, completion counted
// in bytes on the stage's mbarrier) per token per tensor, issued by 16 lanes of warp 0; 16-byte
// cp.async copies run out of outstanding-request slots long before HBM is busy. Gather indices are
// fetched one tile ahead of the copies that need them. Rows sit in shared memory with a 1040-byte
// pitch, which keeps ldmatrix bank-conflict free without a swizzle. Partials (m, l, acc) go to the
// workspace in fp32 and a second kernel merges them; with one split the CTA writes o and lse
// itself. Waits on the mbarriers are bounded: a wait that exceeds its cycle limit records a code in
// a device status word and the CTA stops consuming.
#include "lse_merge.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int HQ = 32, HKV = 8, D = 128, GROUP = HQ / HKV;
constexpr int HPC = 4;        // KV heads per CTA (one per warp); 8 (2 KB rows, one CTA per SM) measured the same
constexpr int HEAD_GROUPS = HKV / HPC;  // CTAs that share one (sequence, split)
constexpr int CTAS_PER_SM = (HPC == 4) ? 2 : 1;
constexpr int TILE = 16;      // tokens per pipeline stage
constexpr int STAGES = 3;
constexpr int THREADS = HPC * 32;
constexpr int ROW_BYTES = HPC * D * 2;            // 1024: the CTA's heads of one token, one tensor
constexpr int PITCH = ROW_BYTES + 16;             // shared-memory row pitch
constexpr int TENSOR_TILE_BYTES = TILE * PITCH;   // 16640
constexpr int STAGE_BYTES = 2 * TENSOR_TILE_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES;  // 99840 -> two CTAs per SM
constexpr int MAX_SPLITS = 64;

__device__ int g_gqa_status = 0;  // 0 = ok; set when a bounded wait gave up

struct Params {
  const __nv_bfloat16* q;
  const unsigned char* k;
  const unsigned char* v;
  const int32_t* indptr;
  const int32_t* indices;
  __nv_bfloat16* o;
  float* lse;
  float* part_acc;  // [batch*32][splits][128]
  float* part_ml;   // [batch*32][splits][2]
  float scale_log2;
  int page_size;
  int num_splits;       // uniform mode: every sequence is cut into this many chunks
  // work-list mode (items != nullptr): chunks of `chunk_tokens` tokens; item i = (sequence, chunk
  // ordinal) or (-1, -1); partials are indexed by item, item_start[b] .. item_start[b+1] are the
  // items of sequence b.
  const int2* items;
  int chunk_tokens;
};

__global__ void __launch_bounds__(THREADS, CTAS_PER_SM) gqa_decode_kernel(Params p) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t s_full[STAGES];
  __shared__ int s_err;  // code of a wait of this CTA that gave up (0 = none), published on exit

  int split, half, b, item = 0;
  if (p.items) {
    ako::pdl_wait();  // the work list is written by the planning kernel launched just before
    item = blockIdx.x / HEAD_GROUPS;
    half = blockIdx.x % HEAD_GROUPS;
    const int2 it = p.items[item];
    b = it.x;
    split = it.y;
    if (b < 0) return;  // unused slot of the worst-case grid
  } else {
    split = blockIdx.x % p.num_splits;
    half = (blockIdx.x / p.num_splits) % HEAD_GROUPS;
    b = blockIdx.x / (p.num_splits * HEAD_GROUPS);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int head0 = half * HPC;
  const int kvh = head0 + warp;
  const uint32_t smem_base = ako::smem_u32(smem);

  ako::pdl_trigger();  // the merge kernel may be scheduled early; it waits for this grid to finish
  const int32_t* idx = p.indices + p.indptr[b];
  const int len = (int)(p.indptr[b + 1] - p.indptr[b]) * p.page_size;
  int chunk = p.items ? p.chunk_tokens : (int)ako::round_up(ako::cdiv(len, p.num_splits), TILE);
  if (chunk < TILE) chunk = TILE;
  const int tok_begin = min(len, split * chunk);
  const int tok_end = min(len, tok_begin + chunk);
  const int ntiles = (tok_end - tok_begin + TILE - 1) / TILE;

  if (ntiles == 0 && (p.num_splits > 1 || p.items)) {
    // Nothing in this chunk (the sequence is shorter than split * chunk, or empty): an empty
    // partial, which the merge skips without reading the accumulator.
    if (g < GROUP && t == 0) {
      float* ml = p.part_ml + (p.items ? ((int64_t)item * HQ + kvh * GROUP + g)
                                       : (((int64_t)b * HQ + kvh * GROUP + g) * p.num_splits + split)) * 2;
      ml[0] = -INFINITY;
      ml[1] = 0.f;
    }
    return;
  }
  // Shared memory starts finite: rows of tokens past the end are never copied, and 0 * stale
  // must not be NaN in the PV product.
  for (int i = threadIdx.x; i < SMEM_BYTES / 16; i += THREADS) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) ako::tc::mbar_init(ako::smem_u32(&s_full[s]), 1);
    ako::tc::mbar_init_fence();
    s_err = 0;
  }
  ako::tc::fence_proxy_async_smem();  // the zero fill is ordered before the bulk copies
  __syncthreads();

  // ---- producer state (warp 0, lanes 0..15: one token of a tile each) ------------------------
  const int64_t head_off = (int64_t)head0 * D * 2;
  // The page id of this lane's token in the next tile to be issued is loaded one iteration early
  // and only LOADED there: nothing depends on it until issue_tile, so warp 0 never stalls on the
  // index fetch in front of the barrier the other warps wait at.
  int32_t page_next = 0;
  auto fetch_row = [&](int tile) {
    int tok = tok_begin + tile * TILE + lane;
    tok = min(tok, max(tok_end - 1, 0));  // a valid address even when this lane has no token
    if (len > 0) page_next = __ldg(idx + (p.page_size == 1 ? tok : tok / p.page_size));
  };
  auto issue_tile = [&](int tile) {  // uses page_next fetched for `tile`
    const int stage = tile % STAGES;
    const uint32_t bar = ako::smem_u32(&s_full[stage]);
    const int tok = tok_begin + tile * TILE + lane;
    const bool valid = lane < TILE && tok < tok_end;
    const int64_t row_next = (p.page_size == 1) ? (int64_t)page_next
                                                : (int64_t)page_next * p.page_size + tok % p.page_size;
    const unsigned m = __ballot_sync(0xffffffffu, valid);
    if (lane == 0) ako::tc::mbar_arrive_expect_tx(bar, (uint32_t)__popc(m) * 2 * ROW_BYTES);
    __syncwarp();
    if (valid) {
      const uint32_t dst = smem_base + stage * STAGE_BYTES + lane * PITCH;
      const int64_t src = row_next * (HKV * D * 2) + head_off;
      ako::tc::bulk_load_1d(dst, p.k + src, ROW_BYTES, bar);
      ako::tc::bulk_load_1d(dst + TENSOR_TILE_BYTES, p.v + src, ROW_BYTES, bar);
    }
  };
  if (warp == 0) {
    for (int s = 0; s < STAGES - 1; ++s) {
      if (s < ntiles) {
        fetch_row(s);
        issue_tile(s);
      }
    }
    fetch_row(STAGES - 1);
  }

  // Q fragments of this warp's group (rows g<4 real, others zero).
  uint32_t qa[8][2];
  {
    const __nv_bfloat16* qrow = p.q + ((int64_t)b * HQ + kvh * GROUP + (g & 3)) * D;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t v0 = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t);
      uint32_t v1 = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t);
      qa[ks][0] = (g < GROUP) ? v0 : 0u;
      qa[ks][1] = (g < GROUP) ? v1 : 0u;
    }
  }

  float oacc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;

  for (int it = 0; it < ntiles; ++it) {
    const int stage = it % STAGES;
    const bool landed = ako::tc::mbar_wait(ako::smem_u32(&s_full[stage]), (uint32_t)((it / STAGES) & 1),
                                           &s_err, 1);
    // every warp has finished tile it-1: its stage is free for tile it+STAGES-1
    if (!__syncthreads_and(landed)) break;  // a wait gave up: the whole CTA stops consuming
    if (warp == 0) {
      ako::tc::fence_proxy_async_smem();  // generic reads of the freed stage before async writes
      if (it + STAGES - 1 < ntiles) issue_tile(it + STAGES - 1);
      fetch_row(it + STAGES);
    }
    const uint32_t Ks = smem_base + stage * STAGE_BYTES + warp * (D * 2);
    const uint32_t Vs = Ks + TENSOR_TILE_BYTES;

    // S = Q K^T : 2 n-tiles of 8 tokens
    float sacc[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
    {
      const int tok = ((lane >> 4) << 3) + (lane & 7);
      const int csel = (lane >> 3) & 1;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t b00, b01, b10, b11;
        ako::ldmatrix_x4(b00, b01, b10, b11, Ks + tok * PITCH + ((2 * ks + csel) << 4));
        const uint32_t a[4] = {qa[ks][0], 0u, qa[ks][1], 0u};
        ako::mma_bf16_16816(sacc[0], a, b00, b01);
        ako::mma_bf16_16816(sacc[1], a, b10, b11);
      }
    }
    // online softmax on row g (tokens: n-tile i, columns 2t, 2t+1)
    const int tile_tok0 = tok_begin + it * TILE;
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int tk = tile_tok0 + i * 8 + 2 * t + j;
        float s = sacc[i][j] * p.scale_log2;
        s = (tk < tok_end) ? s : -INFINITY;
        sacc[i][j] = s;
        mx = fmaxf(mx, s);
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);  // finite: every tile holds at least one valid token
    const float corr = ako::fast_exp2(m_run - m_new);
    float psum = 0.f;
    uint32_t pa[4];
    {
      const float p00 = ako::fast_exp2(sacc[0][0] - m_new), p01 = ako::fast_exp2(sacc[0][1] - m_new);
      const float p10 = ako::fast_exp2(sacc[1][0] - m_new), p11 = ako::fast_exp2(sacc[1][1] - m_new);
      psum = (p00 + p01) + (p10 + p11);
      pa[0] = ako::pack_bf16x2(p00, p01);
      pa[1] = 0u;
      pa[2] = ako::pack_bf16x2(p10, p11);
      pa[3] = 0u;
    }
    psum += __shfl_xor_sync(0xffffffffu, psum, 1);
    psum += __shfl_xor_sync(0xffffffffu, psum, 2);
    l_run = l_run * corr + psum;
    m_run = m_new;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      oacc[i][0] *= corr;
      oacc[i][1] *= corr;
    }
    // O += P V : 16 n-tiles of 8 dims, k = 16 tokens
    {
      const int tok = (((lane >> 3) & 1) << 3) + (lane & 7);
      const int csel = lane >> 4;
#pragma unroll
      for (int nd = 0; nd < 16; nd += 2) {
        uint32_t v00, v01, v10, v11;
        ako::ldmatrix_x4_trans(v00, v01, v10, v11, Vs + tok * PITCH + ((nd + csel) << 4));
        ako::mma_bf16_16816(oacc[nd], pa, v00, v01);
        ako::mma_bf16_16816(oacc[nd + 1], pa, v10, v11);
      }
    }
  }
  if (threadIdx.x == 0 && s_err != 0) atomicCAS(&g_gqa_status, 0, s_err);

  if (g < GROUP) {
    const int64_t rh = (int64_t)b * HQ + kvh * GROUP + g;
    if (p.num_splits == 1 && !p.items) {
      const float inv = (l_run > 0.f) ? 1.f / l_run : 0.f;
      __nv_bfloat16* op = p.o + rh * D;
#pragma unroll
      for (int nd = 0; nd < 16; ++nd)
        *reinterpret_cast<uint32_t*>(op + nd * 8 + 2 * t) =
            ako::pack_bf16x2(oacc[nd][0] * inv, oacc[nd][1] * inv);
      if (t == 0) p.lse[rh] = (l_run > 0.f) ? m_run + log2f(l_run) : -INFINITY;
    } else {
      const int64_t pidx = p.items ? ((int64_t)item * HQ + kvh * GROUP + g) : (rh * p.num_splits + split);
      float* pa_out = p.part_acc + pidx * D;
#pragma unroll
      for (int nd = 0; nd < 16; ++nd)
        *reinterpret_cast<float2*>(pa_out + nd * 8 + 2 * t) = make_float2(oacc[nd][0], oacc[nd][1]);
      if (t == 0) {
        float* ml = p.part_ml + pidx * 2;
        ml[0] = m_run;
        ml[1] = l_run;
      }
    }
  }
}

// Work list for ragged batches: sequence b is cut into max(1, ceil(len_b / chunk)) chunks of `chunk`
// tokens, so every CTA has about the same work whatever the mix of lengths. One block.
__global__ void __launch_bounds__(256) gqa_plan_kernel(const int32_t* __restrict__ indptr, int batch,
                                                       int page_size, int chunk, int max_items,
                                                       int32_t* __restrict__ item_start,
                                                       int2* __restrict__ items) {
  __shared__ int s_scan[256];
  __shared__ int s_base;
  const int tid = threadIdx.x;
  if (tid == 0) s_base = 0;
  __syncthreads();
  for (int b0 = 0; b0 < batch; b0 += 256) {
    const int b = b0 + tid;
    int n = 0;
    if (b < batch) {
      const int len = (indptr[b + 1] - indptr[b]) * page_size;
      n = max(1, (len + chunk - 1) / chunk);
    }
    s_scan[tid] = n;
    __syncthreads();
    for (int off = 1; off < 256; off <<= 1) {  // inclusive Hillis-Steele scan
      const int add = (tid >= off) ? s_scan[tid - off] : 0;
      __syncthreads();
      s_scan[tid] += add;
      __syncthreads();
    }
    const int start = s_base + s_scan[tid] - n;
    if (b < batch) {
      // kv_indptr[batch] beyond the num_kv_indices the workspace was sized for: the list is cut at
      // max_items (those sequences lose their tail), the merge stays inside the partial area, and
      // the status word records it.
      item_start[b] = min(start, max_items);
      for (int c = 0; c < n && start + c < max_items; ++c) items[start + c] = make_int2(b, c);
    }
    __syncthreads();
    if (tid == 255) s_base += s_scan[255];
    __syncthreads();
  }
  if (tid == 0) {
    item_start[batch] = min(s_base, max_items);
    if (s_base > max_items) atomicCAS(&g_gqa_status, 0, 20);
  }
  for (int i = s_base + tid; i < max_items; i += 256) items[i] = make_int2(-1, -1);
}

// Merge of the work-list partials: one block per (sequence, head); 32 threads x 4 columns.
__global__ void __launch_bounds__(D / 4) gqa_merge_items_kernel(
    const float* __restrict__ part_acc, const float* __restrict__ part_ml,
    const int32_t* __restrict__ item_start, __nv_bfloat16* __restrict__ o, float* __restrict__ lse) {
  ako::pdl_wait();
  const int b = blockIdx.x / HQ, h = blockIdx.x % HQ;
  const int i0 = item_start[b], i1 = item_start[b + 1];
  float M = -INFINITY;
  for (int i = i0; i < i1; ++i) M = fmaxf(M, part_ml[((int64_t)i * HQ + h) * 2]);
  float L = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (M > -INFINITY) {
    for (int i = i0; i < i1; ++i) {
      const float* ml = part_ml + ((int64_t)i * HQ + h) * 2;
      if (ml[0] == -INFINITY) continue;
      const float w = exp2f(ml[0] - M);
      L = fmaf(ml[1], w, L);
      const float4 p4 = *reinterpret_cast<const float4*>(part_acc + ((int64_t)i * HQ + h) * D + threadIdx.x * 4);
      acc.x = fmaf(p4.x, w, acc.x);
      acc.y = fmaf(p4.y, w, acc.y);
      acc.z = fmaf(p4.z, w, acc.z);
      acc.w = fmaf(p4.w, w, acc.w);
    }
  }
  const float inv = (L > 0.f) ? 1.f / L : 0.f;
  uint2 pk;
  pk.x = ako::pack_bf16x2(acc.x * inv, acc.y * inv);
  pk.y = ako::pack_bf16x2(acc.z * inv, acc.w * inv);
  *reinterpret_cast<uint2*>(o + (int64_t)blockIdx.x * D + threadIdx.x * 4) = pk;
  if (threadIdx.x == 0) lse[blockIdx.x] = (L > 0.f) ? M + log2f(L) : -INFINITY;
}

// Work-list mode pays a third launch, so it is used where ragged lengths cost more than that:
// batches that fill the GPU several times over with long sequences.
struct Plan {
  bool on;
  int chunk;
  int64_t max_items;
};
Plan pick_plan(int64_t batch, int64_t num_kv_indices, int64_t page_size) {
  Plan pl = {false, 0, 0};
  if (batch <= 0) return pl;
  const int64_t total = num_kv_indices * page_size;
  const int64_t avg_len = total / batch;
  const int64_t slots = 148 * CTAS_PER_SM;
  if (avg_len < 1024 || total < 64 * 1024 || total / 256 * HEAD_GROUPS < 4 * slots) return pl;
  // about six waves of equal chunks, at least 256 tokens each
  int64_t chunk = ako::cdiv(total, 6 * slots / HEAD_GROUPS);
  if (chunk < 256) chunk = 256;
  chunk = ako::round_up(chunk, (int64_t)TILE);
  const int64_t items = ako::cdiv(total, chunk) + batch;
  if (chunk > 0x3fffffff || items * HEAD_GROUPS > 0x7fffffffLL) return pl;
  pl.on = true;
  pl.chunk = (int)chunk;
  pl.max_items = items;
  return pl;
}
size_t plan_workspace(const Plan& pl, int64_t batch) {
  // partial accumulators, partial (m, l), item table, item_start
  return (size_t)pl.max_items * HQ * (D + 2) * sizeof(float) + (size_t)pl.max_items * sizeof(int2) +
         ((size_t)(batch + 1) * sizeof(int32_t) + 15) / 16 * 16;
}

int pick_splits(int64_t batch, int64_t num_kv_indices, int64_t page_size) {
  if (batch <= 0) return 1;
  const int64_t avg_len = num_kv_indices * page_size / batch;
  const int64_t slots = 148 * CTAS_PER_SM;                      // resident CTAs
  const int64_t pairs = HEAD_GROUPS * batch;                    // CTAs per split
  // Long sequences: chunks of about 300 tokens. Every sequence of a batch gets the same split
  // count, so with ragged lengths the longest chunks set the makespan; a sweep at B = 64 and 256
  // (lengths U[128, 8192]) was best between 280 and 450 tokens per chunk and 5 % worse at 900.
  // Short sequences: 128-token chunks, and at least two waves of CTAs when chunks of 128 allow it.
  int64_t s = avg_len / (avg_len >= 2048 ? 300 : 128);
  int64_t t = ako::cdiv(2 * slots, pairs);
  if (t > avg_len / 128) t = avg_len / 128;
  if (s < t) s = t;
  if (s < 1) s = 1;
  // A small batch that still leaves SMs idle: the call's latency is the chunk length, so go down
  // to two 16-token tiles per chunk, up to one wave of CTAs.
  if (pairs * s < slots) {
    const int64_t fine = avg_len / (2 * TILE) > 1 ? avg_len / (2 * TILE) : 1;
    const int64_t one_wave = slots / pairs > 1 ? slots / pairs : 1;
    s = fine < one_wave ? fine : one_wave;
  }
  if (s > MAX_SPLITS) s = MAX_SPLITS;
  return (int)s;
}

}  // namespace

extern "C" size_t ako4x_gqa_paged_decode_workspace_bytes(int64_t batch, int64_t num_kv_indices,
                                                         int64_t page_size) {
  const Plan pl = pick_plan(batch, num_kv_indices, page_size);
  if (pl.on) return plan_workspace(pl, batch);
  const int s = pick_splits(batch, num_kv_indices, page_size);
  if (s == 1) return 0;
  return (size_t)batch * HQ * s * (D + 2) * sizeof(float);
}

extern "C" int ako4x_gqa_paged_decode(const void* q, const void* k_cache, const void* v_cache,
                                      const int32_t* kv_indptr, const int32_t* kv_indices,
                                      float sm_scale, void* o, float* lse, int64_t batch,
                                      int64_t num_kv_indices, int64_t page_size, void* workspace,
                                      size_t workspace_bytes, void* stream) {
  if (batch < 0 || num_kv_indices < 0 || page_size < 1) return AKO4X_EINVAL;
  if (batch == 0) return AKO4X_OK;
  if (!q || !k_cache || !v_cache || !kv_indptr || !o || !lse) return AKO4X_EINVAL;
  if (num_kv_indices > 0 && !kv_indices) return AKO4X_EINVAL;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)o) & 15) return AKO4X_EINVAL;
  const Plan pl = pick_plan(batch, num_kv_indices, page_size);
  const int splits = pl.on ? 1 : pick_splits(batch, num_kv_indices, page_size);
  const size_t need = ako4x_gqa_paged_decode_workspace_bytes(batch, num_kv_indices, page_size);
  if (need > 0 && (!workspace || workspace_bytes < need)) return AKO4X_EWORKSPACE;
  if (need > 0 && ((uintptr_t)workspace & 15)) return AKO4X_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;

  Params p;
  p.q = (const __nv_bfloat16*)q;
  p.k = (const unsigned char*)k_cache;
  p.v = (const unsigned char*)v_cache;
  p.indptr = kv_indptr;
  p.indices = kv_indices;
  p.o = (__nv_bfloat16*)o;
  p.lse = lse;
  p.part_acc = (float*)workspace;
  p.part_ml = p.part_acc ? p.part_acc + (size_t)batch * HQ * splits * D : nullptr;
  p.scale_log2 = sm_scale * AKO_LOG2E;
  p.page_size = (int)page_size;
  p.num_splits = splits;
  p.items = nullptr;
  p.chunk_tokens = 0;

  if (!ako::ensure_dynamic_smem<gqa_decode_kernel>(SMEM_BYTES)) return AKO4X_ELAUNCH;
  if (pl.on) {
    // workspace: [items][32][128] accumulators | [items][32][2] (m, l) | item table | item_start
    p.part_ml = p.part_acc + (size_t)pl.max_items * HQ * D;
    int2* items = reinterpret_cast<int2*>(p.part_ml + (size_t)pl.max_items * HQ * 2);
    int32_t* item_start = reinterpret_cast<int32_t*>(items + pl.max_items);
    p.items = items;
    p.chunk_tokens = pl.chunk;
    gqa_plan_kernel<<<1, 256, 0, st>>>(kv_indptr, (int)batch, (int)page_size, pl.chunk, (int)pl.max_items,
                                       item_start, items);
    AKO_CHECK_LAUNCH();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(pl.max_items * HEAD_GROUPS));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, gqa_decode_kernel, p) != cudaSuccess) return AKO4X_ELAUNCH;
    cudaLaunchConfig_t mcfg = {};
    mcfg.gridDim = dim3((unsigned)(batch * HQ));
    mcfg.blockDim = dim3(D / 4);
    mcfg.stream = st;
    mcfg.attrs = attr;
    mcfg.numAttrs = 1;
    const float* pacc = p.part_acc;
    const float* pml = p.part_ml;
    const int32_t* is = item_start;
    __nv_bfloat16* op = p.o;
    float* lp = p.lse;
    if (cudaLaunchKernelEx(&mcfg, gqa_merge_items_kernel, pacc, pml, is, op, lp) != cudaSuccess)
      return AKO4X_ELAUNCH;
    return AKO4X_OK;
  }
  const int64_t grid = batch * HEAD_GROUPS * splits;
  if (grid > 0x7fffffffLL) return AKO4X_EINVAL;
  gqa_decode_kernel<<<(unsigned)grid, THREADS, SMEM_BYTES, st>>>(p);
  AKO_CHECK_LAUNCH();
  if (splits > 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(batch * HQ));
    cfg.blockDim = dim3(D / 4);
    cfg.dynamicSmemBytes = 0;
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
    if (cudaLaunchKernelEx(&cfg, ako::lse_merge_kernel<D, 4>, pacc, pml, op, lp, ns) != cudaSuccess)
      return AKO4X_ELAUNCH;
  }
  return AKO4X_OK;
}

// Status word of the decode kernel of this file: 0, or the code of a bounded wait that gave up.
// Synchronises the device; meant for tests and post-mortems.
extern "C" int ako4x_gqa_paged_decode_device_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gqa_status, sizeof(int)) != cudaSuccess) return AKO4X_ELAUNCH;
  return v;
}
