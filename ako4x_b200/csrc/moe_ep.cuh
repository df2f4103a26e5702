// Expert-parallel exchange for the FP8 MoE over NVLink peer memory, included by moe.cu inside its
// anonymous namespace (it uses the workspace, the routing lists and the grouped GEMM of that file).
//
// One process per GPU; rank r owns experts [32r, 32r+32). Every rank holds one buffer that all its
// peers can address (mapped peer memory): a block of flag words, a receive area for token rows and
// a return area for result rows. A step has three calls on every rank, each on the caller's
// stream, none of which synchronises the host or calls a collective library:
//   dispatch  the rank's own routing decides which ranks a token goes to (one copy per destination
//             rank, not per expert). Row = e4m3 activations | 56 scales | 8 expert ids | 8 weights
//             (7456 bytes) is STORED straight into the destination's receive area, block
//             [source rank][position], positions in token order. The last CTA to finish publishes
//             the row count and the step number in the destination's flag words.
//   experts   waits (bounded) for the step number of every source, then runs the operator on the
//             received rows with the shipped ids and weights: scatter by local expert, permute,
//             grouped GEMM1 + SwiGLU, GEMM2, and a combine that stores the bf16 partial of every
//             row straight into the SOURCE rank's return area; the last CTA publishes the step
//             number there.
//   finish    waits (bounded) for every peer's step number and sums, in rank order and in fp32,
//             the partial rows of each of its tokens.
// The step number only grows, so flags are never reset. A rank can only start step n+1's dispatch
// after its own step n finished, which needed every peer's step n results, which those peers wrote
// after they had consumed the rows of step n: a receive or return area is never overwritten while
// it is still being read. Waits give up after about two seconds, record a code in the flag block
// and let the kernel finish (with undefined results) instead of hanging.
#pragma once

namespace ep {

constexpr int MAX_WORLD = 8;
constexpr int ROW_BYTES = HID + KB1 * 4 + TOPK * 4 + TOPK * 4;  // 7456
constexpr int OFF_SCALES = HID, OFF_IDS = HID + KB1 * 4, OFF_W = OFF_IDS + TOPK * 4;
constexpr size_t FLAG_BYTES = 4096;
constexpr long long kPeerWaitCycles = 4000000000LL;  // ~2 s

// flag block at the start of every rank's buffer (all words written by peers or by this rank's kernels)
struct Flags {
  int32_t disp_count[MAX_WORLD];  // rows source s sent in the current step
  int32_t disp_step[MAX_WORLD];   // last step whose rows from source s are complete
  int32_t comb_step[MAX_WORLD];   // last step whose results from expert rank g are complete
  int32_t error;                  // 0, or the code of a wait that gave up
  int32_t done_dispatch;          // CTA counters of this rank's own kernels (reset by their last CTA)
  int32_t done_return;
};

struct Peers {
  unsigned char* buf[MAX_WORLD];  // every rank's buffer as mapped into this process
};

__host__ __device__ inline size_t recv_offset() { return FLAG_BYTES; }
__host__ __device__ inline size_t ret_offset(int world, int64_t cap) {
  return FLAG_BYTES + (((size_t)world * cap * ROW_BYTES + 255) & ~(size_t)255);
}
__host__ __device__ inline size_t buffer_bytes(int world, int64_t cap) {
  return ret_offset(world, cap) + (size_t)world * cap * HID * 2;
}

__device__ __forceinline__ int ld_acquire_sys(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int32_t* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
// Spins until *flag >= step; false (and the error word set) when the limit is reached.
__device__ __forceinline__ bool wait_step(const int32_t* flag, int step, int32_t* error, int code) {
  if (ld_acquire_sys(flag) >= step) return true;
  const long long t0 = clock64();
  while (true) {
    if (ld_acquire_sys(flag) >= step) return true;
    if (*reinterpret_cast<volatile int32_t*>(error) != 0) return false;  // another wait already gave up
    if (clock64() - t0 > kPeerWaitCycles) {
      atomicCAS(error, 0, code);
      return false;
    }
    __nanosleep(100);
  }
}

// ---- dispatch 1: stable positions per destination rank (one CTA per destination) -----------------
__global__ void __launch_bounds__(1024) ep_plan_kernel(const int32_t* __restrict__ topk_ids, int tokens, int world,
                                                       int32_t* __restrict__ pos, int32_t* __restrict__ send_count) {
  __shared__ int warp_tot[32];
  __shared__ int s_base, s_chunk;
  const int g = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_base = 0;
  __syncthreads();
  for (int t0 = 0; t0 < tokens; t0 += 1024) {
    const int t = t0 + tid;
    bool hit = false;
    if (t < tokens) {
      const int4* ip = reinterpret_cast<const int4*>(topk_ids + (int64_t)t * TOPK);
      const int4 a = ip[0], b = ip[1];
      const int lo = g * 32, hi = lo + 32;
      hit = (a.x >= lo && a.x < hi) || (a.y >= lo && a.y < hi) || (a.z >= lo && a.z < hi) || (a.w >= lo && a.w < hi) ||
            (b.x >= lo && b.x < hi) || (b.y >= lo && b.y < hi) || (b.z >= lo && b.z < hi) || (b.w >= lo && b.w < hi);
    }
    const unsigned bal = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) warp_tot[warp] = __popc(bal);
    __syncthreads();
    if (warp == 0) {
      const int x = warp_tot[lane];
      int incl = x;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += y;
      }
      warp_tot[lane] = incl - x;
      if (lane == 31) s_chunk = incl;
    }
    __syncthreads();
    if (t < tokens)
      pos[(int64_t)t * world + g] = hit ? s_base + warp_tot[warp] + __popc(bal & ((1u << lane) - 1u)) : -1;
    __syncthreads();
    if (tid == 0) s_base += s_chunk;
    __syncthreads();
  }
  if (tid == 0) send_count[g] = s_base;
}

// ---- dispatch 2: one warp per (token, destination) stores the row into the destination's memory ----
__global__ void __launch_bounds__(256) ep_send_kernel(
    const uint8_t* __restrict__ x, const float* __restrict__ x_scale, const int32_t* __restrict__ topk_ids,
    const float* __restrict__ topk_w, const int32_t* __restrict__ pos, const int32_t* __restrict__ send_count,
    int tokens, int world, int rank, int64_t cap, int step, Peers peers) {
  const int lane = threadIdx.x & 31;
  const int64_t npairs = (int64_t)tokens * world;
  // grid-stride: a CTA fences once, after all of its rows (a system-scope fence after remote stores
  // costs a round trip over NVLink)
  for (int64_t pair = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); pair < npairs;
       pair += (int64_t)gridDim.x * (blockDim.x >> 5)) {  // pair = token * world + dest
    const int p = pos[pair];
    if (p >= 0) {
      const int64_t t = pair / world;
      const int g = (int)(pair - t * world);
      unsigned char* dst = peers.buf[g] + recv_offset() + ((size_t)rank * cap + p) * ROW_BYTES;
      const uint4* src = reinterpret_cast<const uint4*>(x + t * HID);
      uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
      for (int i = 0; i < HID / 16 / 32; ++i) d4[i * 32 + lane] = __ldg(src + i * 32 + lane);
      float* ds = reinterpret_cast<float*>(dst + OFF_SCALES);
      for (int kb = lane; kb < KB1; kb += 32) ds[kb] = x_scale[(int64_t)kb * tokens + t];
      if (lane < TOPK) reinterpret_cast<int32_t*>(dst + OFF_IDS)[lane] = topk_ids[t * TOPK + lane];
      else if (lane < 2 * TOPK) reinterpret_cast<float*>(dst + OFF_W)[lane - TOPK] = topk_w[t * TOPK + lane - TOPK];
    }
  }
  // completion: every CTA fences its stores system-wide, the last one publishes counts and step
  __threadfence_system();
  __syncthreads();
  __shared__ bool s_last;
  Flags* mine = reinterpret_cast<Flags*>(peers.buf[rank]);
  if (threadIdx.x == 0) s_last = (atomicAdd(&mine->done_dispatch, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (threadIdx.x < world) {
      Flags* f = reinterpret_cast<Flags*>(peers.buf[threadIdx.x]);
      f->disp_count[rank] = send_count[threadIdx.x];
      __threadfence_system();
      st_release_sys(&f->disp_step[rank], step);
    }
    if (threadIdx.x == 0) mine->done_dispatch = 0;
  }
}

// ---- experts 1: wait for every source, then read the shipped routing of every received row ------
// Virtual token v = source * cap + position; rows past a source's count do not exist (ids -1).
__global__ void __launch_bounds__(256) ep_recv_route_kernel(
    unsigned char* __restrict__ mybuf, int world, int64_t cap, int step, int32_t* __restrict__ topk_ids,
    float* __restrict__ topk_w, int32_t* __restrict__ pair_pos, int32_t* __restrict__ counts, int local_off,
    int n_local) {
  Flags* f = reinterpret_cast<Flags*>(mybuf);
  __shared__ bool s_ok;
  if (threadIdx.x == 0) {
    bool ok = true;
    for (int s = 0; s < world && ok; ++s) ok = wait_step(&f->disp_step[s], step, &f->error, 50 + s);
    s_ok = ok;
  }
  __syncthreads();
  const int sub = threadIdx.x & 7;                                        // 8 threads per row
  const int64_t v = (int64_t)blockIdx.x * (blockDim.x >> 3) + (threadIdx.x >> 3);
  if (v >= (int64_t)world * cap) return;
  const int s = (int)(v / cap);
  const int64_t i = v - (int64_t)s * cap;
  int id = -1;
  float wgt = 0.f;
  if (s_ok && i < ld_acquire_sys(&f->disp_count[s])) {
    const unsigned char* row = mybuf + recv_offset() + (size_t)v * ROW_BYTES;
    id = reinterpret_cast<const int32_t*>(row + OFF_IDS)[sub];
    wgt = reinterpret_cast<const float*>(row + OFF_W)[sub];
  }
  topk_ids[v * TOPK + sub] = id;
  topk_w[v * TOPK + sub] = wgt;
  pair_pos[v * TOPK + sub] = -1;
  const int le = id - local_off;
  if (id >= 0 && le >= 0 && le < n_local) atomicAdd(&counts[le], 1);
}

// ---- experts 2: permute from the receive area (row stride 7456, scales inside the row) -----------
__global__ void __launch_bounds__(256) ep_permute_kernel(
    const unsigned char* __restrict__ recv, const int32_t* __restrict__ pair_pos, uint8_t* __restrict__ xs,
    float* __restrict__ xs_scale, int64_t vtokens, int64_t cap_pairs) {
  const int lane = threadIdx.x & 31;
  const int64_t slot = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // vtoken*8 + k
  if (slot >= vtokens * TOPK) return;
  const int pos = pair_pos[slot];
  if (pos < 0) return;
  const unsigned char* row = recv + (size_t)(slot / TOPK) * ROW_BYTES;
  const uint4* src = reinterpret_cast<const uint4*>(row);
  uint4* dst = reinterpret_cast<uint4*>(xs + (int64_t)pos * HID);
#pragma unroll
  for (int i = 0; i < HID / 16 / 32; ++i) dst[i * 32 + lane] = src[i * 32 + lane];
  const float* sc = reinterpret_cast<const float*>(row + OFF_SCALES);
  for (int kb = lane; kb < KB1; kb += 32) xs_scale[(int64_t)kb * cap_pairs + pos] = sc[kb];
}

// ---- experts 3: combine a received row's local experts and store the bf16 partial into the SOURCE
//      rank's return area; the last CTA publishes the step number to every source -----------------
__global__ void __launch_bounds__(256) ep_return_kernel(
    const float* __restrict__ y, const int32_t* __restrict__ pair_pos, const float* __restrict__ topk_w,
    const int32_t* __restrict__ topk_ids, int world, int rank, int64_t cap, int step, Peers peers) {
  for (int64_t v = blockIdx.x; v < (int64_t)world * cap; v += gridDim.x) {
  const int s = (int)(v / cap);
  const int64_t i = v - (int64_t)s * cap;
  if (topk_ids[v * TOPK] >= 0) {  // the row exists (ids of missing rows are all -1)
    int pos[TOPK];
    float w[TOPK];
#pragma unroll
    for (int k = 0; k < TOPK; ++k) {
      pos[k] = pair_pos[v * TOPK + k];
      w[k] = topk_w[v * TOPK + k];
    }
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(peers.buf[s] + ret_offset(world, cap)) +
                         ((size_t)rank * cap + i) * HID;
    // eight columns per thread and step: 16-byte stores are what NVLink carries best
    for (int c = threadIdx.x * 8; c < HID; c += 256 * 8) {
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
#pragma unroll
      for (int k = 0; k < TOPK; ++k) {
        if (pos[k] >= 0) {
          const float4 yv = __ldcs(reinterpret_cast<const float4*>(y + (int64_t)pos[k] * HID + c));
          const float4 yu = __ldcs(reinterpret_cast<const float4*>(y + (int64_t)pos[k] * HID + c + 4));
          a.x += yv.x * w[k]; a.y += yv.y * w[k]; a.z += yv.z * w[k]; a.w += yv.w * w[k];
          b.x += yu.x * w[k]; b.y += yu.y * w[k]; b.z += yu.z * w[k]; b.w += yu.w * w[k];
        }
      }
      uint4 pk;
      pk.x = ako::pack_bf16x2(a.x, a.y);
      pk.y = ako::pack_bf16x2(a.z, a.w);
      pk.z = ako::pack_bf16x2(b.x, b.y);
      pk.w = ako::pack_bf16x2(b.z, b.w);
      *reinterpret_cast<uint4*>(out + c) = pk;
    }
  }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ bool s_last;
  Flags* mine = reinterpret_cast<Flags*>(peers.buf[rank]);
  if (threadIdx.x == 0) s_last = (atomicAdd(&mine->done_return, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (threadIdx.x < world) st_release_sys(&reinterpret_cast<Flags*>(peers.buf[threadIdx.x])->comb_step[rank], step);
    if (threadIdx.x == 0) mine->done_return = 0;
  }
}

// ---- finish: wait for every expert rank, then out[t] = bf16( sum over ranks, ascending, fp32 ) -----
__global__ void __launch_bounds__(256) ep_finish_kernel(
    unsigned char* __restrict__ mybuf, const int32_t* __restrict__ pos, __nv_bfloat16* __restrict__ out, int world,
    int64_t cap, int step) {
  Flags* f = reinterpret_cast<Flags*>(mybuf);
  __shared__ bool s_ok;
  if (threadIdx.x == 0) {
    bool ok = true;
    for (int g = 0; g < world && ok; ++g) ok = wait_step(&f->comb_step[g], step, &f->error, 60 + g);
    s_ok = ok;
  }
  __syncthreads();
  const int64_t t = blockIdx.x;
  const __nv_bfloat16* ret = reinterpret_cast<const __nv_bfloat16*>(mybuf + ret_offset(world, cap));
  int p[MAX_WORLD];
#pragma unroll
  for (int g = 0; g < MAX_WORLD; ++g) p[g] = (g < world && s_ok) ? pos[t * world + g] : -1;
  for (int c = threadIdx.x * 8; c < HID; c += 256 * 8) {
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int g = 0; g < MAX_WORLD; ++g) {
      if (p[g] < 0) continue;
      const uint4 v = *reinterpret_cast<const uint4*>(ret + ((size_t)g * cap + p[g]) * HID + c);
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[2 * i] += ako::bf16_lo(w[i]);
        a[2 * i + 1] += ako::bf16_hi(w[i]);
      }
    }
    uint4 o;
    uint32_t* q = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = ako::pack_bf16x2(a[2 * i], a[2 * i + 1]);
    *reinterpret_cast<uint4*>(out + t * HID + c) = o;
  }
}

}  // namespace ep
