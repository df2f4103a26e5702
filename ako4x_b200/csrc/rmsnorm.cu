// RMSNorm over rows of 128 bf16 values (256 bytes per row). HBM-bound: 512 bytes of traffic per
// row. Sixteen lanes own one row (one 16-byte vector each), so a warp instruction moves two
// adjacent rows = 512 contiguous bytes; each thread keeps UNROLL such loads in flight.
#include "common.cuh"

namespace {

constexpr int kHidden = 128;

template <int UNROLL>
__global__ void rmsnorm_h128_kernel(const uint4* __restrict__ x, const uint4* __restrict__ w,
                                    uint4* __restrict__ y, int64_t rows) {
  const int lane16 = threadIdx.x & 15;
  // weight slice of this lane, as fp32
  float wf[8];
  {
    uint4 wv = __ldg(w + lane16);
    const uint32_t* p = reinterpret_cast<const uint32_t*>(&wv);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      wf[2 * i] = ako::bf16_lo(p[i]);
      wf[2 * i + 1] = ako::bf16_hi(p[i]);
    }
  }
  const int64_t rows_per_block = (int64_t)(blockDim.x / 16) * UNROLL;
  const int64_t row0 = (int64_t)blockIdx.x * rows_per_block + (threadIdx.x >> 4);
  const int stride_rows = blockDim.x / 16;

  uint4 v[UNROLL];
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    int64_t r = row0 + (int64_t)u * stride_rows;
    if (r < rows) v[u] = __ldcs(x + r * 16 + lane16);
    else v[u] = make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    const uint32_t* p = reinterpret_cast<const uint32_t*>(&v[u]);
    float f[8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = ako::bf16_lo(p[i]);
      f[2 * i + 1] = ako::bf16_hi(p[i]);
      ss = fmaf(f[2 * i], f[2 * i], ss);
      ss = fmaf(f[2 * i + 1], f[2 * i + 1], ss);
    }
#pragma unroll
    for (int m = 8; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
    const float inv = rsqrtf(ss * (1.0f / kHidden) + 1e-6f);
    uint4 o;
    uint32_t* q = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      q[i] = ako::pack_bf16x2((f[2 * i] * inv) * wf[2 * i], (f[2 * i + 1] * inv) * wf[2 * i + 1]);
    int64_t r = row0 + (int64_t)u * stride_rows;
    if (r < rows) __stcs(y + r * 16 + lane16, o);
  }
}

}  // namespace

extern "C" int ako4x_rmsnorm_h128(const void* x, const void* weight, void* y, int64_t rows,
                                  void* stream) {
  if (rows < 0) return AKO4X_EINVAL;
  if (rows == 0) return AKO4X_OK;
  if (!x || !weight || !y) return AKO4X_EINVAL;
  if (((uintptr_t)x | (uintptr_t)weight | (uintptr_t)y) & 15) return AKO4X_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  const uint4* xp = (const uint4*)x;
  const uint4* wp = (const uint4*)weight;
  uint4* yp = (uint4*)y;
  // Few rows: one row pair per warp so rows spread over SMs. Many rows: 4 loads in flight per
  // thread and 256-thread blocks (64 rows per block).
  if (rows <= 2048) {
    int threads = 32;
    int64_t rpb = 2;
    rmsnorm_h128_kernel<1><<<(unsigned)ako::cdiv(rows, rpb), threads, 0, st>>>(xp, wp, yp, rows);
  } else if (rows <= 65536) {
    int threads = 128;
    int64_t rpb = (threads / 16) * 2;
    rmsnorm_h128_kernel<2><<<(unsigned)ako::cdiv(rows, rpb), threads, 0, st>>>(xp, wp, yp, rows);
  } else {
    int threads = 256;
    int64_t rpb = (threads / 16) * 4;
    rmsnorm_h128_kernel<4><<<(unsigned)ako::cdiv(rows, rpb), threads, 0, st>>>(xp, wp, yp, rows);
  }
  AKO_CHECK_LAUNCH();
  return AKO4X_OK;
}

extern "C" int ako4x_abi_version(void) { return 1; }
