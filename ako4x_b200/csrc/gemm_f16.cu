// Dense GEMM C[M, N] = A[M, K] * B[N, K]^T, fp16 (or bf16) operands, fp32 accumulation, output in
// the operand type: the operator family reference/gemm-n2048-k4096 (N = 2048, K = 4096, M from 1
// to 16 294; the reference's campaign ended with cuBLAS as its best implementation, README.md of
// that folder). Hand-written for sm_100a:
//   * persistent CTAs, one per SM, over output tiles of 128 rows x BN columns (BN = 256, 128 or 32
//     chosen by how many tiles M gives), n fastest so that the CTAs sharing an A tile run side by
//     side and A crosses HBM once (B, 16 MB, stays in L2);
//   * a TMA producer warp fills a ring of K = 64 slices (128-byte-swizzled boxes of A and B);
//   * one thread issues tcgen05.mma kind::f16 (M128 x BN x K16) into one of TWO TMEM accumulators,
//     the whole K dimension per tile, so no partial sums leave TMEM;
//   * four epilogue warps drain the other accumulator (tcgen05.ld, cast, 64-byte stores per row)
//     while the next tile's MMAs run.
// Small M: a tile's K loop is 256 MMAs whatever its width and an M128 x N32 x K16 MMA takes about
// 80 cycles, so one CTA per tile needs 11 us (22-24 us per call, and keeping 64 KB instead of 32 KB
// of B in flight per CTA changed nothing). With a workspace the K dimension is split over up to 8
// CTAs per tile and a second kernel sums the fp32 partial products (gemm_plan below).
// Every wait is bounded; a wait that gives up records its code in the status word below and the
// CTA unwinds through the common exit that frees TMEM.
#include "common.cuh"
#include "tcgen05.cuh"
#include "tma_host.cuh"

namespace {

constexpr int G_BM = 128, G_BK_BYTES = 128, G_THREADS = 192;
constexpr int G_A_BYTES = G_BM * G_BK_BYTES;   // 16 KB per stage
enum { kErrGLoad = 71, kErrGMma = 72, kErrGAcc = 73, kErrGEpi = 74 };

__device__ int g_gemm_status;

template <int BN>
struct GemmCfg {
  static constexpr int B_BYTES = BN * G_BK_BYTES;
  static constexpr int STAGE_BYTES = G_A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128) ? 6 : 8;
  static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024;
};

__host__ __device__ constexpr uint32_t idesc_f16(int m, int n, bool bf16) {
  return (1u << 4) | (bf16 ? ((1u << 7) | (1u << 10)) : 0u) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

struct GemmArgs {
  void* c;
  float* partial;   // split-K: fp32 partial products [split][m][n]; unused when splits == 1
  int m, n, k;
  int a_box_rows;   // rows of A one TMA box brings (128, or fewer when M is small)
  int splits;       // CTAs that share one output tile, each over k / splits of the reduction
};

template <int BN, bool BF16>
__global__ void __launch_bounds__(G_THREADS, 1)
gemm_f16_tc_kernel(GemmArgs p, const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr uint32_t IDESC = idesc_f16(G_BM, BN, BF16);
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t s_full[STAGES];
  __shared__ __align__(8) uint64_t s_empty[STAGES];
  __shared__ __align__(8) uint64_t s_acc_full[2];
  __shared__ __align__(8) uint64_t s_acc_empty[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_err;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t smem_base = (ako::smem_u32(smem_raw) + 1023u) & ~1023u;
  if (tid == 0) {
    s_err = 0;
    for (int s = 0; s < STAGES; ++s) {
      ako::tc::mbar_init(ako::smem_u32(&s_full[s]), 1);
      ako::tc::mbar_init(ako::smem_u32(&s_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ako::tc::mbar_init(ako::smem_u32(&s_acc_full[b]), 1);
      ako::tc::mbar_init(ako::smem_u32(&s_acc_empty[b]), 4);   // one elected arrival per epilogue warp
    }
    ako::tc::mbar_init_fence();
  }
  if (warp == 4) ako::tc::tmem_alloc(ako::smem_u32(&s_tmem_base), Cfg::TMEM_COLS);
  ako::tc::fence_before_thread_sync();
  __syncthreads();
  ako::tc::fence_after_thread_sync();
  const uint32_t tmem_base = s_tmem_base;

  // work item = (output tile, K split), the split fastest
  const int m_tiles = (p.m + G_BM - 1) / G_BM, n_tiles = p.n / BN;
  const int total_tiles = m_tiles * n_tiles * p.splits;
  const int nkb = p.k / 64 / p.splits;
  // bytes one stage receives: A brings a_box_rows rows, B all BN
  const uint32_t stage_tx = (uint32_t)p.a_box_rows * G_BK_BYTES + (uint32_t)Cfg::B_BYTES;

  if (warp == 4) {
    // ================================ TMA producer =============================================
    if (lane == 0) {
      ako::tc::tma_prefetch_desc(&tm_a);
      ako::tc::tma_prefetch_desc(&tm_b);
      int g = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const int ks = tile % p.splits, ot = tile / p.splits;
        const int mt = ot / n_tiles, nt = ot % n_tiles;
        for (int kb0 = 0; kb0 < nkb; ++kb0, ++g) {
          const int kb = ks * nkb + kb0;
          const int stage = g % STAGES;
          const uint32_t ph = (uint32_t)((g / STAGES) & 1);
          if (!ako::tc::mbar_wait(ako::smem_u32(&s_empty[stage]), ph ^ 1u, &s_err, kErrGLoad)) { ok = false; break; }
          const uint32_t bar = ako::smem_u32(&s_full[stage]);
          const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES;
          ako::tc::mbar_arrive_expect_tx(bar, stage_tx);
          ako::tc::tma_load_2d(sa, &tm_a, kb * G_BK_BYTES, mt * G_BM, bar);
          ako::tc::tma_load_2d(sa + G_A_BYTES, &tm_b, kb * G_BK_BYTES, nt * BN, bar);
        }
      }
    }
  } else if (warp == 5) {
    // ================================ MMA issuer ===============================================
    if (lane == 0) {
      const uint32_t a_lo0 = ako::tc::smem_desc_lo(smem_base);
      const uint32_t b_lo0 = ako::tc::smem_desc_lo(smem_base + G_A_BYTES);
      int g = 0, lt = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++lt) {
        const int buf = lt & 1;
        if (!ako::tc::mbar_wait(ako::smem_u32(&s_acc_empty[buf]), (uint32_t)(((lt >> 1) & 1) ^ 1), &s_err, kErrGAcc)) break;
        const uint32_t d = tmem_base + buf * BN;
        for (int kb = 0; kb < nkb; ++kb, ++g) {
          const int stage = g % STAGES;
          if (!ako::tc::mbar_wait(ako::smem_u32(&s_full[stage]), (uint32_t)((g / STAGES) & 1), &s_err, kErrGMma)) { ok = false; break; }
          ako::tc::fence_after_thread_sync();
          const uint32_t a_lo = a_lo0 + stage * (Cfg::STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + stage * (Cfg::STAGE_BYTES >> 4);
          ako::tc::mma_bf16_lohi(d, a_lo, b_lo, IDESC, kb > 0 ? 1u : 0u);
          ako::tc::mma_bf16_lohi(d, a_lo + 2, b_lo + 2, IDESC, 1u);
          ako::tc::mma_bf16_lohi(d, a_lo + 4, b_lo + 4, IDESC, 1u);
          ako::tc::mma_bf16_lohi(d, a_lo + 6, b_lo + 6, IDESC, 1u);
          ako::tc::mma_commit(ako::smem_u32(&s_empty[stage]));
        }
        if (ok) ako::tc::mma_commit(ako::smem_u32(&s_acc_full[buf]));
      }
    }
  } else {
    // ================================ epilogue warps ===========================================
    const int row_in_tile = 32 * warp + lane;   // TMEM lane = accumulator row
    int lt = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++lt) {
      const int ks = tile % p.splits, ot = tile / p.splits;
      const int mt = ot / n_tiles, nt = ot % n_tiles;
      const int buf = lt & 1;
      if (!ako::tc::mbar_wait_warp(ako::smem_u32(&s_acc_full[buf]), (uint32_t)((lt >> 1) & 1), &s_err, kErrGEpi)) break;
      ako::tc::fence_after_thread_sync();
      const int row = mt * G_BM + row_in_tile;
      const uint32_t taddr = tmem_base + ((uint32_t)(32 * warp) << 16) + buf * BN;
      uint16_t* crow = reinterpret_cast<uint16_t*>(p.c) + (int64_t)row * p.n + nt * BN;
      float* prow = p.partial + ((int64_t)ks * p.m + row) * p.n + nt * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        float v[32];
        ako::tc::tmem_ld32(taddr + c, v);
        ako::tc::tmem_ld_wait_regs(v);
        if (row < p.m && p.splits > 1) {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(prow + c + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else if (row < p.m) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              if (BF16) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(v[j + 2 * k], v[j + 2 * k + 1]);
                w[k] = *reinterpret_cast<const uint32_t*>(&h);
              } else {
                const __half2 h = __floats2half2_rn(v[j + 2 * k], v[j + 2 * k + 1]);
                w[k] = *reinterpret_cast<const uint32_t*>(&h);
              }
            }
            *reinterpret_cast<uint4*>(crow + c + j) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      ako::tc::fence_before_thread_sync();
      __syncwarp();
      if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&s_acc_empty[buf]));
    }
  }

  // ================================ common exit ================================================
  ako::tc::fence_before_thread_sync();
  __syncthreads();
  if (tid == 0 && s_err != 0) atomicCAS(&g_gemm_status, 0, s_err);
  if (warp == 4) {
    ako::tc::fence_after_thread_sync();
    ako::tc::tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// Split-K second step: C = cast(sum over splits, in split order, of the fp32 partials). Eight
// values per thread; launched with programmatic dependent launch behind the GEMM.
template <bool BF16>
__global__ void __launch_bounds__(256) gemm_splitk_reduce_kernel(const float* __restrict__ partial, void* __restrict__ c,
                                                                 int64_t mn, int splits) {
  ako::pdl_wait();
  const int64_t i = ((int64_t)blockIdx.x * 256 + threadIdx.x) * 8;
  if (i >= mn) return;
  float acc[8];
  {
    const float4 x = __ldcs(reinterpret_cast<const float4*>(partial + i));
    const float4 y = __ldcs(reinterpret_cast<const float4*>(partial + i + 4));
    acc[0] = x.x; acc[1] = x.y; acc[2] = x.z; acc[3] = x.w; acc[4] = y.x; acc[5] = y.y; acc[6] = y.z; acc[7] = y.w;
  }
  for (int s = 1; s < splits; ++s) {
    const float4 x = __ldcs(reinterpret_cast<const float4*>(partial + s * mn + i));
    const float4 y = __ldcs(reinterpret_cast<const float4*>(partial + s * mn + i + 4));
    acc[0] += x.x; acc[1] += x.y; acc[2] += x.z; acc[3] += x.w; acc[4] += y.x; acc[5] += y.y; acc[6] += y.z; acc[7] += y.w;
  }
  uint32_t w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (BF16) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
      w[k] = *reinterpret_cast<const uint32_t*>(&h);
    } else {
      const __half2 h = __floats2half2_rn(acc[2 * k], acc[2 * k + 1]);
      w[k] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
  *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(c) + i) = make_uint4(w[0], w[1], w[2], w[3]);
}

template <int BN, bool BF16>
int launch_gemm(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int splits, float* partial,
                cudaStream_t st) {
  using Cfg = GemmCfg<BN>;
  const int a_box_rows = (m >= G_BM) ? G_BM : (int)((m + 7) / 8 * 8);
  CUtensorMap tm_a, tm_b;
  if (!ako::tma::byte_matrix_map(&tm_a, a, (uint64_t)m, (uint64_t)k * 2, (uint32_t)a_box_rows) ||
      !ako::tma::byte_matrix_map(&tm_b, b, (uint64_t)n, (uint64_t)k * 2, (uint32_t)BN))
    return AKO4X_ELAUNCH;
  if (!ako::ensure_dynamic_smem<gemm_f16_tc_kernel<BN, BF16>>((int)Cfg::SMEM)) return AKO4X_ELAUNCH;
  GemmArgs p;
  p.c = c;
  p.m = (int)m;
  p.n = (int)n;
  p.k = (int)k;
  p.a_box_rows = a_box_rows;
  p.splits = splits;
  p.partial = partial;
  const int64_t tiles = ((m + G_BM - 1) / G_BM) * (n / BN) * splits;
  const int grid = (int)std::min<int64_t>(tiles, ako::sm_count());
  gemm_f16_tc_kernel<BN, BF16><<<grid, G_THREADS, Cfg::SMEM, st>>>(p, tm_a, tm_b);
  AKO_CHECK_LAUNCH();
  if (splits > 1) {
    const int64_t mn = m * n;
    const unsigned blocks = (unsigned)((mn / 8 + 255) / 256);
    if (ako::launch_pdl(true, gemm_splitk_reduce_kernel<BF16>, dim3(blocks), dim3(256), 0, st, (const float*)partial, c,
                        mn, splits) != cudaSuccess)
      return AKO4X_ELAUNCH;
  }
  return AKO4X_OK;
}

// Tile width and K split by how many work items the GPU gets. Full-width tiles (256 columns)
// without a split once they fill three quarters of the SMs. Below that a tile's K loop (256 MMAs
// whatever the tile width) is what a call waits for: tiles of 128 columns, and K cut into 2, 4 or 8
// pieces handled by different CTAs (summed by a second kernel) until there are 128 work items.
// Measured, whole call, cold L2: M = 16: 15.4 us (unsplit 26.6), M = 128: 17.4, M = 256: 19.5,
// M = 512: 23.5, M = 969: 30.7 (no split; 256 columns x 2 splits: 29.7).
struct GemmPlan {
  int bn, splits;
};
inline GemmPlan gemm_plan(int64_t m, int64_t n, int64_t k, bool have_workspace) {
  const int64_t mt = (m + G_BM - 1) / G_BM;
  const int sms = ako::sm_count();
  if (mt * (n / 256) * 4 >= 3 * sms) return {256, 1};
  if (!have_workspace) return {(mt * (n / 128) * 4 >= 3 * sms) ? 128 : 32, 1};
  int s = 1;
  while (s < 8 && mt * (n / 128) * s < 128 && (k / 64) % (2 * s) == 0) s *= 2;
  return {128, s};
}

}  // namespace

extern "C" size_t ako4x_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k) {
  if (m <= 0 || n <= 0 || k <= 0 || n % 256 != 0 || k % 64 != 0) return 0;
  const GemmPlan pl = gemm_plan(m, n, k, true);
  return pl.splits > 1 ? (size_t)pl.splits * (size_t)m * (size_t)n * sizeof(float) : 0;
}

static int gemm_entry(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int is_bf16,
                      void* workspace, size_t workspace_bytes, void* stream) {
  if (m < 0 || n <= 0 || k <= 0 || m > (1 << 24)) return AKO4X_EINVAL;
  if (n % 256 != 0 || k % 64 != 0) return AKO4X_EUNSUPPORTED_SHAPE;
  if (m == 0) return AKO4X_OK;
  if (!a || !b || !c) return AKO4X_EINVAL;
  if (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)workspace) & 15) return AKO4X_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  const GemmPlan pl = gemm_plan(m, n, k, workspace != nullptr);
  if (pl.splits > 1 && workspace_bytes < (size_t)pl.splits * (size_t)m * (size_t)n * sizeof(float)) return AKO4X_EWORKSPACE;
  float* part = (float*)workspace;
  if (is_bf16) {
    if (pl.bn == 256) return launch_gemm<256, true>(a, b, c, m, n, k, pl.splits, part, st);
    if (pl.bn == 128) return launch_gemm<128, true>(a, b, c, m, n, k, pl.splits, part, st);
    return launch_gemm<32, true>(a, b, c, m, n, k, 1, part, st);
  }
  if (pl.bn == 256) return launch_gemm<256, false>(a, b, c, m, n, k, pl.splits, part, st);
  if (pl.bn == 128) return launch_gemm<128, false>(a, b, c, m, n, k, pl.splits, part, st);
  return launch_gemm<32, false>(a, b, c, m, n, k, 1, part, st);
}

extern "C" int ako4x_gemm_f16_nt(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                                 int is_bf16, void* stream) {
  return gemm_entry(a, b, c, m, n, k, is_bf16, nullptr, 0, stream);
}

extern "C" int ako4x_gemm_f16_nt_ws(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                                    int is_bf16, void* workspace, size_t workspace_bytes, void* stream) {
  return gemm_entry(a, b, c, m, n, k, is_bf16, workspace, workspace_bytes, stream);
}

// Status word of the GEMM kernels: 0, or the code of the first bounded wait that gave up (71
// producer, 72 issuer on operands, 73 issuer on an accumulator, 74 epilogue). Synchronises the
// device; meant for tests and post-mortems.
extern "C" int ako4x_gemm_device_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)) != cudaSuccess) return AKO4X_ELAUNCH;
  return v;
}
