// The grouped FP8 block-scale GEMM as a CTA PAIR (tcgen05 cta_group::2), included by moe.cu after
// moe_gemm_tc.cuh (it reuses that file's constants, tile conventions and promotion code).
//
// What bounded the one-CTA kernel: a 128 x 256 tile needs 48 KB of operands per K block (16 KB of
// activations, 32 KB of weights), and an SM draws about 64 B/clk from L2: 750 cycles against 512
// cycles of MMA. Two CTAs of a cluster that share a 256 x 256 tile each load their own 128 rows of
// activations and HALF of the weight rows (32 KB per CTA and K block); the MMA, issued by the even
// CTA for both, reads the weight halves from both CTAs' shared memory and writes each CTA's 128
// accumulator rows into that CTA's TMEM. Promotion, SwiGLU and the stores are per CTA, as before.
//   - tile list: (expert, n-tile, PAIR of m-tiles); CTA r of the pair owns m-tile 2*mp + r (an expert
//     with an odd number of m-tiles gives its last pair an empty second half: rows <= 0);
//   - every CTA's producer thread TMA-loads into its own ring; completion is counted on the EVEN
//     CTA's mbarrier (cp.async.bulk.tensor ... .cta_group::2, no multicast);
//   - tcgen05.commit with a CTA mask frees the stage in both CTAs and publishes the accumulator to
//     both; the promotion warps of both CTAs arrive on the even CTA's "accumulator free" barrier;
//   - TMEM is allocated and freed with cta_group::2 by one warp of EACH CTA, with cluster barriers
//     around set-up and tear-down. Every wait is bounded as in the one-CTA kernel.
#pragma once

constexpr int T2_STAGES = 6;
constexpr int T2_B_BYTES = 128 * 128;                    // this CTA's half of the weight tile
constexpr int T2_STAGE_BYTES = TC_A_BYTES + T2_B_BYTES;  // 32 KB
constexpr int T2_SMEM = T2_STAGES * T2_STAGE_BYTES + TC_EXTRA_BYTES + 1024;

__device__ __forceinline__ uint32_t t2_cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ void t2_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// shared::cluster address of `addr` (a shared::cta address of this CTA's layout) in CTA `rank`
__device__ __forceinline__ uint32_t t2_mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// Arrival on a barrier of the pair's even CTA. Relaxed: what the barrier orders here is TMEM traffic
// (the tcgen05.ld of this thread's warp against the next MMA into the buffer), which the
// tcgen05 fences around the arrival and the wait take care of; a release at cluster scope measured
// 1 500 - 2 400 cycles per arrival, once per warp and K block.
__device__ __forceinline__ void t2_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void t2_tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(dst_smem), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void t2_tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols) : "memory");
}
// 2-D tiled load into this CTA's shared memory, bytes counted on the mbarrier at cluster address `bar`
__device__ __forceinline__ void t2_tma_load_2d(uint32_t dst, const void* tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::
          "r"(dst),
      "l"(tmap), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
template <bool ACCUMULATE>
__device__ __forceinline__ void t2_mma_f8(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
  asm volatile(
      "{\n.reg .b64 da, db;\n.reg .pred p;\n"
      "mov.b64 da, {%1, %4};\n"
      "mov.b64 db, {%2, %4};\n"
      "setp.ne.b32 p, %5, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], da, db, %3, p;\n}\n" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(ako::tc::kSmemDescHiSw128), "n"(ACCUMULATE ? 1 : 0)
      : "memory");
}
// arrives (once) on the mbarrier at the same shared-memory offset in both CTAs of the pair
__device__ __forceinline__ void t2_commit_both(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::"r"(bar),
               "h"((unsigned short)3)
               : "memory");
}

// tile = (expert, n-tile, m-tile pair), m-pair fastest; CTA `crank` owns m-tile 2 * mp + crank
template <int NT_TILES>
__device__ __forceinline__ TileInfo t2_tile_info(const GemmParams& p, const int* s_cum, int tile, int crank) {
  TileInfo ti;
  int e = 0;
  while (s_cum[e + 1] * NT_TILES <= tile) ++e;
  const int mp_e = s_cum[e + 1] - s_cum[e];
  const int rem = tile - s_cum[e] * NT_TILES;
  const int mt = 2 * (rem % mp_e) + crank;
  ti.e = e;
  ti.nt = rem / mp_e;
  ti.row0 = p.offsets[e] + mt * TC_BM;
  ti.rows = min(TC_BM, p.counts[e] - mt * TC_BM);   // <= 0 for the empty half of an odd last pair
  return ti;
}

template <int WHICH>
__global__ void __launch_bounds__(TC_THREADS, 1)
moe_gemm_tc2_kernel(GemmParams p, const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b) {
  constexpr int NKB = (WHICH == 1) ? KB1 : KB2;
  constexpr int NT_TILES = (WHICH == 1) ? (INTER / 128) : (HID / TC_BN);
  constexpr uint32_t IDESC = ako::tc::idesc_e4m3_f32(2 * TC_BM, TC_BN);   // M = 256 over the pair

  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t s_full[T2_STAGES];
  __shared__ __align__(8) uint64_t s_empty[T2_STAGES];
  __shared__ __align__(8) uint64_t s_acc_full[2];
  __shared__ __align__(8) uint64_t s_acc_empty[2];
  __shared__ __align__(8) uint64_t s_xchg[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_cum[MAX_LOCAL + 1];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int crank = (int)t2_cluster_ctarank();
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const uint32_t smem_base = (ako::smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* extra = smem_raw + (smem_base - ako::smem_u32(smem_raw)) + T2_STAGES * T2_STAGE_BYTES;
  float (*s_amax)[2][TC_BM] = reinterpret_cast<float (*)[2][TC_BM]>(extra);

  if (tid == 0) {
    for (int s = 0; s < T2_STAGES; ++s) {
      ako::tc::mbar_init(ako::smem_u32(&s_full[s]), 1);     // used in the even CTA: its own arrive.expect_tx
      ako::tc::mbar_init(ako::smem_u32(&s_empty[s]), 1);    // one commit arrival, in each CTA
    }
    for (int b = 0; b < 2; ++b) {
      ako::tc::mbar_init(ako::smem_u32(&s_acc_full[b]), 1);
      ako::tc::mbar_init(ako::smem_u32(&s_acc_empty[b]), 2 * TC_WORKERS / 32);  // even CTA: warps of both CTAs
      ako::tc::mbar_init(ako::smem_u32(&s_xchg[b]), TC_WORKERS / 32);
    }
    ako::tc::mbar_init_fence();
  }
  if (warp == 8) t2_tmem_alloc(ako::smem_u32(&s_tmem_base), TC_TMEM_COLS);
  ako::pdl_wait();
  ako::pdl_trigger();
  if (tid == 0) {
    int acc = 0;
    for (int e = 0; e < p.n_local; ++e) {
      s_cum[e] = acc;
      acc += ((p.counts[e] + TC_BM - 1) / TC_BM + 1) / 2;   // m-tile pairs
    }
    s_cum[p.n_local] = acc;
  }
  ako::tc::fence_before_thread_sync();
  __syncthreads();
  t2_cluster_sync();   // both CTAs' barriers are initialised before anybody signals across
  ako::tc::fence_after_thread_sync();
  const uint32_t tmem_base = s_tmem_base;
  const int total_tiles = s_cum[p.n_local] * NT_TILES;
  // the even CTA's barriers, as seen from this CTA
  const uint32_t acc_empty_leader0 = t2_mapa(ako::smem_u32(&s_acc_empty[0]), 0);
  const uint32_t acc_empty_leader1 = t2_mapa(ako::smem_u32(&s_acc_empty[1]), 0);

  if (warp >= 10) {
    ako::tc::reg_dec<TC_REGS_OTHER>();  // donor warps
  } else if (warp == 9) {
    // ================================ TMA producer (each CTA, its own ring) =====================
    ako::tc::reg_dec<TC_REGS_OTHER>();
    if (lane == 0) {
      ako::tc::tma_prefetch_desc(&tm_a);
      ako::tc::tma_prefetch_desc(&tm_b);
      int g = 0;
      bool ok = true;
      for (int tile = pair_id; ok && tile < total_tiles; tile += num_pairs) {
        const TileInfo ti = t2_tile_info<NT_TILES>(p, s_cum, tile, crank);
        for (int kb = 0; kb < NKB; ++kb, ++g) {
          const int stage = g % T2_STAGES;
          const uint32_t ph = (g / T2_STAGES) & 1;
          if (!ako::tc::mbar_wait(ako::smem_u32(&s_empty[stage]), ph ^ 1u, p.error, kErrLoad)) { ok = false; break; }
          const uint32_t sa = smem_base + stage * T2_STAGE_BYTES;
          const uint32_t sb = sa + TC_A_BYTES;
          const uint32_t bar = t2_mapa(ako::smem_u32(&s_full[stage]), 0);
          // the even CTA announces the bytes of BOTH CTAs; the odd CTA's copies only count down
          if (crank == 0) ako::tc::mbar_arrive_expect_tx(ako::smem_u32(&s_full[stage]), 2 * T2_STAGE_BYTES);
          t2_tma_load_2d(sa, &tm_a, kb * 128, ti.row0, bar);
          if (WHICH == 1) {
            // rows of the 256-row weight tile: [g1 0-63 | g2 0-63 | g1 64-127 | g2 64-127]; this CTA
            // loads the two 64-row boxes of its half
            const int wr = ti.e * (2 * INTER) + ti.nt * 128 + 64 * crank;
            t2_tma_load_2d(sb, &tm_b, kb * 128, wr, bar);
            t2_tma_load_2d(sb + 64 * 128, &tm_b, kb * 128, wr + INTER, bar);
          } else {
            t2_tma_load_2d(sb, &tm_b, (kb & 15) * 128, ti.e * HID + ti.nt * TC_BN + 128 * crank, bar);
          }
        }
      }
    }
  } else if (warp == 8) {
    // ================================ MMA issuer (even CTA, for the pair) ========================
    ako::tc::reg_dec<TC_REGS_OTHER>();
    if (lane == 0 && crank == 0) {
      const uint32_t a_lo0 = ako::tc::smem_desc_lo(smem_base);
      const uint32_t b_lo0 = ako::tc::smem_desc_lo(smem_base + TC_A_BYTES);
      int g = 0, stage = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = pair_id; ok && tile < total_tiles; tile += num_pairs) {
        for (int kb = 0; kb < NKB; ++kb, ++g) {
          const int buf = g & 1;
          const uint32_t aph = (g >> 1) & 1;
          if (!ako::tc::mbar_wait(ako::smem_u32(&s_acc_empty[buf]), aph ^ 1u, p.error, kErrMmaAcc)) { ok = false; break; }
          if (!ako::tc::mbar_wait(ako::smem_u32(&s_full[stage]), ph, p.error, kErrMmaFull)) { ok = false; break; }
          ako::tc::fence_after_thread_sync();
          const uint32_t a_lo = a_lo0 + stage * (T2_STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + stage * (T2_STAGE_BYTES >> 4);
          const uint32_t d = tmem_base + buf * TC_BN;
          t2_mma_f8<false>(d, a_lo, b_lo, IDESC);
          t2_mma_f8<true>(d, a_lo + 2, b_lo + 2, IDESC);
          t2_mma_f8<true>(d, a_lo + 4, b_lo + 4, IDESC);
          t2_mma_f8<true>(d, a_lo + 6, b_lo + 6, IDESC);
          t2_commit_both(ako::smem_u32(&s_empty[stage]));
          t2_commit_both(ako::smem_u32(&s_acc_full[buf]));
          if (++stage == T2_STAGES) { stage = 0; ph ^= 1u; }
        }
      }
    }
  } else {
    // ================================ promotion threads =========================================
    ako::tc::reg_inc<TC_REGS_WORKER>();
    const int half = warp >> 2;        // which 128 accumulator columns
    const int q = warp & 3;            // TMEM lane quarter
    const int r = 32 * q + lane;       // accumulator row of this thread
    bool ok = true;
    int g = 0;
    int tcount = 0;
    for (int tile = pair_id; ok && tile < total_tiles; tile += num_pairs, ++tcount) {
      const TileInfo ti = t2_tile_info<NT_TILES>(p, s_cum, tile, crank);
      const int tile_par = tcount & 1;
      const bool live = r < ti.rows;
      const float* asp = p.a_scale + (live ? ti.row0 + r : 0);
      const float* bsp0;
      const float* bsp1;
      if (WHICH == 1) {
        bsp0 = p.w_scale + ((int64_t)ti.e * (2 * INTER / 128) + ti.nt) * KB1;
        bsp1 = bsp0 + (int64_t)(INTER / 128) * KB1;
      } else {
        bsp0 = p.w_scale + ((int64_t)ti.e * (HID / 128) + ti.nt * 2 + half) * (INTER / 128);
        bsp1 = bsp0;
      }
      float acc[128];
#pragma unroll
      for (int j = 0; j < 128; ++j) acc[j] = 0.f;
      float sa_n = live ? __ldg(asp) : 0.f;
      float b0_n = __ldg(bsp0), b1_n = __ldg(bsp1);
#pragma unroll 1
      for (int kb = 0; kb < NKB; ++kb, ++g) {
        float sa = sa_n;
        const float s0 = sa * b0_n, s1 = sa * b1_n;
        if (kb + 1 < NKB) {
          const int nk = (WHICH == 1) ? (kb + 1) : ((kb + 1) & 15);
          sa_n = live ? __ldg(asp + (int64_t)nk * p.a_scale_stride) : 0.f;
          b0_n = __ldg(bsp0 + nk);
          b1_n = __ldg(bsp1 + nk);
        }
        const int buf = g & 1;
        const uint32_t aph = (g >> 1) & 1;
        if (!ako::tc::mbar_wait(ako::smem_u32(&s_acc_full[buf]), aph, p.error, kErrEpilogue)) { ok = false; break; }
        ako::tc::fence_after_thread_sync();
        const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + buf * TC_BN + half * 128;
        float v0[32], v1[32];
        ako::tc::tmem_ld32(taddr, v0);
        ako::tc::tmem_ld32(taddr + 32, v1);
        ako::tc::tmem_ld_wait_regs(v0);
        ako::tc::tmem_ld_wait_regs(v1);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          acc[j] = fmaf(v0[j], s0, acc[j]);
          acc[32 + j] = fmaf(v1[j], s0, acc[32 + j]);
        }
        ako::tc::tmem_ld32(taddr + 64, v0);
        ako::tc::tmem_ld32(taddr + 96, v1);
        ako::tc::tmem_ld_wait_regs(v0);
        ako::tc::tmem_ld_wait_regs(v1);
        ako::tc::fence_before_thread_sync();
        __syncwarp();
        if (lane == 0) t2_arrive_cluster(buf ? acc_empty_leader1 : acc_empty_leader0);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          acc[64 + j] = fmaf(v0[j], s1, acc[64 + j]);
          acc[96 + j] = fmaf(v1[j], s1, acc[96 + j]);
        }
      }
      if (!ok) break;

      if (WHICH == 2) {
        // A thread holds 128 columns of ONE row; stored directly, a warp's instruction would touch
        // 32 rows with 16 bytes each. Each warp transposes 32-column chunks through its own 4 KB
        // of shared memory (16-byte groups XOR-swizzled by row: conflict-free both ways) so that an
        // instruction writes four rows of 128 contiguous bytes.
        float4* stg = reinterpret_cast<float4*>(extra) + warp * 256;
        float* ytile = p.y + (int64_t)ti.row0 * HID + ti.nt * TC_BN + half * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int g4 = 0; g4 < 8; ++g4)
            stg[lane * 8 + (g4 ^ (lane & 7))] =
                make_float4(acc[32 * c + 4 * g4], acc[32 * c + 4 * g4 + 1], acc[32 * c + 4 * g4 + 2], acc[32 * c + 4 * g4 + 3]);
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = 4 * i + (lane >> 3), gg = lane & 7;
            const float4 val = stg[rr * 8 + (gg ^ (rr & 7))];
            const int trow = 32 * q + rr;
            if (trow < ti.rows)
              *reinterpret_cast<float4*>(ytile + (int64_t)trow * HID + 32 * c + 4 * gg) = val;
          }
          __syncwarp();
        }
      } else {
        // SwiGLU on this thread's 64 columns of h, row maximum across the two column halves.
        // Rows that are not live may hold garbage (another expert's rows): keep it out of smem.
        float mx = 0.f;
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const float x1 = acc[j], x2 = acc[64 + j];
          const float h = __fdividef(x2, 1.0f + __expf(-x2)) * x1;
          acc[j] = h;
          mx = fmaxf(mx, fabsf(h));
        }
        s_amax[tile_par][half][r] = live ? mx : 0.f;
        // exchange through a bounded mbarrier (256 arrivals), never an unbounded bar.sync
        __syncwarp();
        if (lane == 0) ako::tc::mbar_arrive(ako::smem_u32(&s_xchg[tile_par]));
        if (!ako::tc::mbar_wait(ako::smem_u32(&s_xchg[tile_par]), (uint32_t)((tcount >> 1) & 1), p.error,
                                kErrEpilogue)) { ok = false; break; }
        const float amax = fmaxf(s_amax[tile_par][0][r], s_amax[tile_par][1][r]);
        if (live) {
          int ex = ((__float_as_int(amax) >> 23) & 0xff) - 127 - 7;  // amax / 2^ex < 256
          ex = max(ex, -100);
          const float sc = __int_as_float((ex + 127) << 23);
          const float inv = __int_as_float((127 - ex) << 23);
          uint8_t* hp = p.hq + (int64_t)(ti.row0 + r) * (2 * INTER) + ti.nt * 128 + half * 64;
#pragma unroll
          for (int c = 0; c < 4; ++c) {  // 16 columns = 16 bytes per store
            uint32_t hi_w[4], lo_w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              uint32_t hw = 0, lw = 0;
#pragma unroll
              for (int hh = 0; hh < 2; ++hh) {
                const float a0 = acc[16 * c + 4 * k + 2 * hh] * inv, a1 = acc[16 * c + 4 * k + 2 * hh + 1] * inv;
                const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(a0, a1), __NV_SATFINITE, __NV_E4M3);
                const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(hi, __NV_E4M3);
                const float2 hf2 = __half22float2(*reinterpret_cast<const __half2*>(&hr));
                const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
                    make_float2(a0 - hf2.x, a1 - hf2.y), __NV_SATFINITE, __NV_E4M3);
                hw |= (uint32_t)hi << (16 * hh);
                lw |= (uint32_t)lo << (16 * hh);
              }
              hi_w[k] = hw;
              lo_w[k] = lw;
            }
            *reinterpret_cast<uint4*>(hp + 16 * c) = make_uint4(hi_w[0], hi_w[1], hi_w[2], hi_w[3]);
            *reinterpret_cast<uint4*>(hp + INTER + 16 * c) = make_uint4(lo_w[0], lo_w[1], lo_w[2], lo_w[3]);
          }
          if (half == 0) p.h_scale[(int64_t)ti.nt * p.h_scale_stride + ti.row0 + r] = sc;
        }
      }
    }
  }

  // ================================ common exit ================================================
  ako::tc::fence_before_thread_sync();
  __syncthreads();
  t2_cluster_sync();   // the peer may still be reading this CTA's shared memory or writing its TMEM
  if (warp == 8) {
    ako::tc::fence_after_thread_sync();
    t2_tmem_dealloc(tmem_base, TC_TMEM_COLS);
  }
}
