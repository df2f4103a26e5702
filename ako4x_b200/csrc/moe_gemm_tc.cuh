// Grouped FP8 block-scale GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), included by
// moe.cu inside its anonymous namespace (it uses GemmParams and the size constants defined there).
//
// One persistent CTA per SM walks the tile list (expert, n-tile, m-tile). A tile is 128 rows x 256
// weight rows; every K step of 128 (one scale block) is four tcgen05.mma M128 N256 K32 e4m3
// instructions into one of two 256-column TMEM accumulators. 9 warps, two roles:
//   warp 8      one thread issues the MMAs; tcgen05.commit frees the shared-memory stage and
//               publishes the TMEM accumulator of the K block;
//   warps 0-7   256 worker threads. Each iteration g they (1) cp.async their share of K block g+3
//               (A rows gathered by token in GEMM1, weight rows) into a 4-stage ring of
//               128-byte-swizzled K-major tiles, (2) wait for their copies of K block g+1, fence them
//               towards the async proxy and arrive on its `full` barrier, (3) pull the partial
//               accumulator of K block g out of TMEM (tcgen05.ld), release the buffer, and promote
//               it into fp32 registers with  a_scale[row, kb] * w_scale[block, kb]  -- the 128x128
//               block-scale rule. The promotion of block g overlaps the MMAs of block g+1.
//               Thread (warp w, lane l) owns accumulator row 32*(w%4)+l and columns 128*(w/4)...
// GEMM1 orders the weight rows of a tile as [g1 0-63 | g2 0-63 | g1 64-127 | g2 64-127] of one
// 128-column block of h, so each worker owns matching linear/gate columns and applies SwiGLU, the
// two-piece e4m3 quantisation and 64-byte row stores by itself. GEMM2 stores fp32 y.
// No register re-balancing (setmaxnreg) is used: 288 threads leave 224 registers per thread.
// Every mbarrier wait is bounded; a timeout sets p.error and both roles unwind to a common exit
// that frees TMEM.
#pragma once
// (tcgen05.cuh is included by moe.cu at file scope, before the anonymous namespace opens)

constexpr int TC_BM = 128;
constexpr int TC_BN = 256;
constexpr int TC_STAGES = 4;
constexpr int TC_LAG = 3;                       // K blocks issued ahead of the one being promoted
constexpr int TC_A_BYTES = TC_BM * 128;
constexpr int TC_B_BYTES = TC_BN * 128;
constexpr int TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;
constexpr int TC_SMEM = TC_STAGES * TC_STAGE_BYTES + 1024;  // + slack for 1024-byte alignment
constexpr int TC_WORKERS = 256;
constexpr int TC_THREADS = TC_WORKERS + 32;
constexpr int TC_TMEM_COLS = 512;

enum : int { kErrLoad = 1, kErrMmaFull = 2, kErrMmaAcc = 3, kErrEpilogue = 4 };

struct TileInfo {
  int e, nt, row0, rows;
};

template <int NT_TILES>
__device__ __forceinline__ TileInfo tc_tile_info(const GemmParams& p, const int* s_cum, int tile) {
  TileInfo ti;
  int e = 0;
  while (s_cum[e + 1] * NT_TILES <= tile) ++e;
  const int mt_e = s_cum[e + 1] - s_cum[e];
  const int rem = tile - s_cum[e] * NT_TILES;
  const int mt = rem % mt_e;
  ti.e = e;
  ti.nt = rem / mt_e;
  ti.row0 = p.offsets[e] + mt * TC_BM;
  ti.rows = min(TC_BM, p.counts[e] - mt * TC_BM);
  return ti;
}

template <int WHICH>
__global__ void __launch_bounds__(TC_THREADS, 1) moe_gemm_tc_kernel(GemmParams p) {
  constexpr int NKB = (WHICH == 1) ? KB1 : KB2;
  constexpr int NT_TILES = (WHICH == 1) ? (INTER / 128) : (HID / TC_BN);
  constexpr int64_t W_ROW = (WHICH == 1) ? HID : INTER;      // bytes per weight row
  constexpr int64_t A_ROW = (WHICH == 1) ? HID : 2 * INTER;  // bytes per activation row
  constexpr uint32_t IDESC = ako::tc::idesc_e4m3_f32(TC_BM, TC_BN);

  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t s_full[TC_STAGES];
  __shared__ __align__(8) uint64_t s_empty[TC_STAGES];
  __shared__ __align__(8) uint64_t s_acc_full[2];
  __shared__ __align__(8) uint64_t s_acc_empty[2];
  __shared__ __align__(8) uint64_t s_xchg[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_cum[MAX_LOCAL + 1];
  __shared__ float s_amax[2][2][TC_BM];  // [tile parity][column half][row]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t smem_base = (ako::smem_u32(smem_raw) + 1023u) & ~1023u;

  if (tid == 0) {
    int acc = 0;
    for (int e = 0; e < p.n_local; ++e) {
      s_cum[e] = acc;
      acc += (p.counts[e] + TC_BM - 1) / TC_BM;
    }
    s_cum[p.n_local] = acc;
    for (int s = 0; s < TC_STAGES; ++s) {
      ako::tc::mbar_init(ako::smem_u32(&s_full[s]), TC_WORKERS);
      ako::tc::mbar_init(ako::smem_u32(&s_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ako::tc::mbar_init(ako::smem_u32(&s_acc_full[b]), 1);
      ako::tc::mbar_init(ako::smem_u32(&s_acc_empty[b]), TC_WORKERS);
      ako::tc::mbar_init(ako::smem_u32(&s_xchg[b]), TC_WORKERS);
    }
    ako::tc::mbar_init_fence();
  }
  if (warp == 8) ako::tc::tmem_alloc(ako::smem_u32(&s_tmem_base), TC_TMEM_COLS);
  ako::tc::fence_before_thread_sync();
  __syncthreads();
  ako::tc::fence_after_thread_sync();
  const uint32_t tmem_base = s_tmem_base;
  const int total_tiles = s_cum[p.n_local] * NT_TILES;
  // K blocks this CTA runs in total (tiles blockIdx.x, +gridDim.x, ...)
  const int my_tiles = (total_tiles > (int)blockIdx.x) ? (total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const int G = my_tiles * NKB;

  if (warp == 8) {
    // ================================ MMA issuer ===============================================
    if (lane == 0) {
      for (int g = 0; g < G; ++g) {
        const int stage = g % TC_STAGES;
        const uint32_t ph = (g / TC_STAGES) & 1;
        const int buf = g & 1;
        const uint32_t aph = (g >> 1) & 1;
        if (!ako::tc::mbar_wait(ako::smem_u32(&s_acc_empty[buf]), aph ^ 1u, p.error, kErrMmaAcc)) break;
        if (!ako::tc::mbar_wait(ako::smem_u32(&s_full[stage]), ph, p.error, kErrMmaFull)) break;
        ako::tc::fence_after_thread_sync();
        const uint32_t sa = smem_base + stage * TC_STAGE_BYTES;
        const uint32_t sb = sa + TC_A_BYTES;
        const uint32_t d = tmem_base + buf * TC_BN;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          ako::tc::mma_f8(d, ako::tc::smem_desc_k_sw128(sa + ks * 32), ako::tc::smem_desc_k_sw128(sb + ks * 32),
                          IDESC, ks > 0 ? 1u : 0u);
        ako::tc::mma_commit(ako::smem_u32(&s_empty[stage]));
        ako::tc::mma_commit(ako::smem_u32(&s_acc_full[buf]));
      }
    }
  } else {
    // ================================ workers: load + promote ==================================
    const int half = warp >> 2;        // which 128 accumulator columns
    const int q = warp & 3;            // TMEM lane quarter
    const int r = 32 * q + lane;       // accumulator row of this thread
    bool ok = true;

    // ---- load cursor ------------------------------------------------------------------------
    int ld_g = 0;                      // next K block to issue
    int ld_tile = blockIdx.x, ld_kb = 0;
    int a_src[4] = {-1, -1, -1, -1};
    const uint8_t* ld_wbase = p.w;
    int ld_nt = 0;
    auto load_setup = [&]() {
      const TileInfo ti = tc_tile_info<NT_TILES>(p, s_cum, ld_tile);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int rr = (tid >> 3) + 32 * j;
        int src = -1;
        if (rr < ti.rows) src = (WHICH == 1) ? p.sorted_token[ti.row0 + rr] : ti.row0 + rr;
        a_src[j] = src;
      }
      ld_wbase = p.w + (int64_t)ti.e * ((WHICH == 1) ? (int64_t)2 * INTER * HID : (int64_t)HID * INTER);
      ld_nt = ti.nt;
    };
    // Issues the copies of K block ld_g (one cp.async group, possibly empty) and advances.
    auto load_issue = [&]() {
      if (ok && ld_g < G) {
        if (ld_kb == 0) load_setup();
        const int stage = ld_g % TC_STAGES;
        const uint32_t ph = (ld_g / TC_STAGES) & 1;
        if (!ako::tc::mbar_wait(ako::smem_u32(&s_empty[stage]), ph ^ 1u, p.error, kErrLoad)) {
          ok = false;
        } else {
          const uint32_t sa = smem_base + stage * TC_STAGE_BYTES;
          const uint32_t sb = sa + TC_A_BYTES;
          const int c = tid & 7;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int rr = (tid >> 3) + 32 * j;
            const bool valid = a_src[j] >= 0;
            ako::cp_async16(sa + rr * 128 + ((c ^ (rr & 7)) << 4),
                            p.a + (int64_t)(valid ? a_src[j] : 0) * A_ROW + (int64_t)ld_kb * 128 + c * 16, valid);
          }
          const int wkb = (WHICH == 1) ? ld_kb : (ld_kb & 15);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int rr = (tid >> 3) + 32 * j;
            int64_t wrow;
            if (WHICH == 1) {
              // [g1 0-63 | g2 0-63 | g1 64-127 | g2 64-127] of h columns nt*128 ..
              const int gate = (rr >> 6) & 1, blk = rr >> 7;
              wrow = (int64_t)gate * INTER + ld_nt * 128 + blk * 64 + (rr & 63);
            } else {
              wrow = (int64_t)ld_nt * TC_BN + rr;
            }
            ako::cp_async16(sb + rr * 128 + ((c ^ (rr & 7)) << 4),
                            ld_wbase + wrow * W_ROW + (int64_t)wkb * 128 + c * 16, true);
          }
          ++ld_g;
          if (++ld_kb == NKB) { ld_kb = 0; ld_tile += gridDim.x; }
        }
      }
      ako::cp_async_commit();
    };
    // Waits until this thread's copies of K block `g` have landed (at most `newer` younger groups
    // may still be in flight), then publishes them.
    auto publish = [&](int g) {
      ako::tc::fence_proxy_async_smem();
      ako::tc::mbar_arrive(ako::smem_u32(&s_full[g % TC_STAGES]));
    };

    // pipeline prologue: K blocks 0 .. LAG-1 in flight, block 0 published
#pragma unroll
    for (int i = 0; i < TC_LAG; ++i) load_issue();
    if (G > 0 && ok) {
      ako::cp_async_wait<TC_LAG - 1>();
      publish(0);
    }

    int g = 0;
    int tcount = 0;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++tcount) {
      const TileInfo ti = tc_tile_info<NT_TILES>(p, s_cum, tile);
      const int tile_par = tcount & 1;
      int src = -1;
      if (r < ti.rows) src = (WHICH == 1) ? p.sorted_token[ti.row0 + r] : ti.row0 + r;
      const float* asp = p.a_scale + (src >= 0 ? src : 0);
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
      float sa_n = (src >= 0) ? __ldg(asp) : 0.f;
      float b0_n = __ldg(bsp0), b1_n = __ldg(bsp1);
#pragma unroll 1
      for (int kb = 0; kb < NKB; ++kb, ++g) {
        // (1) keep the ring full, (2) publish K block g+1
        load_issue();
        if (!ok) break;
        if (g + 1 < G) {
          ako::cp_async_wait<TC_LAG - 1>();
          publish(g + 1);
        }
        // (3) promote K block g
        float sa = sa_n;
        if (WHICH == 2 && kb >= 16) sa *= 0.0625f;
        const float s0 = sa * b0_n, s1 = sa * b1_n;
        if (kb + 1 < NKB) {
          const int nk = (WHICH == 1) ? (kb + 1) : ((kb + 1) & 15);
          sa_n = (src >= 0) ? __ldg(asp + (int64_t)nk * p.a_scale_stride) : 0.f;
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
        ako::tc::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          acc[j] = fmaf(v0[j], s0, acc[j]);
          acc[32 + j] = fmaf(v1[j], s0, acc[32 + j]);
        }
        ako::tc::tmem_ld32(taddr + 64, v0);
        ako::tc::tmem_ld32(taddr + 96, v1);
        ako::tc::tmem_ld_wait();
        ako::tc::fence_before_thread_sync();
        ako::tc::mbar_arrive(ako::smem_u32(&s_acc_empty[buf]));
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          acc[64 + j] = fmaf(v0[j], s1, acc[64 + j]);
          acc[96 + j] = fmaf(v1[j], s1, acc[96 + j]);
        }
      }
      if (!ok) break;

      if (WHICH == 2) {
        if (r < ti.rows) {
          float* yp = p.y + (int64_t)(ti.row0 + r) * HID + ti.nt * TC_BN + half * 128;
#pragma unroll
          for (int j = 0; j < 128; j += 4)
            *reinterpret_cast<float4*>(yp + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
        }
      } else {
        // SwiGLU on this thread's 64 columns of h, row maximum across the two column halves
        float mx = 0.f;
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const float x1 = acc[j], x2 = acc[64 + j];
          const float h = (x2 / (1.0f + __expf(-x2))) * x1;
          acc[j] = h;
          mx = fmaxf(mx, fabsf(h));
        }
        s_amax[tile_par][half][r] = mx;
        // exchange through a bounded mbarrier (256 arrivals), never an unbounded bar.sync
        ako::tc::mbar_arrive(ako::smem_u32(&s_xchg[tile_par]));
        if (!ako::tc::mbar_wait(ako::smem_u32(&s_xchg[tile_par]), (uint32_t)((tcount >> 1) & 1), p.error,
                                kErrEpilogue)) { ok = false; break; }
        const float amax = fmaxf(s_amax[tile_par][0][r], s_amax[tile_par][1][r]);
        if (r < ti.rows) {
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
                    make_float2((a0 - hf2.x) * 16.f, (a1 - hf2.y) * 16.f), __NV_SATFINITE, __NV_E4M3);
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
    ako::cp_async_wait<0>();  // no copy of this thread is left in flight at exit
  }

  // ================================ common exit ================================================
  ako::tc::fence_before_thread_sync();
  __syncthreads();
  if (warp == 8) {
    ako::tc::fence_after_thread_sync();
    ako::tc::tmem_dealloc(tmem_base, TC_TMEM_COLS);
  }
}
