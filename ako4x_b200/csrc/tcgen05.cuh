// Thin inline-PTX wrappers for the Blackwell (sm_100a) tensor-core path: tensor memory (TMEM)
// allocation, tcgen05.mma with shared-memory matrix descriptors, tcgen05.commit / tcgen05.ld,
// mbarriers with BOUNDED waits, and the proxy fence that makes cp.async-written shared memory
// visible to the tensor core. Every wait gives up after a clock-cycle limit and reports through an
// error word instead of spinning forever.
#pragma once
#include "common.cuh"

namespace ako {
namespace tc {

// ---- mbarrier --------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
// Non-blocking test of the phase: returns at once. A waiter polling with this wakes within a few
// tens of cycles of the completion; try_wait may leave it suspended far longer.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity. Returns false when `*err` is already set or when the
// cycle limit is reached (then `*err` is set to `code`); the caller must unwind, not retry.
// `err` is a word that starts every launch at 0: a shared-memory word of the CTA (which the kernel
// copies into its device status word on exit) or a word of the call's workspace that the call
// clears. A status word that outlives the call must not be passed here: once set, it would make
// every later launch give up its waits early.
constexpr long long kWaitLimitCycles = 400000000LL;  // ~0.2 s at 1.9 GHz
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err, int code) {
  if (mbar_test_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (mbar_test_wait(bar, parity)) return true;
    if ((++spins & 1023u) == 0u) {
      if (*reinterpret_cast<volatile int*>(err) != 0) return false;
      if (clock64() - t0 > kWaitLimitCycles) {
        atomicCAS(err, 0, code);
        return false;
      }
    }
  }
}

// The same wait made warp-uniform: every lane of the (converged) warp polls, and the warp goes on
// only if all lanes saw the phase. Roles that shuffle or __syncwarp after a wait use this form, so
// that an error path cannot split the warp.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, int* err, int code) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, err, code) ? 1 : 0) != 0;
}

// ---- TMA (bulk tensor copy global -> shared, completion counted in bytes on an mbarrier) ------
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// 2-D tiled load of the box described by `tmap` at element coordinates (x = innermost, y = row)
// into shared memory at `dst`; x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::
          "r"(dst),
      "l"(tmap), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// 3-D tiled load (x innermost); the same alignment rule for x.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tmap, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n" ::
          "r"(dst),
      "l"(tmap), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// 1-D bulk copy of `bytes` (multiple of 16, both addresses 16-byte aligned) global -> shared.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(tmap) : "memory");
}

// ---- fences ----------------------------------------------------------------------------------
// Generic-proxy writes to shared memory (st.shared, cp.async) -> visible to the async proxy
// (tcgen05.mma operand reads).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}
__device__ __forceinline__ void fence_before_thread_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void fence_after_thread_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
}

// ---- tensor memory ---------------------------------------------------------------------------
// One full warp allocates `cols` (power of two, 32..512) TMEM columns; the base address is written
// to the shared-memory word at `dst_smem`.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(dst_smem),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols) : "memory");
}

// ---- descriptors -----------------------------------------------------------------------------
// Instruction descriptor: D fp32, A and B e4m3, both K-major, dense, M x N tile.
__host__ __device__ constexpr uint32_t idesc_e4m3_f32(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// K-major operand tiles in shared memory: rows of 128 bytes, 8-row groups contiguous (1024 B), the
// 16-byte chunks of a row XOR-swizzled with (row & 7) -- the 128-byte swizzle TMA writes. The
// 64-bit descriptor = low word (start address >> 4 in bits 0-13, LBO = 1 in bits 16-29) and high
// word (SBO = 1024 >> 4, version 1 at bit 14, SWIZZLE_128B = 2 at bits 29-31).
// D[tmem] (+)= A[smem] * B[smem]^T, one K = 32 slice of e4m3, issued by ONE thread, with the two
// descriptors given as halves: both tiles share the high
// word, and the low word (start address >> 4, LBO) advances by plain 32-bit adds -- 2 per K = 32
// slice, bytes >> 4 per tile. The issuing thread is a single dependent instruction stream, so every
// instruction saved between two MMAs shortens the gap in which the tensor pipe may drain.
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t saddr) {
  return ((saddr >> 4) & 0x3FFFu) | (1u << 16);
}
constexpr uint32_t kSmemDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
template <bool ACCUMULATE>
__device__ __forceinline__ void mma_f8_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
  asm volatile(
      "{\n.reg .b64 da, db;\n.reg .pred p;\n"
      "mov.b64 da, {%1, %4};\n"
      "mov.b64 db, {%2, %4};\n"
      "setp.ne.b32 p, %5, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %3, p;\n}\n" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(kSmemDescHiSw128), "n"(ACCUMULATE ? 1 : 0)
      : "memory");
}

// bf16 operands (kind::f16, K = 16 per instruction = 32 bytes, so the same +2 per K slice).
__host__ __device__ constexpr uint32_t idesc_bf16_f32(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}
// The same fields for an operand stored with its M (or N) dimension contiguous ("MN-major"), 128-byte
// swizzle: 64 elements of 16 bits along M are one 128-byte row, 8 consecutive reduction indices
// are the 8 rows of a 1024-byte group. The low word then carries the byte distance between
// successive 64-element blocks along M (LBO), the high word the distance between successive
// 8-index groups along the reduction (SBO, 1024 bytes in kSmemDescHiSw128). A tile that was staged
// as K-major rows of 128 bytes for one product can so be read transposed by another.
__device__ __forceinline__ uint32_t smem_desc_lo_mn(uint32_t saddr, uint32_t lbo_bytes) {
  return ((saddr >> 4) & 0x3FFFu) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
// Instruction descriptor bit that declares the A operand MN-major.
constexpr uint32_t kIdescAMnMajor = 1u << 15;
__device__ __forceinline__ void mma_bf16_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n.reg .b64 da, db;\n.reg .pred p;\n"
      "mov.b64 da, {%1, %4};\n"
      "mov.b64 db, {%2, %4};\n"
      "setp.ne.b32 p, %5, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n}\n" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(kSmemDescHiSw128), "r"(accumulate)
      : "memory");
}

// Arrives on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar)
               : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives columns [col, col+32) of
// TMEM lane (lane_base + i). A warp may only touch the lane quarter 32 * (warp_id % 4).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
// Waits for this thread's tcgen05.ld; it names the destination registers of the load it completes,
// so that the compiler cannot schedule a use of them above it.
__device__ __forceinline__ void tmem_ld_wait_regs(float (&v)[32]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;\n"
      : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
        "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
        "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
        "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
        "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
      :
      : "memory");
}

// 32 lanes x 16 consecutive fp32 columns (same addressing as tmem_ld32).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait_regs16(float (&v)[16]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;\n"
      : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
        "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
        "+r"(r[15])
      :
      : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns, registers -> TMEM: thread i of the warp writes columns
// [col, col+16) of TMEM lane (lane_base + i). Same lane-quarter rule as the loads.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// Waits until this thread's tcgen05.st have been performed.
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// bf16 MMA whose A operand (128 rows x 16 reduction elements) sits in TMEM: row i in lane i, the 16
// bf16 values packed two per 32-bit column (even element in the low half) in columns [a_tmem, a_tmem+8).
__device__ __forceinline__ void mma_bf16_tmem_a(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n.reg .b64 db;\n.reg .pred p;\n"
      "mov.b64 db, {%2, %4};\n"
      "setp.ne.b32 p, %5, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n}\n" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(kSmemDescHiSw128), "r"(accumulate)
      : "memory");
}

// ---- register re-balancing between warp groups ---------------------------------------------------
template <int N>
__device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(N));
}

}  // namespace tc
}  // namespace ako
