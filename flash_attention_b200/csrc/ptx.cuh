// Inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk[.tensor]), tcgen05
// (tensor-memory alloc / mma / cp / ld / st / commit / fences) and a few packed
// math helpers.  Everything that waits is bounded: see mbar_wait().
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>

namespace fa4 {

// ---------------------------------------------------------------------------------------------
// status word (global) + abort flag (shared): the no-hang contract
//
// Status word: (code << 24) | (site << 16) | (launch epoch << 8) | (blockIdx.x & 0xff).  The first
// failure stays in the word until the host reads and clears it (compare-and-swap from 0), but it
// stops only the CTAs of the launch that recorded it: a later launch carries another epoch (the
// host counts launches modulo 256) and runs normally beside a stale word.
// ---------------------------------------------------------------------------------------------
constexpr uint32_t kStatusWaitExpired = 1u;

struct WaitCtx {
  volatile uint32_t* s_abort;  // shared-memory flag, set by the first role that gives up
  uint32_t* g_status;          // device status word (may be null)
  uint64_t budget_ns;          // limit of one wait
  uint32_t epoch = 0;          // launch epoch (0..255) recorded with a failure
};

// True when the status word holds a failure recorded by THIS launch (another CTA gave up).
__device__ __forceinline__ bool status_poisoned(const uint32_t* g_status, uint32_t epoch) {
  if (g_status == nullptr) return false;
  const uint32_t v = *reinterpret_cast<const volatile uint32_t*>(g_status);
  return v != 0u && ((v >> 8) & 0xffu) == epoch;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void report_status(const WaitCtx& w, uint32_t code, uint32_t site) {
  *w.s_abort = 1u;
  if (w.g_status != nullptr) {
    atomicCAS(w.g_status, 0u,
              (code << 24) | ((site & 0xffu) << 16) | ((w.epoch & 0xffu) << 8) | (blockIdx.x & 0xffu));
  }
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking probe of a phase (try_wait may suspend the thread for a system-defined time when
// the phase is not complete; a probe must not).
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// One poll of a blocking wait: try_wait with a short suspend-time hint.  Measured against the
// alternatives on the attention kernel: the default (system-chosen) suspend time was 2-3 % slower,
// pure test_wait polling 4 % slower.
#ifndef FA4_WAIT_HINT_NS
#define FA4_WAIT_HINT_NS 64
#endif
__device__ __forceinline__ bool mbar_poll(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"((uint32_t)FA4_WAIT_HINT_NS)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the CTA is aborting (this wait ran out, or another
// role's did); the caller must then leave its loop and go to the common tear-down.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& w,
                                          uint32_t site) {
  if (mbar_poll(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if (mbar_poll(bar, parity)) return true;
    }
    if (*w.s_abort) return false;
    if (globaltimer_ns() - t0 > w.budget_ns) {
      report_status(w, kStatusWaitExpired, site);
      return false;
    }
  }
}

// The same bounded wait for roles with slack (producer, scale copier, epilogue): a longer suspend
// hint per poll, so that a warp that waits most of the time takes fewer issue slots from the
// softmax warps of its scheduler.
template <uint32_t kHintNs>
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, const WaitCtx& w,
                                                  uint32_t site) {
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      uint32_t ok;
      asm volatile(
          "{\n"
          ".reg .pred p;\n"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
          "selp.b32 %0, 1, 0, p;\n"
          "}\n"
          : "=r"(ok)
          : "r"(bar), "r"(parity), "r"(kHintNs)
          : "memory");
      if (ok) return true;
    }
    if (*w.s_abort) return false;
    if (globaltimer_ns() - t0 > w.budget_ns) {
      report_status(w, kStatusWaitExpired, site);
      return false;
    }
  }
}

// Division by a divisor fixed at launch, as multiply-high + shift (dividends below 2^31).
struct FastDiv {
  uint32_t mul, shr;
};
inline FastDiv make_fastdiv(uint32_t d) {
  FastDiv f{0u, 0u};
  if (d > 1) {
    while ((1u << f.shr) < d) ++f.shr;
    f.mul = static_cast<uint32_t>((((1ull << f.shr) - d) << 32) / d + 1);
  }
  return f;
}
__device__ __forceinline__ int fast_div(int n, FastDiv f) {
  return static_cast<int>((__umulhi(static_cast<uint32_t>(n), f.mul) + static_cast<uint32_t>(n)) >> f.shr);
}

// ---------------------------------------------------------------------------------------------
// proxy / tcgen05 fences
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// TMA
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(m), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Tiled store shared -> global (bulk async group); coordinates must not be negative.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, uint32_t src, int c0, int c1,
                                             int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(m), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Waits until the bulk stores of this thread have finished READING shared memory.
__device__ __forceinline__ void bulk_wait_group_read0() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// Waits until the bulk stores of this thread have completed.
__device__ __forceinline__ void bulk_wait_group0() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
// 1-D bulk copy global -> shared; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// tensor memory
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor (64 bit) of the tcgen05 family:
//   [0,14) start address >> 4, [16,30) leading byte offset >> 4, [32,46) stride byte offset >> 4,
//   [46,48) descriptor version (1 on sm_100), [49,52) base offset, [61,64) swizzle mode.
constexpr uint32_t kSwizzleNone = 0, kSwizzle128 = 2, kSwizzle64 = 4, kSwizzle32 = 6;
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes, uint32_t swizzle) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3fffu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(swizzle) << 61;
  return d;
}

// The same descriptor for the tiles the attention kernels use (K-major rows of 64 bytes, 64-byte
// swizzle, 8-row groups 512 bytes apart): only the address field varies, the upper word is fixed.
__device__ __forceinline__ uint64_t make_desc_sw64(uint32_t saddr) {
  constexpr uint32_t hi = (512u >> 4) | (1u << 14) | (kSwizzle64 << 29);
  const uint32_t lo = ((saddr >> 4) & 0x3fffu) | (1u << 16);
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// Rows of 32 bytes (one 64-element step), 32-byte swizzle, 8-row groups 256 bytes apart.
__device__ __forceinline__ uint64_t make_desc_sw32(uint32_t saddr) {
  constexpr uint32_t hi = (256u >> 4) | (1u << 14) | (kSwizzle32 << 29);
  const uint32_t lo = ((saddr >> 4) & 0x3fffu) | (1u << 16);
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// Instruction descriptor of kind::mxf4nvf4 (e2m1 x e2m1, ue4m3 scales of 16-element blocks,
// fp32 accumulate, both operands K-major, K = 64 per instruction):
//   [7,10) A format (1 = e2m1), [10,13) B format, [15] A major, [16] B major (0 = K),
//   [17,23) N >> 3, [23] scale format (0 = ue4m3), [24,29) M >> 4, [29,31) A scale id,
//   [4,6) B scale id, [31] K size (0 = 64).
__host__ __device__ constexpr uint32_t make_idesc_nvf4(uint32_t m, uint32_t n) {
  return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T with block scales in tensor memory; one thread issues.
__device__ __forceinline__ void mma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X "
      "[%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem),
      "r"(sfb_tmem)
      : "memory");
}

// Copy one 32-row x 16-byte scale-factor chunk (512 contiguous bytes of shared memory) into
// 4 tensor-memory columns, replicated over the four 32-lane quadrants.
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint32_t saddr) {
  constexpr uint32_t hi = (128u >> 4) | (1u << 14);
  uint64_t desc;
  asm("mov.b64 %0, {%1, %2};" : "=l"(desc) : "r"((saddr >> 4) & 0x3fffu), "r"(hi));
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc)
               : "memory");
}

// tcgen05.ld / st, shape 32x32b: thread `lane` of warp w touches tensor-memory lane
// 32*(w%4)+lane, N consecutive 32-bit columns starting at the column of taddr.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
      "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
      "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
      "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr)
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// math helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Eight fp32 -> eight e2m1 (round to nearest even, saturating) packed little-endian: value i
// lands in nibble i of the result.
__device__ __forceinline__ uint32_t pack8_e2m1(float v0, float v1, float v2, float v3, float v4,
                                               float v5, float v6, float v7) {
  uint32_t out;
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
      "mov.b32 %0, {b0, b1, b2, b3};\n"
      "}\n"
      : "=r"(out)
      : "f"(v0), "f"(v1), "f"(v2), "f"(v3), "f"(v4), "f"(v5), "f"(v6), "f"(v7));
  return out;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t out;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(out) : "f"(hi), "f"(lo));
  return out;
}

// Byte offset of 16-byte chunk `chunk` (0..3) of row `row` inside a K-major tile whose rows
// are 64 bytes, in the 64-byte swizzle that both TMA (SWIZZLE_64B) and the tcgen05 shared
// memory descriptor (swizzle mode 4) use: 8-row groups of 512 bytes, chunk ^= (row / 2) % 4.
__device__ __forceinline__ uint32_t sw64_offset(uint32_t row, uint32_t chunk) {
  return (row >> 3) * 512u + (row & 7u) * 64u + ((chunk ^ ((row >> 1) & 3u)) << 4);
}

}  // namespace fa4
