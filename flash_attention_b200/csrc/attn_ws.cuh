// Warp-specialised variant: the production kernel.
//
// Roles of the 16 warps of a CTA (one CTA per SM, one 128-row query tile per CTA):
//   warps 0-3   softmax warpgroup 0: K/V blocks 0, 2, 4, ... of the tile (visit order)
//   warps 4-7   softmax warpgroup 1: K/V blocks 1, 3, 5, ...
//               one thread = one query row: exponentials, P -> e2m1, row sums, O correction
//   warp  8     TMA producer: Q once, then K and V tiles with their scale factors into two rings
//   warp  9     QK^T issuer: tcgen05.cp of the Q/K scale factors and the block-scaled tcgen05.mma
//               for S = Q K^T (two S buffers in tensor memory); owns tensor memory
//   warp 10     PV issuer: tcgen05.cp of the P/V scale factors and tcgen05.mma for O += P V.
//               Two issuing threads because one thread needs on the order of 100 clocks per
//               tcgen05 instruction or barrier wait next to the busy softmax warps, and a block
//               needs 18 of them; split in two they stay below the softmax time of a block.
//   warp 11     idle (completes the warpgroup for setmaxnreg)
//   warps 12-15 statistics warpgroup: for EVERY block, in order, reads S from tensor memory in
//               64-column halves, keeps the running reference maximum of each row and publishes
//               the per-block exponents (softmax.cuh block_exponents) in shared memory.
//
// Why a statistics warpgroup: the exponentials of a block (1024 clocks of the XU pipe per SM)
// can only start once the row maximum of the whole block is known.  With the maximum computed
// by the softmax threads themselves, every block paid load -> max -> hand-over -> exp in
// sequence, and with two softmax warps per scheduler the non-exp part (about as long as the exp
// part, all latency) could not be hidden.  Moving the maxima to their own warps shortens the
// softmax threads' serial part to load -> exp and keeps the running maximum in one thread per
// row, so no hand-over between the two softmax warpgroups is needed.
//
// The reference kernel (flash_attn/cute/flash_fwd_sm100.py:216-222) keeps two 128-row query
// stages with S and O for both in tensor memory (4 x 128 columns = all of it).  The block-scaled
// instruction needs tensor-memory columns for the scale factors as well, so this kernel keeps ONE
// query stage with S double-buffered across K/V blocks (S0, S1, O = 384 columns + 56 columns of
// scales) and lets the two softmax warpgroups alternate over K/V blocks.
//
// The correction step (rescale O when the reference maximum moves; separate warps in the
// reference, flash_fwd_sm100.py:2230-2351) is done by the softmax warpgroup of the block that
// moved the maximum: with the lazy threshold it is rare after the first block.
//
// Barriers (all mbarriers, every wait bounded):
//   q_full             producer -> QK issuer   Q tile + scales landed
//   k_full[], v_full[] producer -> issuers     K / V tile + scales landed in ring stage
//   s_full[stage]      QK issuer -> stats, softmax: S buffer holds block i (tcgen05.commit); also
//                                              tells the producer that the K stage is free
//   s_free[2]          stats + softmax -> QK issuer: S buffer read by both (256 arrivals)
//   st_ready[2]        stats -> softmax WG     exponents of block i published (128 arrivals)
//   st_free[2]         softmax WG -> stats     exponents slot consumed (128 arrivals)
//   p_full[2]          softmax WG -> PV issuer P block + its scales in shared memory (128 arrivals)
//   pv_done[stage]     PV issuer -> softmax, producer: PV of block i complete: P buffer and V
//                                              stage free, O stable (tcgen05.commit)
//   fin                both softmax WGs        row sums published for the final combine
//   drain[2]           issuers                 tensor-core work drained on the abort path
#pragma once
#include "attn_common.cuh"
#include "attn_serial.cuh"  // tensor-memory map, tile byte sizes

namespace fa4 {

// Optional per-role timeline (compile with -DFA4_TRACE): lane 0 of every warp of ONE CTA appends
// (event, block index, clock64) records to a global buffer set by fa4_nvfp4_debug_set_trace.
#ifdef FA4_TRACE
__device__ unsigned long long* g_trace_buf = nullptr;   // [16 warps][kTraceCap][2]
__device__ int g_trace_cta = 0;
constexpr int kTraceCap = 1024;
#define FA4_TRACE_DECL int trace_n = 0;
#define FA4_TRACE_EV(ev, idx)                                                                  \
  do {                                                                                         \
    if (g_trace_buf != nullptr && (int)blockIdx.x == g_trace_cta && (threadIdx.x & 31) == 0 && \
        trace_n < kTraceCap) {                                                                 \
      unsigned long long* r_ = g_trace_buf + ((threadIdx.x >> 5) * kTraceCap + trace_n) * 2;   \
      r_[0] = ((unsigned long long)(ev) << 32) | (unsigned)(idx);                              \
      r_[1] = clock64();                                                                       \
      ++trace_n;                                                                               \
    }                                                                                          \
  } while (0)
#else
#define FA4_TRACE_DECL
#define FA4_TRACE_EV(ev, idx) do {} while (0)
#endif

namespace ws {

constexpr int kStagesK = 4;
constexpr int kStagesV = 4;
constexpr int kThreads = 512;
constexpr int kProducerWarp = 8;
constexpr int kIssuerWarp = 9;    // QK^T issuer, owns tensor memory
constexpr int kPvIssuerWarp = 10;
constexpr int kStatsWarp0 = 12;
// registers per thread after setmaxnreg: 256 * 200 + 128 * 40 + 128 * 72 = 65536
constexpr int kRegsSoftmax = 200;
constexpr int kRegsOther = 40;
constexpr int kRegsStats = 72;

// per-row record the statistics warpgroup publishes for one block
struct alignas(16) RowStats {
  float noff[8];   // exponent offsets of the 8 key blocks
  uint32_t ue[2];  // packed (e + 127) bytes
  float m_prev;    // reference maximum before this block (raw units)
  float m_new;     // reference maximum from this block on
};
static_assert(sizeof(RowStats) == 48, "RowStats is read with three 16-byte loads");

// shared-memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kOffQ = 0;                                  // 8 KB
constexpr uint32_t kOffK = kOffQ + kTileBytes;                 // kStagesK x 8 KB
constexpr uint32_t kOffV = kOffK + kStagesK * kTileBytes;      // kStagesV x 8 KB
constexpr uint32_t kOffP = kOffV + kStagesV * kTileBytes;      // 2 x 8 KB
constexpr uint32_t kOffSFQ = kOffP + 2 * kTileBytes;           // 1 KB
constexpr uint32_t kOffSFK = kOffSFQ + kSfBytes;               // kStagesK x 1 KB
constexpr uint32_t kOffSFV = kOffSFK + kStagesK * kSfBytes;    // kStagesV x 1 KB
constexpr uint32_t kOffSFP = kOffSFV + kStagesV * kSfBytes;    // 2 x 1 KB
constexpr uint32_t kOffStats = kOffSFP + 2 * kSfBytes;         // 2 x 128 x RowStats
constexpr uint32_t kOffFin = kOffStats + 2 * 128 * 48;         // 2 x 128 x (sum, ref) floats
constexpr uint32_t kOffBar = kOffFin + 2 * 128 * 8;
constexpr int kNumBars = 1 + 2 * kStagesK + 2 * kStagesV + 2 * 4 + 3;
constexpr uint32_t kOffMisc = kOffBar + 8 * kNumBars;          // tmem slot, abort flag
constexpr uint32_t kSmemUsed = kOffMisc + 16;
constexpr uint32_t kSmemRequest = kSmemUsed + 1024 > 120 * 1024 ? kSmemUsed + 1024 : 120 * 1024;

enum Site {
  kSiteQFull = 10, kSiteKEmpty, kSiteVEmpty, kSiteKFull, kSiteVFull, kSiteSFull, kSiteSFree,
  kSitePFull, kSitePvDone, kSiteStReady, kSiteStFree, kSiteFin, kSiteFinalO
};

struct Bars {
  uint32_t q_full, k_full, v_full, s_full, s_free, st_ready, st_free, p_full, pv_done, fin, drain;
  __device__ explicit Bars(uint32_t b) {
    q_full = b;
    k_full = q_full + 8;
    v_full = k_full + 8 * kStagesK;
    s_full = v_full + 8 * kStagesV;   // kStagesK barriers, indexed by block % kStagesK
    pv_done = s_full + 8 * kStagesK;  // kStagesV barriers, indexed by block % kStagesV
    s_free = pv_done + 8 * kStagesV;
    st_ready = s_free + 16;
    st_free = st_ready + 16;
    p_full = st_free + 16;
    fin = p_full + 16;
    drain = fin + 8;
  }
};

// Probe first, block (bounded) only if the probe failed; result is warp-uniform.
__device__ __forceinline__ bool wait_probed(bool probed, uint32_t bar, uint32_t parity,
                                            const WaitCtx& wc, uint32_t site) {
  if (__all_sync(0xffffffffu, probed)) return true;
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, wc, site));
}

}  // namespace ws

__global__ void __launch_bounds__(ws::kThreads, 1)
attn_fwd_ws_kernel(const __grid_constant__ CUtensorMap tm_q,
                   const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const KernelParams p) {
  using namespace ws;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  const Bars bars(base + kOffBar);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + kOffMisc);
  volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(gbase + kOffMisc + 4);
  RowStats* s_stats = reinterpret_cast<RowStats*>(gbase + kOffStats);            // [2][128]
  volatile float* s_fin = reinterpret_cast<volatile float*>(gbase + kOffFin);    // [2][128][2]

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const WaitCtx wc{s_abort, p.status, p.budget_ns};

  if (tid == 0) {
    *s_abort = 0u;
    mbar_init(bars.q_full, 1);
    for (int s = 0; s < kStagesK; ++s) mbar_init(bars.k_full + 8 * s, 1);
    for (int s = 0; s < kStagesV; ++s) mbar_init(bars.v_full + 8 * s, 1);
    for (int s = 0; s < kStagesK; ++s) mbar_init(bars.s_full + 8 * s, 1);
    for (int s = 0; s < kStagesV; ++s) mbar_init(bars.pv_done + 8 * s, 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(bars.s_free + 8 * b, 256);
      mbar_init(bars.st_ready + 8 * b, 128);
      mbar_init(bars.st_free + 8 * b, 128);
      mbar_init(bars.p_full + 8 * b, 128);
    }
    mbar_init(bars.fin, 256);
    mbar_init(bars.drain, 1);
    mbar_init(bars.drain + 8, 1);
    fence_barrier_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == kIssuerWarp) {
    tmem_alloc(base + kOffMisc, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const bool poisoned =
      (p.status != nullptr) && (*reinterpret_cast<volatile uint32_t*>(p.status) != 0u);

  const Tile t = decode_tile(p, blockIdx.x);
  const int n = poisoned ? 0 : t.n_blocks;
  constexpr uint32_t idesc = make_idesc_nvf4(128, 128);
  FA4_TRACE_DECL
  FA4_TRACE_EV(0, 0);

  if (warp >= kStatsWarp0) {
    // =========================================== statistics warpgroup ===========================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsStats));
    const int row = tid & 127;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    float m_run = kNegInf;
    bool ok = true;
    for (int i = 0; ok && i < n; ++i) {
      const int b = i & 1, nb = n - 1 - i;
      const uint32_t bar_s = bars.s_full + 8 * (i % kStagesK), par_s = (i / kStagesK) & 1;
      const uint32_t bar_f = bars.st_free + 8 * b, par_f = ((i - 2) >> 1) & 1;
      const bool r_s = mbar_try_wait(bar_s, par_s);
      const bool r_f = (i >= 2) ? mbar_try_wait(bar_f, par_f) : true;
      ok = wait_probed(r_s, bar_s, par_s, wc, kSiteSFull);
      if (!ok) break;
      FA4_TRACE_EV(30, i);
      tc_fence_after_sync();
      const bool masked = block_needs_mask(p, t, nb);
      const int limit = causal_limit(p, t, row, nb);
      float bm[8];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float s[64];
        tmem_ld32(lane_addr + (b ? kTmS1 : kTmS0) + 64 * h, reinterpret_cast<uint32_t*>(&s[0]));
        tmem_ld32(lane_addr + (b ? kTmS1 : kTmS0) + 64 * h + 32, reinterpret_cast<uint32_t*>(&s[32]));
        tc_wait_ld();
        if (masked) {
#pragma unroll
          for (int c = 0; c < 64; ++c) s[c] = (64 * h + c <= limit) ? s[c] : kNegInf;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float m0 = fmax3(s[16 * q], s[16 * q + 1], s[16 * q + 2]);
          float m1 = fmax3(s[16 * q + 3], s[16 * q + 4], s[16 * q + 5]);
          m0 = fmax3(m0, s[16 * q + 6], s[16 * q + 7]);
          m1 = fmax3(m1, s[16 * q + 8], s[16 * q + 9]);
          m0 = fmax3(m0, s[16 * q + 10], s[16 * q + 11]);
          m1 = fmax3(m1, s[16 * q + 12], s[16 * q + 13]);
          m0 = fmax3(m0, s[16 * q + 14], s[16 * q + 15]);
          bm[4 * h + q] = fmaxf(m0, m1);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(bars.s_free + 8 * b);
      const float m01 = fmax3(bm[0], bm[1], bm[2]);
      const float m23 = fmax3(bm[3], bm[4], bm[5]);
      const float m_loc = fmax3(fmaxf(m01, m23), bm[6], bm[7]);
      const float m_new = next_reference(m_run, m_loc, p.sl2);
      RowStats rs;
      block_exponents(bm, m_new, p.sl2, rs.noff, rs.ue);
      rs.m_prev = m_run;
      rs.m_new = m_new;
      m_run = m_new;
      // the slot is free once the softmax warpgroup of block i-2 has read it
      ok = wait_probed(r_f, bar_f, par_f, wc, kSiteStFree);
      if (!ok) break;
      uint4* dst = reinterpret_cast<uint4*>(&s_stats[b * 128 + row]);
      const uint4* src = reinterpret_cast<const uint4*>(&rs);
      dst[0] = src[0];
      dst[1] = src[1];
      dst[2] = src[2];
      mbar_arrive(bars.st_ready + 8 * b);
      FA4_TRACE_EV(31, i);
    }
  } else if (warp >= 8) {
    // registers move from this warpgroup to the softmax warpgroups
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
    if (warp == kProducerWarp) {
      // ========================================= TMA producer ===================================
      if (lane == 0 && n > 0) {
        mbar_arrive_expect_tx(bars.q_full, kTileBytes + kSfBytes);
        tma_load_4d(base + kOffQ, &tm_q, bars.q_full, 0, t.h, t.m_blk * kBlockM, t.b);
        bulk_load(base + kOffSFQ,
                  p.q_sf + t.b * p.qsf_stride_b + t.h * p.qsf_stride_h + (int64_t)t.m_blk * kSfBytes,
                  kSfBytes, bars.q_full);
        const uint8_t* ksf = p.k_sf + t.b * p.ksf_stride_b + t.hk * p.ksf_stride_h;
        const uint8_t* vsf = p.v_sf + t.b * p.vsf_stride_b + t.hk * p.vsf_stride_h;
        bool ok = true;
        int issued_k = 0, issued_v = 0;
        // K runs two blocks ahead of V: QK^T of block i+2 is issued before PV of block i.
        for (int step = 0; ok && step < n + 2; ++step) {
          const int ik = step, iv = step - 2;
          if (ik < n) {
            const int st = ik % kStagesK, nb = n - 1 - ik;
            // stage st is free once QK^T of block ik - kStagesK has completed (its s_full phase)
            if (ik >= kStagesK) {
              const int j = ik - kStagesK;
              ok = mbar_wait(bars.s_full + 8 * (j % kStagesK), (j / kStagesK) & 1, wc, kSiteKEmpty);
              if (!ok) break;
            }
            mbar_arrive_expect_tx(bars.k_full + 8 * st, kTileBytes + kSfBytes);
            tma_load_4d(base + kOffK + st * kTileBytes, &tm_k, bars.k_full + 8 * st, 0, t.hk,
                        nb * kBlockN, t.b);
            bulk_load(base + kOffSFK + st * kSfBytes, ksf + (int64_t)nb * kSfBytes, kSfBytes,
                      bars.k_full + 8 * st);
            issued_k = ik + 1;
          }
          if (iv >= 0 && iv < n) {
            const int st = iv % kStagesV, nb = n - 1 - iv;
            if (iv >= kStagesV) {
              const int j = iv - kStagesV;
              ok = mbar_wait(bars.pv_done + 8 * (j % kStagesV), (j / kStagesV) & 1, wc, kSiteVEmpty);
              if (!ok) break;
            }
            mbar_arrive_expect_tx(bars.v_full + 8 * st, kTileBytes + kSfBytes);
            tma_load_4d(base + kOffV + st * kTileBytes, &tm_v, bars.v_full + 8 * st,
                        nb * (kBlockN / 2), 0, t.hk, t.b);
            bulk_load(base + kOffSFV + st * kSfBytes, vsf + (int64_t)nb * kSfBytes, kSfBytes,
                      bars.v_full + 8 * st);
            issued_v = iv + 1;
          }
        }
        if (!ok) {
          // bounded drain: let the copies already issued land before the CTA's memory is released
          const uint64_t t0 = globaltimer_ns();
          const uint64_t lim = 50ull * 1000 * 1000;
          for (int i = issued_k > kStagesK ? issued_k - kStagesK : 0; i < issued_k; ++i) {
            while (!mbar_try_wait(bars.k_full + 8 * (i % kStagesK), (i / kStagesK) & 1) &&
                   globaltimer_ns() - t0 < lim) {}
          }
          for (int i = issued_v > kStagesV ? issued_v - kStagesV : 0; i < issued_v; ++i) {
            while (!mbar_try_wait(bars.v_full + 8 * (i % kStagesV), (i / kStagesV) & 1) &&
                   globaltimer_ns() - t0 < lim) {}
          }
          while (!mbar_try_wait(bars.q_full, 0) && globaltimer_ns() - t0 < lim) {}
        }
      }
    } else if (warp == kIssuerWarp) {
      // ========================================= QK^T issuer ====================================
      if (lane == 0 && n > 0) {
        bool ok = mbar_wait(bars.q_full, 0, wc, kSiteQFull);
        if (ok) {
          tc_fence_after_sync();
          tc_cp_sf(tmem + kTmSFQ, base + kOffSFQ);
          tc_cp_sf(tmem + kTmSFQ + 4, base + kOffSFQ + 512);
        }
        const uint64_t dq0 = make_desc_sw64(base + kOffQ), dq1 = make_desc_sw64(base + kOffQ + 32);
        for (int i = 0; ok && i < n; ++i) {
          const int st = i % kStagesK, b = i & 1;
          if (i >= 2) {
            // S buffer b is free once block i-2 has been read by the stats and softmax warps
            ok = mbar_wait(bars.s_free + 8 * b, ((i - 2) >> 1) & 1, wc, kSiteSFree);
            if (!ok) break;
          }
          ok = mbar_wait(bars.k_full + 8 * st, (i / kStagesK) & 1, wc, kSiteKFull);
          if (!ok) break;
          FA4_TRACE_EV(20, i);
          tc_fence_after_sync();
          const uint32_t sfk = tmem + kTmSFK + 8 * b;
          const uint32_t ksf = base + kOffSFK + st * kSfBytes, kt = base + kOffK + st * kTileBytes;
          tc_cp_sf(sfk, ksf);
          tc_cp_sf(sfk + 4, ksf + 512);
          const uint32_t s_tm = tmem + (b ? kTmS1 : kTmS0);
          mma_nvf4(s_tm, dq0, make_desc_sw64(kt), idesc, tmem + kTmSFQ, sfk, 0u);
          mma_nvf4(s_tm, dq1, make_desc_sw64(kt + 32), idesc, tmem + kTmSFQ + 4, sfk + 4, 1u);
          tc_commit(bars.s_full + 8 * st);
          FA4_TRACE_EV(27, i);
        }
        if (!ok) {
          // bounded drain of the tensor-core work already issued, before tensor memory is freed
          const uint64_t t0 = globaltimer_ns();
          tc_commit(bars.drain);
          while (!mbar_try_wait(bars.drain, 0) && globaltimer_ns() - t0 < 50ull * 1000 * 1000) {}
        }
      }
    } else if (warp == kPvIssuerWarp) {
      // ========================================= PV issuer ======================================
      if (lane == 0 && n > 0) {
        bool ok = true;
        for (int i = 0; ok && i < n; ++i) {
          const int st = i % kStagesV, b = i & 1;
          ok = mbar_wait(bars.v_full + 8 * st, (i / kStagesV) & 1, wc, kSiteVFull);
          if (!ok) break;
          ok = mbar_wait(bars.p_full + 8 * b, (i >> 1) & 1, wc, kSitePFull);
          if (!ok) break;
          FA4_TRACE_EV(22, i);
          tc_fence_after_sync();
          const uint32_t sfp = tmem + kTmSFP + 8 * b, sfv = tmem + kTmSFV + 8 * b;
          const uint32_t psf = base + kOffSFP + b * kSfBytes, vsf = base + kOffSFV + st * kSfBytes;
          const uint32_t pt = base + kOffP + b * kTileBytes, vt = base + kOffV + st * kTileBytes;
          tc_cp_sf(sfp, psf);
          tc_cp_sf(sfv, vsf);
          mma_nvf4(tmem + kTmO, make_desc_sw64(pt), make_desc_sw64(vt), idesc, sfp, sfv,
                   i > 0 ? 1u : 0u);
          tc_cp_sf(sfp + 4, psf + 512);
          tc_cp_sf(sfv + 4, vsf + 512);
          mma_nvf4(tmem + kTmO, make_desc_sw64(pt + 32), make_desc_sw64(vt + 32), idesc, sfp + 4,
                   sfv + 4, 1u);
          tc_commit(bars.pv_done + 8 * st);
          FA4_TRACE_EV(23, i);
        }
        if (!ok) {
          const uint64_t t0 = globaltimer_ns();
          tc_commit(bars.drain + 8);
          while (!mbar_try_wait(bars.drain + 8, 0) && globaltimer_ns() - t0 < 50ull * 1000 * 1000) {}
        }
      }
    }
  } else {
    // =========================================== softmax warpgroups =============================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    const int g = warp >> 2;        // warpgroup 0 / 1
    const int row = tid & 127;      // tile row == tensor-memory lane
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    float m_ref = kNegInf, l_sum = 0.f;
    bool ok = true;

    for (int i = g; ok && i < n; i += 2) {
      const int u = i >> 1, nb = n - 1 - i;
      FA4_TRACE_EV(1, i);
      // Probe both barriers this block depends on back to back so that their latencies overlap;
      // the blocking (bounded) wait only runs for a probe that failed.  st_ready implies s_full.
      const uint32_t bar_r = bars.st_ready + 8 * g, par_r = u & 1;
      const uint32_t bar_p = bars.pv_done + 8 * ((i - 2) % kStagesV), par_p = ((i - 2) / kStagesV) & 1;
      const bool r_r = mbar_try_wait(bar_r, par_r);
      const bool r_p = (i >= 2) ? mbar_try_wait(bar_p, par_p) : true;
      ok = wait_probed(r_r, bar_r, par_r, wc, kSiteStReady);
      if (!ok) break;
      tc_fence_after_sync();
      float s[128];
#pragma unroll
      for (int c = 0; c < 4; ++c)
        tmem_ld32(lane_addr + (g ? kTmS1 : kTmS0) + 32 * c, reinterpret_cast<uint32_t*>(&s[32 * c]));
      // this row's exponents (read while the tensor-memory load is in flight)
      RowStats rs;
      {
        const uint4* src = reinterpret_cast<const uint4*>(&s_stats[g * 128 + row]);
        uint4* dst = reinterpret_cast<uint4*>(&rs);
        dst[0] = src[0];
        dst[1] = src[1];
        dst[2] = src[2];
      }
      tc_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(bars.s_free + 8 * g);
      mbar_arrive(bars.st_free + 8 * g);

      if (block_needs_mask(p, t, nb)) mask_row(s, causal_limit(p, t, row, nb));

      // own partial row sum follows the reference
      if (rs.m_new != m_ref) l_sum *= reference_factor(m_ref, rs.m_new, p.sl2);
      m_ref = rs.m_new;

      // correction: O holds blocks 0..i-1 relative to m_prev
      if (i > 0 && __any_sync(0xffffffffu, rs.m_new != rs.m_prev)) {
        ok = __all_sync(0xffffffffu,
                        mbar_wait(bars.pv_done + 8 * ((i - 1) % kStagesV), ((i - 1) / kStagesV) & 1, wc,
                                  kSitePvDone));
        if (!ok) break;
        tc_fence_after_sync();
        const float f = (rs.m_new != rs.m_prev) ? reference_factor(rs.m_prev, rs.m_new, p.sl2) : 1.f;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(lane_addr + kTmO + 32 * c, o);
          tc_wait_ld();
#pragma unroll
          for (int x = 0; x < 32; ++x) o[x] = __float_as_uint(__uint_as_float(o[x]) * f);
          tmem_st32(lane_addr + kTmO + 32 * c, o);
        }
        tc_wait_st();
      }

      // P buffer g is free once PV of block i-2 has completed
      ok = wait_probed(r_p, bar_p, par_p, wc, kSitePvDone);
      if (!ok) break;
      FA4_TRACE_EV(6, i);
      l_sum += quantize_row(s, rs.noff, rs.ue, p.sl2, gbase + kOffP + g * kTileBytes, row);
      FA4_TRACE_EV(7, i);
      uint8_t* ssf = gbase + kOffSFP + g * kSfBytes;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        *reinterpret_cast<uint32_t*>(ssf + 512 * j + (row & 31) * 16 + (row >> 5) * 4) =
            block_scale_bytes(rs.ue[j]);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();  // orders the O rescale stores before the issuer's next MMA
      mbar_arrive(bars.p_full + 8 * g);
    }

    // ---- final combine of the two partial row sums ------------------------------------------------
    if (ok && n > 0) {
      s_fin[(g * 128 + row) * 2] = l_sum;
      s_fin[(g * 128 + row) * 2 + 1] = m_ref;
      mbar_arrive(bars.fin);
      ok = __all_sync(0xffffffffu, mbar_wait(bars.fin, 0, wc, kSiteFin));
      if (ok) {
        const float l_other = s_fin[((g ^ 1) * 128 + row) * 2];
        const float m_other = s_fin[((g ^ 1) * 128 + row) * 2 + 1];
        const float m_fin = fmaxf(m_ref, m_other);
        const float l_tot = l_sum * reference_factor(m_ref, m_fin, p.sl2) +
                            l_other * reference_factor(m_other, m_fin, p.sl2);
        l_sum = (m_fin == kNegInf) ? 0.f : l_tot;
        m_ref = m_fin;
        ok = __all_sync(0xffffffffu,
                        mbar_wait(bars.pv_done + 8 * ((n - 1) % kStagesV), ((n - 1) / kStagesV) & 1, wc,
                                  kSiteFinalO));
        tc_fence_after_sync();
      }
    }

    // ---- epilogue: warpgroup g stores output columns [64 g, 64 g + 64) ------------------------------
    if (ok && !poisoned) {
      const int q_idx = t.m_blk * kBlockM + row;
      __nv_bfloat16* orow =
          p.out + t.b * p.o_stride_b + (int64_t)q_idx * p.o_stride_s + t.h * p.o_stride_h;
      const bool empty = (n == 0) || !(l_sum > 0.f);
      const float scale = empty ? 0.f : p.out_scale / l_sum;
#pragma unroll 1
      for (int c = 2 * g; c < 2 * g + 2; ++c) {
        uint32_t o[32];
        if (n > 0) {
          tmem_ld32(lane_addr + kTmO + 32 * c, o);
          tc_wait_ld();
        }
        if (empty) {
#pragma unroll
          for (int x = 0; x < 32; ++x) o[x] = 0u;
        }
        store_out_32(orow + 32 * c, o, scale);
      }
      if (g == 0 && p.lse != nullptr) {
        p.lse[((int64_t)t.b * p.Hq + t.h) * p.Sq + q_idx] = finish_lse(m_ref, l_sum, p.sl2);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kIssuerWarp) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace fa4
