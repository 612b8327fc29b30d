// Warp-specialised, persistent variant: the production kernel.
//
// One CTA per SM walks a static list of 128-row query tiles (longest first, snake order over
// the CTAs).  Roles of its 24 warps:
//   warps 0-15  softmax: four warpgroups, one thread = HALF a query row of one K/V block
//               (64 keys).  warpgroup k = warp / 4:  column half = k & 1 (keys 0-63 / 64-127),
//               block parity = k >> 1 (blocks 0,2,4,.. / 1,3,5,.. of a tile in visit order,
//               so that the summation order of a row depends on its tile only).
//               exponentials, P -> e2m1, row sums, O correction, O -> bf16 staging tile
//   warps 16-19 statistics warpgroup: for EVERY block, in order, reads S from tensor memory in
//               32-column chunks, keeps the running reference maximum of each row and publishes
//               the block maxima and the reference in shared memory (the softmax threads derive
//               the per-block exponents from them, softmax.cuh block_exponents4)
//   warp 20     TMA producer: Q (double buffered across tiles), K and V rings, scale factors
//   warp 21     QK^T issuer: tcgen05.cp of the Q/K scale factors and the block-scaled tcgen05.mma
//               for S = Q K^T (two S buffers in tensor memory); owns tensor memory
//   warp 22     PV issuer: tcgen05.cp of the P/V scale factors and tcgen05.mma for O += P V
//   warp 23     output store: sends the staged bf16 O tile of every query tile with TMA
//
// Why this shape (measured on B200, see the timeline facility below):
//  * The exponentials of a block cost 1024 clocks of the XU pipe per SM (16 ex2/clk), far more
//    than its tensor-core time (256 clocks), so the kernel is organised around keeping the XU
//    pipe busy.
//  * ex2 can only start once the row maximum of the whole block is known.  The statistics
//    warpgroup takes the maxima (and the running maximum, one thread per row, no hand-over) off
//    the exponentiating threads, whose serial part shrinks to load -> exp.
//  * Everything around the exponentials is latency (barrier probes, tensor-memory loads, shared
//    memory), roughly as long as the exponentials themselves.  Two warps per scheduler could not
//    hide it; with the maxima gone a thread no longer needs the whole row in registers, so the
//    row is split in two halves and four softmax warps per scheduler overlap each other.
//  * One thread needs on the order of 100 clocks per tcgen05 instruction or barrier wait next to
//    the busy softmax warps and a block needs 18 of them: two issuing threads.
//  * Prologue and epilogue of a tile (first loads, last PV, O to global memory) were a fifth of
//    a tile's time: the CTA is persistent, the producer and the QK^T issuer run ahead into the
//    next tile while the softmax warps finish the current one (Q is double buffered; only
//    the first PV of a tile waits until O has been read out of tensor memory).
//
// The reference kernel (flash_attn/cute/flash_fwd_sm100.py:216-222) keeps two 128-row query
// stages with S and O for both in tensor memory (4 x 128 columns = all of it).  The block-scaled
// instruction needs tensor-memory columns for the scale factors as well, so this kernel keeps ONE
// query stage with S double-buffered across K/V blocks (S0, S1, O = 384 columns + 56 columns of
// scales).  The correction step (rescale O when the reference maximum moves; separate warps in
// the reference, flash_fwd_sm100.py:2230-2351) is done by the softmax warpgroups of the block
// that moved the maximum: with the lazy threshold it is rare after the first block.
//
// Block indices: i = index inside the tile (0 = last visible K/V block, the reference's visit
// order), G = blocks_before_this_tile + i = running index that picks ring stages, S/P buffers
// and barrier phases, so that the pipeline never drains between tiles.
//
// Barriers (all mbarriers, every wait bounded):
//   q_full[2]/q_empty[2] producer <-> QK issuer  Q tile + scales of a tile (q_empty by commit)
//   k_full[], v_full[]   producer -> issuers     K / V tile + scales landed in ring stage
//   s_full[stage]        QK issuer -> stats      S buffer holds block G (tcgen05.commit; the softmax
//                                                warps learn it through st_ready); also
//                                                tells the producer that the K stage is free
//   s_free[2]            stats + softmax -> QK issuer: S buffer read by all (384 arrivals)
//   st_ready[2]          stats -> softmax        exponents of block G published (128 arrivals)
//   st_free[2]           softmax -> stats        exponents slot consumed (256 arrivals)
//   p_full[stage]        softmax -> PV issuer    P block + its scales in shared memory (256);
//                                                one barrier per P tile so that the softmax can
//                                                never be two phases ahead of the issuer
//   pv_done[stage]       PV issuer -> softmax, producer: PV of block G complete: P buffer and V
//                                                stage free, O stable (tcgen05.commit)
//   fin                  softmax warpgroups      partial row sums published (512, once per tile)
//   o_free               softmax -> PV issuer    O copied to registers (512, once per tile)
//   o_staged             softmax -> store warp   bf16 O tile complete in the staging buffer (512)
//   stage_free           store warp -> softmax   TMA has read the staging buffer (1)
//   drain[2]             issuers                 tensor-core work drained on the abort path
#pragma once
#include "attn_common.cuh"
#include "attn_common.cuh"

namespace fa4 {

namespace ws {

constexpr int kStagesK = 4;
constexpr int kStagesV = 4;
constexpr int kStagesP = 4;   // P tiles in shared memory (a block's P is rewritten once PV of block G-4 is done)
// The softmax warps learn that P tile G % kStagesP is free from the pv_done barrier of block
// G - kStagesP, whose phase must not have been reused by a later block yet.
static_assert(kStagesP <= kStagesV, "P tiles are recycled through the pv_done barriers of the V stages");
constexpr int kThreads = 768;
constexpr int kStatsWarp0 = 16;
constexpr int kProducerWarp = 20;
constexpr int kIssuerWarp = 21;    // QK^T issuer, owns tensor memory
constexpr int kPvIssuerWarp = 22;
constexpr int kStoreWarp = 23;     // sends the staged output tile with TMA
// registers per thread after setmaxnreg: 512 * 96 + 128 * 56 + 128 * 40 = 61440 = 768 * 80
constexpr int kRegsSoftmax = 96;
constexpr int kRegsStats = 56;
constexpr int kRegsOther = 40;
constexpr int kRegsLaunch = 80;
static_assert(512 * kRegsSoftmax + 128 * kRegsStats + 128 * kRegsOther <= kThreads * kRegsLaunch,
              "setmaxnreg targets exceed the CTA's register allocation");
static_assert(kRegsSoftmax > kRegsLaunch && kRegsOther < kRegsLaunch, "inc / dec directions");

// per-row record the statistics warpgroup publishes for one block
struct alignas(16) RowStats {
  float bm[8];      // maxima of the 8 key blocks (raw units, masked keys excluded)
  uint32_t pad[2];
  float m_prev;     // reference maximum before this block (raw units)
  float m_new;      // reference maximum from this block on
};
static_assert(sizeof(RowStats) == 48, "RowStats is read with 16-byte loads");

// shared-memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kOffQ = 0;                                  // 2 x 8 KB
constexpr uint32_t kOffK = kOffQ + 2 * kTileBytes;             // kStagesK x 8 KB
constexpr uint32_t kOffV = kOffK + kStagesK * kTileBytes;      // kStagesV x 8 KB
constexpr uint32_t kOffP = kOffV + kStagesV * kTileBytes;      // kStagesP x 8 KB
constexpr uint32_t kOffSFQ = kOffP + kStagesP * kTileBytes;    // 2 x 1 KB
constexpr uint32_t kOffSFK = kOffSFQ + 2 * kSfBytes;           // kStagesK x 1 KB
constexpr uint32_t kOffSFV = kOffSFK + kStagesK * kSfBytes;    // kStagesV x 1 KB
constexpr uint32_t kOffSFP = kOffSFV + kStagesV * kSfBytes;    // kStagesP x 1 KB
constexpr uint32_t kOffOut = kOffSFP + kStagesP * kSfBytes;    // 32 KB: bf16 O tile staged for the TMA store
constexpr uint32_t kOffStats = kOffOut + 32 * 1024;            // 2 x 128 x RowStats
constexpr uint32_t kOffFin = kOffStats + 2 * 128 * 48;         // 2 tiles x 4 WGs x 128 x (sum, ref)
constexpr uint32_t kOffBar = kOffFin + 2 * 4 * 128 * 8;
constexpr int kNumBars = 4 + 2 * kStagesK + 2 * kStagesV + 2 * 3 + kStagesP + 4 + 2;
constexpr uint32_t kOffMisc = kOffBar + 8 * kNumBars;          // tmem slot, abort flag
constexpr uint32_t kSmemUsed = kOffMisc + 16;
constexpr uint32_t kSmemRequest = kSmemUsed + 1024;
static_assert(kSmemRequest > 114 * 1024, "one CTA per SM: every CTA allocates all of tensor memory");

enum Site {
  kSiteQFull = 10, kSiteQEmpty, kSiteKEmpty, kSiteVEmpty, kSiteKFull, kSiteVFull, kSiteSFull,
  kSiteSFree, kSitePFull, kSitePvDone, kSiteStReady, kSiteStFree, kSiteFin, kSiteFinalO, kSiteOFree,
  kSiteOStaged, kSiteStageFree
};

// barrier indices (8 bytes each from the barrier base); kept as constants so that only the base
// address lives in a register
struct Bars {
  uint32_t base;
  static constexpr uint32_t kQFull = 0, kQEmpty = 2, kKFull = 4, kVFull = kKFull + kStagesK,
                            kSFull = kVFull + kStagesV, kPvDone = kSFull + kStagesK,
                            kSFree = kPvDone + kStagesV, kStReady = kSFree + 2, kStFree = kStReady + 2,
                            kPFull = kStFree + 2, kFin = kPFull + kStagesP, kOFree = kFin + 1,
                            kDrain = kOFree + 1, kOStaged = kDrain + 2, kStageFree = kOStaged + 1,
                            kCount = kStageFree + 1;
  __device__ explicit Bars(uint32_t b) : base(b) {}
  __device__ __forceinline__ uint32_t at(uint32_t idx) const { return base + 8u * idx; }
};
static_assert(Bars::kCount <= kNumBars, "barrier area too small");

// Probe first, block (bounded) only if the probe failed; result is warp-uniform.
__device__ __forceinline__ bool wait_probed(bool probed, uint32_t bar, uint32_t parity,
                                            const WaitCtx& wc, uint32_t site) {
  if (__all_sync(0xffffffffu, probed)) return true;
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, wc, site));
}

// O[:, 32 * nchunks columns from taddr] *= f for this thread's row.  Rare (the reference maximum
// moved by more than the lazy threshold), so it is kept out of line: its 32 registers would
// otherwise be added to the pressure of the exponential loop.
__device__ __noinline__ void rescale_accumulator(uint32_t taddr, float f, int nchunks) {
  for (int c = 0; c < nchunks; ++c) {
    uint32_t o[32];
    tmem_ld32(taddr + 32 * c, o);
    tc_wait_ld();
#pragma unroll
    for (int x = 0; x < 32; ++x) o[x] = __float_as_uint(__uint_as_float(o[x]) * f);
    tmem_st32(taddr + 32 * c, o);
  }
}

// Keys with in-chunk index > limit of this thread's 64 scores at taddr become -inf.  Only on
// diagonal blocks; out of line like the rescale.
__device__ __noinline__ void mask_scores_in_tmem(uint32_t taddr, int limit) {
  for (int c = 0; c < 2; ++c) {
    // tcgen05.ld / st are warp-collective: the skip must be decided by the whole warp
    if (__all_sync(0xffffffffu, limit >= 32 * c + 31)) continue;  // chunk fully visible
    uint32_t v[32];
    tmem_ld32(taddr + 32 * c, v);
    tc_wait_ld();
#pragma unroll
    for (int x = 0; x < 32; ++x) v[x] = (32 * c + x <= limit) ? v[x] : 0xff800000u;
    tmem_st32(taddr + 32 * c, v);
  }
  tc_wait_st();
}

// The same with a lower limit as well (local attention): keys outside [lower, limit] become -inf.
__device__ __noinline__ void mask_scores_in_tmem_range(uint32_t taddr, int lower, int limit) {
  for (int c = 0; c < 2; ++c) {
    if (__all_sync(0xffffffffu, limit >= 32 * c + 31 && lower <= 32 * c)) continue;  // fully visible
    uint32_t v[32];
    tmem_ld32(taddr + 32 * c, v);
    tc_wait_ld();
#pragma unroll
    for (int x = 0; x < 32; ++x) v[x] = (32 * c + x <= limit && 32 * c + x >= lower) ? v[x] : 0xff800000u;
    tmem_st32(taddr + 32 * c, v);
  }
  tc_wait_st();
}

// Tile end: 32 accumulator columns of this thread's row -> registers (then the accumulator may be
// overwritten: arrive on o_free_bar), scaled, rounded to bf16 and written into the staging tile in
// shared memory, from where the store warp sends whole 128-byte rows with TMA (rows past Sq of a
// partial tile are clipped by the tensor map).  Staging layout: boxes of 64 output columns, 128
// rows x 128 bytes each, with the 128-byte swizzle of the tensor map: 16-byte chunk j of row r sits
// at chunk j ^ (r % 8).  o_free_bar == 0: the tile had no visible key, nothing to read, zeros are
// staged.  Direct 16-byte row stores from the softmax threads cost ~2000 clocks per tile in the
// load/store unit (32 different rows per instruction).
template <bool kHasColumns>
__device__ __noinline__ void stage_accumulator_chunk(uint32_t taddr, uint8_t* staging, int row, int wg,
                                                     float scale, uint32_t o_free_bar) {
  uint8_t* box_row = staging + (wg >> 1) * (16 * 1024) + row * 128;
  if (o_free_bar == 0u) {
    if constexpr (kHasColumns) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        const int chunk = ((wg & 1) * 4 + v) ^ (row & 7);
        *reinterpret_cast<uint4*>(box_row + chunk * 16) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    return;
  }
  uint32_t o[32];
  if constexpr (kHasColumns) {
    tmem_ld32(taddr, o);
    tc_wait_ld();
  }
  tc_fence_before_sync();
  mbar_arrive(o_free_bar);
  if constexpr (kHasColumns) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      uint4 w;
      w.x = pack_bf16x2(__uint_as_float(o[8 * v + 0]) * scale, __uint_as_float(o[8 * v + 1]) * scale);
      w.y = pack_bf16x2(__uint_as_float(o[8 * v + 2]) * scale, __uint_as_float(o[8 * v + 3]) * scale);
      w.z = pack_bf16x2(__uint_as_float(o[8 * v + 4]) * scale, __uint_as_float(o[8 * v + 5]) * scale);
      w.w = pack_bf16x2(__uint_as_float(o[8 * v + 6]) * scale, __uint_as_float(o[8 * v + 7]) * scale);
      const int chunk = ((wg & 1) * 4 + v) ^ (row & 7);
      *reinterpret_cast<uint4*>(box_row + chunk * 16) = w;
    }
  }
}

// Split-KV flavour of the same step: the 32 columns go out as fp32 (normalised by this split's
// row sum) into the partial-output workspace.
__device__ __noinline__ void store_accumulator_partial(uint32_t taddr, float* dst, float scale,
                                                       uint32_t o_free_bar) {
  float4* d4 = reinterpret_cast<float4*>(dst);
  if (o_free_bar == 0u) {
    if (dst != nullptr) {
#pragma unroll
      for (int v = 0; v < 8; ++v) d4[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    return;
  }
  uint32_t o[32];
  tmem_ld32(taddr, o);
  tc_wait_ld();
  tc_fence_before_sync();
  mbar_arrive(o_free_bar);
  if (dst == nullptr) return;
#pragma unroll
  for (int v = 0; v < 8; ++v) {
    d4[v] = make_float4(__uint_as_float(o[4 * v]) * scale, __uint_as_float(o[4 * v + 1]) * scale,
                        __uint_as_float(o[4 * v + 2]) * scale, __uint_as_float(o[4 * v + 3]) * scale);
  }
}

// Tile visited by CTA `cta` in round `it`: rounds alternate direction so that, with tiles sorted
// by decreasing work, every CTA gets about the same total.
__device__ __forceinline__ int tile_of_round(int it, int cta, int ncta) {
  return it * ncta + ((it & 1) ? (ncta - 1 - cta) : cta);
}

// Shared-memory descriptor of 64-element step j of a Q or K tile (128 rows of kD / 2 bytes).
template <int kD>
__device__ __forceinline__ uint64_t make_desc_qk(uint32_t tile_addr, int j) {
  if constexpr (kD == 128) {
    return make_desc_sw64(tile_addr + 32 * j);
  } else {
    return make_desc_sw32(tile_addr);
  }
}

}  // namespace ws

// kD: head dimension of Q, K and V (128 or 64).  It sets the number of 64-element steps of
// Q K^T, the width of O (tensor-memory columns, N of the P V instruction), the rows of a V tile and
// the bytes of a Q / K tile (128 rows of kD / 2 bytes: 64-byte-swizzled rows for 128, 32-byte for
// 64); the shared-memory slots keep the size of the larger case.
// kGeneral: split-KV work list with fp32 partial outputs (num_splits > 1) and / or the left and
// right window limits of local attention.
// kWindow: the window half of kGeneral (mask arithmetic of the hot loops); general calls without a
// window leave it out, which measured a third faster.
template <int kD, bool kGeneral, bool kWindow = kGeneral>
__global__ void __launch_bounds__(ws::kThreads, 1)
attn_fwd_ws_kernel(const __grid_constant__ CUtensorMap tm_q,
                   const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v,
                   const __grid_constant__ CUtensorMap tm_o, const KernelParams p) {
  using namespace ws;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  const Bars bars(base + kOffBar);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + kOffMisc);
  volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(gbase + kOffMisc + 4);
  RowStats* s_stats = reinterpret_cast<RowStats*>(gbase + kOffStats);            // [2][128]
  volatile float* s_fin = reinterpret_cast<volatile float*>(gbase + kOffFin);    // [2][4][128][2]

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const WaitCtx wc{s_abort, p.status, p.budget_ns, p.epoch};
  const int num_tiles = p.num_m_blocks * p.Hq * p.B * (kGeneral ? p.num_splits : 1);
  const int ncta = gridDim.x, cta = blockIdx.x;

  if (tid == 0) {
    *s_abort = 0u;
    for (int b = 0; b < 2; ++b) {
      mbar_init(bars.at(Bars::kQFull + b), 1);
      mbar_init(bars.at(Bars::kQEmpty + b), 1);
      mbar_init(bars.at(Bars::kSFree + b), 384);
      mbar_init(bars.at(Bars::kStReady + b), 128);
      mbar_init(bars.at(Bars::kStFree + b), 256);
      mbar_init(bars.at(Bars::kDrain + b), 1);
    }
    for (int s = 0; s < kStagesP; ++s) mbar_init(bars.at(Bars::kPFull + s), 256);
    for (int s = 0; s < kStagesK; ++s) mbar_init(bars.at(Bars::kKFull + s), 1);
    for (int s = 0; s < kStagesV; ++s) mbar_init(bars.at(Bars::kVFull + s), 1);
    for (int s = 0; s < kStagesK; ++s) mbar_init(bars.at(Bars::kSFull + s), 1);
    for (int s = 0; s < kStagesV; ++s) mbar_init(bars.at(Bars::kPvDone + s), 1);
    mbar_init(bars.at(Bars::kFin), 512);
    mbar_init(bars.at(Bars::kOFree), 512);
    mbar_init(bars.at(Bars::kOStaged), 512);
    mbar_init(bars.at(Bars::kStageFree), 1);
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
  static_assert(kD == 128 || kD == 64, "head dimensions built: 128 and 64");
  constexpr uint32_t idesc_qk = make_idesc_nvf4(128, 128);
  constexpr uint32_t idesc_pv = make_idesc_nvf4(128, kD);
  constexpr int kSteps = kD / 64;                      // 64-element steps of Q K^T
  constexpr uint32_t kQkBytes = 128u * kD / 2;         // bytes of a Q or K tile
  constexpr uint32_t kQkSfBytes = kSteps * 512u;       // its scale chunks (128 rows x kD / 16)
  constexpr uint32_t kVBytes = kD * 64u;               // V tile: kD rows of 128 keys

  // Every role walks the same tile list with the same counters:
  //   gb = number of K/V blocks of the tiles before the current one, ti = number of non-empty
  //   tiles before the current one.  A failure recorded by any CTA stops all of them at their
  //   next tile.
#define FA4_FOR_EACH_TILE                                                                        \
  uint32_t gb = 0, ti = 0;                                                                       \
  bool ok = true;                                                                                \
  for (int it = 0, tile = tile_of_round(0, cta, ncta); ok && tile < num_tiles;                   \
       ++it, tile = tile_of_round(it, cta, ncta))

  if (warp >= kProducerWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
    if (warp == kProducerWarp && lane == 0) {
      // ========================================= TMA producer ===================================
      uint32_t issued_k = 0, issued_v = 0, issued_q = 0;
      FA4_FOR_EACH_TILE {
        const Tile t = decode_tile<kGeneral>(p, tile);
        const int n = t.n_blocks;
        if (n == 0) continue;
        if (status_poisoned(p.status, p.epoch)) {
          *s_abort = 1u;  // another CTA failed: stop this one quickly
          break;
        }
        const uint32_t qb = ti & 1;
        if (ti >= 2) {
          ok = mbar_wait(bars.at(Bars::kQEmpty + qb), ((ti - 2) >> 1) & 1, wc, kSiteQEmpty);
          if (!ok) break;
        }
        mbar_arrive_expect_tx(bars.at(Bars::kQFull + qb), kQkBytes + kQkSfBytes);
        tma_load_4d(base + kOffQ + qb * kTileBytes, &tm_q, bars.at(Bars::kQFull + qb), 0, t.h,
                    t.m_blk * kBlockM, t.b);
        bulk_load(base + kOffSFQ + qb * kSfBytes,
                  p.q_sf + t.b * p.qsf_stride_b + t.h * p.qsf_stride_h + (int64_t)t.m_blk * kQkSfBytes,
                  kQkSfBytes, bars.at(Bars::kQFull + qb));
        issued_q = ti + 1;
        // where logical K/V block nb of this batch entry lives: (batch coordinate, block inside
        // it) -- the entry itself, or a page of the pool and the block inside the page
        auto locate = [&](int nb, int& kb, int& nbl) {
          kb = t.b;
          nbl = nb;
          if constexpr (kGeneral) {
            if (p.page_table != nullptr) {
              const int key0 = nb * kBlockN, pg = key0 / p.page_size;
              kb = p.page_table[(int64_t)t.b * p.pages_per_seq + pg];
              nbl = (key0 - pg * p.page_size) / kBlockN;
            }
          }
        };
        // K runs two blocks ahead of V: QK^T of block i+2 is issued before PV of block i.
        for (int step = 0; ok && step < n + 2; ++step) {
          const int ik = step, iv = step - 2;
          if (ik < n) {
            const uint32_t G = gb + ik, st = G % kStagesK;
            const int nb = (kGeneral ? t.nb_top : n - 1) - ik;
            // stage st is free once QK^T of block G - kStagesK has completed (its s_full phase)
            if (G >= kStagesK) {
              const uint32_t j = G - kStagesK;
              ok = mbar_wait(bars.at(Bars::kSFull + (j % kStagesK)), (j / kStagesK) & 1, wc, kSiteKEmpty);
              if (!ok) break;
            }
            mbar_arrive_expect_tx(bars.at(Bars::kKFull + st), kQkBytes + kQkSfBytes);
            int kb, nbl;
            locate(nb, kb, nbl);
            tma_load_4d(base + kOffK + st * kTileBytes, &tm_k, bars.at(Bars::kKFull + st), 0, t.hk,
                        nbl * kBlockN, kb);
            bulk_load(base + kOffSFK + st * kSfBytes,
                      p.k_sf + kb * p.ksf_stride_b + t.hk * p.ksf_stride_h + (int64_t)nbl * kQkSfBytes,
                      kQkSfBytes, bars.at(Bars::kKFull + st));
            issued_k = G + 1;
          }
          if (iv >= 0 && iv < n) {
            const uint32_t G = gb + iv, st = G % kStagesV;
            const int nb = (kGeneral ? t.nb_top : n - 1) - iv;
            if (G >= kStagesV) {
              const uint32_t j = G - kStagesV;
              ok = mbar_wait(bars.at(Bars::kPvDone + (j % kStagesV)), (j / kStagesV) & 1, wc, kSiteVEmpty);
              if (!ok) break;
            }
            mbar_arrive_expect_tx(bars.at(Bars::kVFull + st), kVBytes + kSfBytes);
            int kb, nbl;
            locate(nb, kb, nbl);
            tma_load_4d(base + kOffV + st * kTileBytes, &tm_v, bars.at(Bars::kVFull + st),
                        nbl * (kBlockN / 2), 0, t.hk, kb);
            bulk_load(base + kOffSFV + st * kSfBytes,
                      p.v_sf + kb * p.vsf_stride_b + t.hk * p.vsf_stride_h + (int64_t)nbl * kSfBytes,
                      kSfBytes, bars.at(Bars::kVFull + st));
            issued_v = G + 1;
          }
        }
        gb += n;
        ti += 1;
      }
      if (!ok) {
        // bounded drain: let the copies already issued land before the CTA's memory is released
        const uint64_t t0 = globaltimer_ns();
        const uint64_t lim = 50ull * 1000 * 1000;
        for (uint32_t i = issued_k > kStagesK ? issued_k - kStagesK : 0; i < issued_k; ++i) {
          while (!mbar_try_wait(bars.at(Bars::kKFull + (i % kStagesK)), (i / kStagesK) & 1) &&
                 globaltimer_ns() - t0 < lim) {}
        }
        for (uint32_t i = issued_v > kStagesV ? issued_v - kStagesV : 0; i < issued_v; ++i) {
          while (!mbar_try_wait(bars.at(Bars::kVFull + (i % kStagesV)), (i / kStagesV) & 1) &&
                 globaltimer_ns() - t0 < lim) {}
        }
        for (uint32_t i = issued_q > 2 ? issued_q - 2 : 0; i < issued_q; ++i) {
          while (!mbar_try_wait(bars.at(Bars::kQFull + (i & 1)), (i >> 1) & 1) && globaltimer_ns() - t0 < lim) {}
        }
      }
    } else if (warp == kIssuerWarp && lane == 0) {
      // ========================================= QK^T issuer ====================================
      FA4_FOR_EACH_TILE {
        const Tile t = decode_tile<kGeneral>(p, tile);
        const int n = t.n_blocks;
        if (n == 0) continue;
        if (status_poisoned(p.status, p.epoch)) {
          *s_abort = 1u;  // another CTA failed: stop this one quickly
          break;
        }
        const uint32_t qb = ti & 1;
        ok = mbar_wait(bars.at(Bars::kQFull + qb), (ti >> 1) & 1, wc, kSiteQFull);
        if (!ok) break;
        tc_fence_after_sync();
        uint64_t dq[kSteps];
#pragma unroll
        for (int j = 0; j < kSteps; ++j) {
          tc_cp_sf(tmem + kTmSFQ + 4 * j, base + kOffSFQ + qb * kSfBytes + 512 * j);
          dq[j] = make_desc_qk<kD>(base + kOffQ + qb * kTileBytes, j);
        }
        for (int i = 0; i < n; ++i) {
          const uint32_t G = gb + i, st = G % kStagesK, b = G & 1;
          if (G >= 2) {
            // S buffer b is free once block G-2 has been read by the stats and softmax warps
            ok = mbar_wait(bars.at(Bars::kSFree + b), ((G - 2) >> 1) & 1, wc, kSiteSFree);
            if (!ok) break;
          }
          ok = mbar_wait(bars.at(Bars::kKFull + st), (G / kStagesK) & 1, wc, kSiteKFull);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t sfk = tmem + kTmSFK + 8 * b;
          const uint32_t ksf = base + kOffSFK + st * kSfBytes, kt = base + kOffK + st * kTileBytes;
          const uint32_t s_tm = tmem + (b ? kTmS1 : kTmS0);
#pragma unroll
          for (int j = 0; j < kSteps; ++j) tc_cp_sf(sfk + 4 * j, ksf + 512 * j);
#pragma unroll
          for (int j = 0; j < kSteps; ++j) {
            mma_nvf4(s_tm, dq[j], make_desc_qk<kD>(kt, j), idesc_qk, tmem + kTmSFQ + 4 * j, sfk + 4 * j,
                     j > 0 ? 1u : 0u);
          }
          tc_commit(bars.at(Bars::kSFull + st));
        }
        if (!ok) break;
        tc_commit(bars.at(Bars::kQEmpty + qb));  // the Q buffer is free once the tile's QK^T have run
        gb += n;
        ti += 1;
      }
      if (!ok) {
        // bounded drain of the tensor-core work already issued, before tensor memory is freed
        const uint64_t t0 = globaltimer_ns();
        tc_commit(bars.at(Bars::kDrain));
        while (!mbar_try_wait(bars.at(Bars::kDrain), 0) && globaltimer_ns() - t0 < 50ull * 1000 * 1000) {}
      }
    } else if (warp == kPvIssuerWarp && lane == 0) {
      // ========================================= PV issuer ======================================
      FA4_FOR_EACH_TILE {
        const Tile t = decode_tile<kGeneral>(p, tile);
        const int n = t.n_blocks;
        if (n == 0) continue;
        if (status_poisoned(p.status, p.epoch)) {
          *s_abort = 1u;  // another CTA failed: stop this one quickly
          break;
        }
        for (int i = 0; i < n; ++i) {
          const uint32_t G = gb + i, st = G % kStagesV, b = G & 1;
          ok = mbar_wait(bars.at(Bars::kVFull + st), (G / kStagesV) & 1, wc, kSiteVFull);
          if (!ok) break;
          ok = mbar_wait(bars.at(Bars::kPFull + (G % kStagesP)), (G / kStagesP) & 1, wc, kSitePFull);
          if (!ok) break;
          if (i == 0 && ti >= 1) {
            // O of the previous tile must have been copied out of tensor memory
            ok = mbar_wait(bars.at(Bars::kOFree), (ti - 1) & 1, wc, kSiteOFree);
            if (!ok) break;
          }
          tc_fence_after_sync();
          const uint32_t sfp = tmem + kTmSFP + 8 * b, sfv = tmem + kTmSFV + 8 * b;
          const uint32_t ps = G % kStagesP;
          const uint32_t psf = base + kOffSFP + ps * kSfBytes, vsf = base + kOffSFV + st * kSfBytes;
          const uint32_t pt = base + kOffP + ps * kTileBytes, vt = base + kOffV + st * kTileBytes;
          tc_cp_sf(sfp, psf);
          tc_cp_sf(sfv, vsf);
          mma_nvf4(tmem + kTmO, make_desc_sw64(pt), make_desc_sw64(vt), idesc_pv, sfp, sfv,
                   i > 0 ? 1u : 0u);
          tc_cp_sf(sfp + 4, psf + 512);
          tc_cp_sf(sfv + 4, vsf + 512);
          mma_nvf4(tmem + kTmO, make_desc_sw64(pt + 32), make_desc_sw64(vt + 32), idesc_pv, sfp + 4,
                   sfv + 4, 1u);
          tc_commit(bars.at(Bars::kPvDone + st));
        }
        if (!ok) break;
        gb += n;
        ti += 1;
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        tc_commit(bars.at(Bars::kDrain + 1));
        while (!mbar_try_wait(bars.at(Bars::kDrain + 1), 0) && globaltimer_ns() - t0 < 50ull * 1000 * 1000) {}
      }
    } else if (warp == kStoreWarp && lane == 0) {
      // ========================================= output store ===================================
      // (the split-KV path writes fp32 partial outputs directly and does not use this role)
      if (!(kGeneral && p.num_splits > 1)) {
        tma_prefetch_desc(&tm_o);
        FA4_FOR_EACH_TILE {
          const Tile t = decode_tile<kGeneral>(p, tile);
          ok = mbar_wait(bars.at(Bars::kOStaged), it & 1, wc, kSiteOStaged);
          if (!ok) break;
#pragma unroll
          for (int bx = 0; bx < kD / 64; ++bx) {
            tma_store_4d(&tm_o, base + kOffOut + bx * 16 * 1024, 64 * bx, t.h, t.m_blk * kBlockM, t.b);
          }
          bulk_commit_group();
          bulk_wait_group_read0();
          mbar_arrive(bars.at(Bars::kStageFree));
          (void)gb;
          (void)ti;
        }
        bulk_wait_group0();  // the last stores complete before the CTA's shared memory goes away
      }
    }
  } else if (warp >= kStatsWarp0) {
    // =========================================== statistics warpgroup ===========================
    // 768 threads launch with 80 registers each (65536 / 768 rounded down to a multiple of 8):
    // a warpgroup that ends up above that must use .inc, below .dec
    if constexpr (kRegsStats > kRegsLaunch) {
      asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsStats));
    } else if constexpr (kRegsStats < kRegsLaunch) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsStats));
    }
    const int row = tid & 127;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    FA4_FOR_EACH_TILE {
      const Tile t = decode_tile<kGeneral>(p, tile);
      const int n = t.n_blocks;
      if (n == 0) continue;
      if (status_poisoned(p.status, p.epoch)) {
          *s_abort = 1u;  // another CTA failed: stop this one quickly
          break;
        }
      float m_run = kNegInf;
      for (int i = 0; i < n; ++i) {
        const uint32_t G = gb + i, b = G & 1;
        const int nb = (kGeneral ? t.nb_top : n - 1) - i;
        const uint32_t bar_s = bars.at(Bars::kSFull + (G % kStagesK)), par_s = (G / kStagesK) & 1;
        const uint32_t bar_f = bars.at(Bars::kStFree + b), par_f = ((G - 2) >> 1) & 1;
        const bool r_s = mbar_test(bar_s, par_s);
        const bool r_f = (G >= 2) ? mbar_test(bar_f, par_f) : true;
        ok = wait_probed(r_s, bar_s, par_s, wc, kSiteSFull);
        if (!ok) break;
        tc_fence_after_sync();
        const bool masked = block_needs_mask<kGeneral, kWindow>(p, t, nb);
        const int limit = causal_limit<kGeneral, kWindow>(p, t, row, nb);
        [[maybe_unused]] const int lower = kWindow ? lower_limit(p, t, row, nb) : 0;
        float bm[8];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float s[32];
          tmem_ld32(lane_addr + (b ? kTmS1 : kTmS0) + 32 * c, reinterpret_cast<uint32_t*>(&s[0]));
          tc_wait_ld();
          if (masked) {
#pragma unroll
            for (int x = 0; x < 32; ++x) {
              bool vis = 32 * c + x <= limit;
              if constexpr (kWindow) vis = vis && (32 * c + x >= lower);
              s[x] = vis ? s[x] : kNegInf;
            }
          }
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            float m0 = fmax3(s[16 * q], s[16 * q + 1], s[16 * q + 2]);
            float m1 = fmax3(s[16 * q + 3], s[16 * q + 4], s[16 * q + 5]);
            m0 = fmax3(m0, s[16 * q + 6], s[16 * q + 7]);
            m1 = fmax3(m1, s[16 * q + 8], s[16 * q + 9]);
            m0 = fmax3(m0, s[16 * q + 10], s[16 * q + 11]);
            m1 = fmax3(m1, s[16 * q + 12], s[16 * q + 13]);
            m0 = fmax3(m0, s[16 * q + 14], s[16 * q + 15]);
            bm[2 * c + q] = fmaxf(m0, m1);
          }
        }
        tc_fence_before_sync();
        mbar_arrive(bars.at(Bars::kSFree + b));
        if constexpr (kGeneral) {
          // tanh is monotone: capping the eight block maxima is capping every score under them
          if (p.softcap_c1 != 0.f) {
#pragma unroll
            for (int q = 0; q < 8; ++q) bm[q] = soft_cap(bm[q], p.softcap_c1);
          }
        }
        const float m01 = fmax3(bm[0], bm[1], bm[2]);
        const float m23 = fmax3(bm[3], bm[4], bm[5]);
        const float m_loc = fmax3(fmaxf(m01, m23), bm[6], bm[7]);
        const float m_new = next_reference(m_run, m_loc, p.sl2);
        // the exponents themselves are derived by the softmax threads, each for its own four
        // blocks: this warpgroup is serial over all blocks of the CTA and publishes as early as
        // it can
        const float m_prev = m_run;
        m_run = m_new;
        // the slot is free once the softmax warpgroups of block G-2 have read it
        ok = wait_probed(r_f, bar_f, par_f, wc, kSiteStFree);
        if (!ok) break;
        uint4* dst = reinterpret_cast<uint4*>(&s_stats[b * 128 + row]);
        dst[0] = make_uint4(__float_as_uint(bm[0]), __float_as_uint(bm[1]), __float_as_uint(bm[2]),
                            __float_as_uint(bm[3]));
        dst[1] = make_uint4(__float_as_uint(bm[4]), __float_as_uint(bm[5]), __float_as_uint(bm[6]),
                            __float_as_uint(bm[7]));
        dst[2] = make_uint4(0u, 0u, __float_as_uint(m_prev), __float_as_uint(m_new));
        mbar_arrive(bars.at(Bars::kStReady + b));
      }
      if (!ok) break;
      gb += n;
      ti += 1;
    }
  } else {
    // =========================================== softmax warpgroups =============================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    const int wg = warp >> 2;          // 0..3
    const int half = wg & 1;           // key columns [64 half, 64 half + 64) of a block
    const uint32_t g = wg >> 1;        // takes the blocks with running index G % 2 == g
    const int row = (warp & 3) * 32 + lane;  // tile row == tensor-memory lane
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);

    FA4_FOR_EACH_TILE {
      const Tile t = decode_tile<kGeneral>(p, tile);
      const int n = t.n_blocks;
      const bool poisoned =
          status_poisoned(p.status, p.epoch);
      if (poisoned) {
        *s_abort = 1u;
        break;
      }
      float m_ref = kNegInf, l_sum = 0.f;

      for (int i = (g - gb) & 1; i < n; i += 2) {
        const uint32_t G = gb + i, b = G & 1;  // b == g: S / P / stats buffer of this block
        const int nb = (kGeneral ? t.nb_top : n - 1) - i;
        // Probe the barriers this block depends on early so that their latencies overlap; the
        // blocking (bounded) wait only runs for a probe that failed.
        const uint32_t bar_r = bars.at(Bars::kStReady + b), par_r = (G >> 1) & 1;
        const uint32_t bar_p = bars.at(Bars::kPvDone + ((G - kStagesP) % kStagesV)),
                       par_p = ((G - kStagesP) / kStagesV) & 1;
        const bool r_p = (G >= kStagesP) ? mbar_test(bar_p, par_p) : true;

        // 1. the statistics of this block are published only after its Q K^T has completed and
        //    been read by the statistics warps (which waited on s_full and fenced), so this one
        //    wait covers the scores as well; it saves a barrier round trip per block
        ok = wait_probed(mbar_test(bar_r, par_r), bar_r, par_r, wc, kSiteStReady);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t s_addr = lane_addr + (b ? kTmS1 : kTmS0) + 64 * half;
        if (block_needs_mask<kGeneral, kWindow>(p, t, nb)) {
          if constexpr (kWindow) {
            mask_scores_in_tmem_range(s_addr, lower_limit(p, t, row, nb) - 64 * half,
                                      causal_limit<true>(p, t, row, nb) - 64 * half);
          } else {
            mask_scores_in_tmem(s_addr, causal_limit<kGeneral, kWindow>(p, t, row, nb) - 64 * half);
          }
        }
        float s[64];
        tmem_ld32(s_addr, reinterpret_cast<uint32_t*>(&s[0]));
        tmem_ld32(s_addr + 32, reinterpret_cast<uint32_t*>(&s[32]));
        // 2. read the statistics while the scores travel
        const uint4* st_row = reinterpret_cast<const uint4*>(&s_stats[b * 128 + row]);
        const uint4 v_bm = st_row[half];
        const uint4 v_misc = st_row[2];
        mbar_arrive(bars.at(Bars::kStFree + b));
        const float m_prev = __uint_as_float(v_misc.z), m_new = __uint_as_float(v_misc.w);
        const float bm4[4] = {__uint_as_float(v_bm.x), __uint_as_float(v_bm.y), __uint_as_float(v_bm.z),
                              __uint_as_float(v_bm.w)};
        float noff4[4];
        uint32_t ue;
        block_exponents4(bm4, m_new, p.sl2, noff4, ue);
        if (m_new != m_ref) l_sum *= reference_factor(m_ref, m_new, p.sl2);
        m_ref = m_new;
        tc_wait_ld();
        tc_fence_before_sync();
        mbar_arrive(bars.at(Bars::kSFree + b));
        if constexpr (kGeneral) {
          if (p.softcap_c1 != 0.f) {
#pragma unroll
            for (int x = 0; x < 64; ++x) s[x] = soft_cap(s[x], p.softcap_c1);
          }
        }

        // 3. exponentials and quantisation; P tile G % kStagesP is free once PV of block
        //    G - kStagesP has completed
        ok = wait_probed(r_p, bar_p, par_p, wc, kSitePvDone);
        if (!ok) break;
        uint8_t* p_tile = gbase + kOffP + (G % kStagesP) * kTileBytes;
        uint4 chunk;
        l_sum += quantize_pair(&s[0], noff4[0], noff4[1],
                               __byte_perm(ue, 0u, 0x4440u), __byte_perm(ue, 0u, 0x4441u), p.sl2, chunk);
        *reinterpret_cast<uint4*>(p_tile + sw64_offset(row, 2 * half)) = chunk;
        l_sum += quantize_pair(&s[32], noff4[2], noff4[3],
                               __byte_perm(ue, 0u, 0x4442u), __byte_perm(ue, 0u, 0x4443u), p.sl2, chunk);
        *reinterpret_cast<uint4*>(p_tile + sw64_offset(row, 2 * half + 1)) = chunk;
        // scales of this half: one 64-key MMA step = scale word `half`
        *reinterpret_cast<uint32_t*>(gbase + kOffSFP + (G % kStagesP) * kSfBytes + 512 * half + (row & 31) * 16 +
                                     (row >> 5) * 4) = block_scale_bytes(ue);

        // 4. correction (rare, out of line, after the scores are consumed): O holds blocks
        //    0..i-1 relative to m_prev and must move to m_new before PV of this block is issued,
        //    i.e. before the arrival on p_full; this warpgroup rescales its 64 columns of O
        if (i > 0 && __any_sync(0xffffffffu, m_new != m_prev)) {
          ok = __all_sync(0xffffffffu, mbar_wait(bars.at(Bars::kPvDone + ((G - 1) % kStagesV)),
                                                 ((G - 1) / kStagesV) & 1, wc, kSitePvDone));
          if (!ok) break;
          tc_fence_after_sync();
          const float f = (m_new != m_prev) ? reference_factor(m_prev, m_new, p.sl2) : 1.f;
          rescale_accumulator(lane_addr + kTmO + (kD / 2) * half, f, kD / 64);
          tc_wait_st();
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();  // orders the O rescale stores before the issuer's next MMA
        mbar_arrive(bars.at(Bars::kPFull + (G % kStagesP)));
      }
      if (!ok) break;

      // ---- tile end: combine the four partial row sums, read O, store ---------------------------
      const int q_idx = t.m_blk * kBlockM + row;
      float scale = 0.f, m_fin = kNegInf, l_tot = 0.f;
      if (n > 0) {
        volatile float* fin_slot = s_fin + (ti & 1) * (4 * 128 * 2);
        // slot order = (parity of the block index inside the tile, half): the summation order of
        // a row then depends on its tile only, not on what the CTA processed before
        const uint32_t slot = (((g ^ gb) & 1u) << 1) | (uint32_t)half;
        fin_slot[(slot * 128 + row) * 2] = l_sum;
        fin_slot[(slot * 128 + row) * 2 + 1] = m_ref;
        mbar_arrive(bars.at(Bars::kFin));
        ok = __all_sync(0xffffffffu, mbar_wait(bars.at(Bars::kFin), ti & 1, wc, kSiteFin));
        if (!ok) break;
        float lw[4], mw[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          lw[w] = fin_slot[(w * 128 + row) * 2];
          mw[w] = fin_slot[(w * 128 + row) * 2 + 1];
          m_fin = fmaxf(m_fin, mw[w]);
        }
#pragma unroll
        for (int w = 0; w < 4; ++w) l_tot += lw[w] * reference_factor(mw[w], m_fin, p.sl2);
        if (m_fin == kNegInf) l_tot = 0.f;
        if constexpr (kGeneral) {
          // the sink joins the row sum once (split 0), relative to the row's reference maximum
          if (p.sink != nullptr && t.split == 0 && m_fin != kNegInf) {
            l_tot += ex2_approx(static_cast<float>(kShift) + p.sink[t.h] * 1.4426950408889634f -
                                m_fin * p.sl2);
          }
        }
        const uint32_t Gl = gb + n - 1;
        ok = __all_sync(0xffffffffu,
                        mbar_wait(bars.at(Bars::kPvDone + (Gl % kStagesV)), (Gl / kStagesV) & 1, wc, kSiteFinalO));
        if (!ok) break;
        tc_fence_after_sync();
        scale = (l_tot > 0.f) ? p.out_scale / l_tot : 0.f;
      }
      // warpgroup k stores output columns [32 k, 32 k + 32); with kD = 64 two of them only arrive
      if (kGeneral && p.num_splits > 1 && (kD == 128 || wg < kD / 32)) {
        float* prow = p.o_partial +
                      ((((int64_t)t.split * p.B + t.b) * p.Sq + q_idx) * p.Hq + t.h) * kD + 32 * wg;
        store_accumulator_partial(lane_addr + kTmO + 32 * wg, q_idx < p.Sq ? prow : nullptr, scale,
                                  n > 0 ? bars.at(Bars::kOFree) : 0u);
      } else {
        if (it >= 1) {
          // the staging tile is free once the store warp's TMA has read the previous tile out of it
          ok = __all_sync(0xffffffffu, mbar_wait(bars.at(Bars::kStageFree), (it - 1) & 1, wc, kSiteStageFree));
          if (!ok) break;
        }
        if (kD == 128 || wg < kD / 32) {
          stage_accumulator_chunk<true>(lane_addr + kTmO + 32 * wg, gbase + kOffOut, row, wg, scale,
                                        n > 0 ? bars.at(Bars::kOFree) : 0u);
        } else {
          stage_accumulator_chunk<false>(0u, gbase + kOffOut, row, wg, 0.f, n > 0 ? bars.at(Bars::kOFree) : 0u);
        }
        fence_proxy_async_smem();
        mbar_arrive(bars.at(Bars::kOStaged));
      }
      if (wg == 0 && q_idx < p.Sq) {
        float lse_v = finish_lse(m_fin, l_tot, p.sl2);
        if constexpr (kGeneral) {
          // a row without visible keys still has its sink: LSE = sink, output zero
          if (p.sink != nullptr && t.split == 0 && m_fin == kNegInf) lse_v = p.sink[t.h];
        }
        if (kGeneral && p.num_splits > 1) {
          p.lse_partial[(((int64_t)t.split * p.B + t.b) * p.Hq + t.h) * p.Sq + q_idx] = lse_v;
        } else if (p.lse != nullptr) {
          p.lse[((int64_t)t.b * p.Hq + t.h) * p.Sq + q_idx] = lse_v;
        }
      }
      gb += n;
      ti += (n > 0) ? 1u : 0u;
    }
  }
#undef FA4_FOR_EACH_TILE

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kIssuerWarp) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace fa4
