// Warp-specialised kernel with 64-key sub-blocks and FOUR score buffers (split-KV and KV-cache views
// stay with attn_ws.cuh).
//
// The kernel of attn_ws.cuh keeps two 128-column S buffers in tensor memory and lets two pairs of
// softmax warpgroups alternate over the 128-key blocks, a thread owning half a row.  The two
// warpgroups of a pair move in lockstep, so a scheduler sees only two independent softmax
// "strands", each with ~1000 clocks of exponentials and ~2000 clocks of latency-bound prologue /
// epilogue per block: the exponential unit idles ~40 % of the time, and every tile end drains
// the pipeline while the softmax warps read the accumulator out.
//
// Here a K/V block of 128 keys is processed as two sub-blocks of 64 keys, S has four buffers of 64
// columns (the same 256 tensor-memory columns), and each of the four softmax warpgroups owns one
// buffer: a thread holds the 64 scores of one WHOLE row of one sub-block -- the same register
// footprint -- so it takes the maxima itself (no statistics warpgroup), and the four warpgroups
// are independent strands at different phases.
//
//   warps 0-15  softmax: warpgroup w takes the sub-blocks with running index J % 4 == w; the
//               running reference maximum of a row is handed from the warpgroup of sub-block
//               J - 1 to that of J through shared memory
//   warp 16     TMA producer (Q double buffered, K / V rings of 128-key tiles)
//   warp 17     QK^T issuer: per K tile one N = 128 product into two neighbouring S buffers
//   warp 18     P V issuer: per sub-block one K = 64 step into O
//   warp 19     copies the K / V scale tiles into tensor memory as they land
//   warps 20-23 epilogue: combine the partial row sums, read O out, TMA store, LSE -- while the
//               softmax warpgroups already work on the next tile
//
// Sub-block j of a tile (visit order): keys 64 j .. 64 j + 63, ascending.  (The 128-key kernel
// visits the last visible block first; with 64-key steps that order makes the first references
// of a causal tile rest on one or two keys, and with the small lazy threshold that NVFP4 block
// scales allow nearly every tile then pays several accumulator corrections, each of which
// drains the P V pipeline.  Ascending, the first sub-block is fully visible.)
// J = 2 * (blocks before this tile) + j selects buffers, P slots and barrier phases.  Operand
// formats, P quantisation, lazy reference and bounded waits are those of attn_ws.cuh.
#pragma once
#include "attn_ws.cuh"

namespace fa4 {
namespace ws64 {

constexpr int kStagesK = 4, kStagesV = 4;  // 128-key tiles
constexpr int kSBufs = 4;                  // S buffers of 64 columns
constexpr int kPSlots = 8;                 // P tiles of 64 keys (4 KB each)
constexpr int kThreads = 768;
constexpr int kProducerWarp = 16, kIssuerWarp = 17, kPvIssuerWarp = 18, kCopyWarp = 19, kEpilogueWarp0 = 20;
// Registers are a per-scheduler resource: 16384 per SM sub-partition, warp w living on sub-partition
// w % 4.  With 21-24 warps a sub-partition holds 6, so the launch gets 80 registers per thread and
// the CTA's pool per sub-partition is 6 x 32 x 80 = 15360.  setmaxnreg.inc draws from that pool
// (NOT from the whole register file) and blocks until it can be served: a budget above the pool
// never returns.  Per sub-partition: four softmax warps at 96, one service warp at 40 and one
// epilogue warp at 56 use exactly the pool.
constexpr int kRegsSoftmax = 96, kRegsOther = 40, kRegsEpilogue = 56, kRegsLaunch = 80;
static_assert(kThreads == 768, "six warps per sub-partition");
static_assert(4 * kRegsSoftmax + kRegsOther + kRegsEpilogue <= 6 * kRegsLaunch,
              "register pool of a sub-partition");
static_assert((kThreads / 128) * 32 * kRegsLaunch <= 16384, "register file of a sub-partition");

// tensor memory: S[4] x 64 columns, O 128, scale factors
// (O at column 256 and Q scales at 384 as in the 128-key kernel); K and V scales have one slot of
// 8 columns per shared-memory stage, written by the copy warp as soon as the tile has landed
// (sized for head dim 192: three 64-element steps, 12 scale columns per Q / K tile)
constexpr uint32_t kTmS64 = 0, kTmSFQ64 = 384 /* 12 */, kTmSFK64 = 396 /* 4 x 12 */, kTmSFV64 = 444 /* 4 x 8 */,
                   kTmSFP64 = 476 /* 4 x 4 */;
static_assert(kTmSFP64 + 16 <= 512, "tensor memory columns");
// shared-memory slots of a Q / K tile and of its scales, sized for head dim 192 (128 rows of 96
// bytes as three 32-byte-wide sub-tiles; three scale chunks)
constexpr uint32_t kQkSlot = 128 * 96, kQkSfSlot = 3 * 512;
constexpr uint32_t kSlackNs = 500;         // suspend hint of the waits of roles with slack
constexpr uint32_t kPTileBytes = 128 * 32;  // 128 rows x 64 e2m1 keys

constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffK = kOffQ + 2 * kQkSlot;
constexpr uint32_t kOffV = kOffK + kStagesK * kQkSlot;
constexpr uint32_t kOffP = kOffV + kStagesV * kTileBytes;
constexpr uint32_t kOffSFQ = kOffP + kPSlots * kPTileBytes;
constexpr uint32_t kOffSFK = kOffSFQ + 2 * kQkSfSlot;
constexpr uint32_t kOffSFV = kOffSFK + kStagesK * kQkSfSlot;
constexpr uint32_t kOffSFP = kOffSFV + kStagesV * kSfBytes;      // kPSlots x 512
constexpr uint32_t kOffOut = kOffSFP + kPSlots * 512;            // 32 KB staging tile
constexpr uint32_t kOffHand = kOffOut + 32 * 1024;               // kSBufs x 128 reference maxima
constexpr uint32_t kOffFin = kOffHand + kSBufs * 128 * 4;        // 2 tiles x 4 WGs x 128 x (sum, ref)
constexpr uint32_t kOffBar = kOffFin + 2 * 4 * 128 * 8;

struct Bars {
  uint32_t base;
  static constexpr uint32_t kQFull = 0, kQEmpty = 2, kKFull = 4, kVFull = kKFull + kStagesK,
                            kKFree = kVFull + kStagesV, kVFree = kKFree + kStagesK,
                            kSFull = kVFree + kStagesV, kSFree = kSFull + kSBufs,
                            kHand = kSFree + kSBufs, kPFull = kHand + 4 * kSBufs, kPvDone = kPFull + kPSlots,
                            kFin = kPvDone + kPSlots, kFinFree = kFin + 2, kOFree = kFinFree + 2,
                            kEpi = kOFree + 1, kKsf = kEpi + 1, kVsf = kKsf + kStagesK,
                            kDrain = kVsf + kStagesV, kCount = kDrain + 3;
  __device__ explicit Bars(uint32_t b) : base(b) {}
  __device__ __forceinline__ uint32_t at(uint32_t idx) const { return base + 8u * idx; }
};
constexpr uint32_t kOffMisc = kOffBar + 8 * Bars::kCount;
constexpr uint32_t kSmemUsed = kOffMisc + 16;
constexpr uint32_t kSmemRequest = kSmemUsed + 1024;
static_assert(kSmemRequest <= 227 * 1024, "shared memory");

enum Site64 {
  kS64QFull = 40, kS64QEmpty, kS64KFree, kS64VFree, kS64KFull, kS64VFull, kS64SFull, kS64SFree,
  kS64PFull, kS64PvDone, kS64Hand, kS64Fin, kS64FinFree, kS64FinalO, kS64OFree, kS64Ksf, kS64Vsf, kS64Epi
};

// Visit order of a windowed tile: the i-th visited 128-key block.  Ascending from the first block
// the window reaches, EXCEPT that the two blocks at the window's left edge -- where the lower rows
// of the tile see a few keys or none, so that references taken there would be low -- are visited
// last: a tile starts at a block every row sees whole.  (The right edge, the diagonal, is last in
// ascending order anyway.)  rotate: the tile is cut on the left and has more than two blocks.
__device__ __forceinline__ int window_visit_block(int i, int n, int nb_lo, bool rotate) {
  if (!rotate) return nb_lo + i;
  return i < n - 2 ? nb_lo + 2 + i : nb_lo + (i - (n - 2));
}
__device__ __forceinline__ bool window_rotates(const KernelParams& p, const Tile& t) {
  return p.win_left >= 0 && t.n_blocks > 2 && (t.m_blk * kBlockM + t.sk - t.sq - p.win_left) > 0;
}

// byte offset of 16-byte chunk c (0, 1) of row r in a P tile (rows of 32 bytes, 32-byte swizzle)
__device__ __forceinline__ uint32_t sw32_offset(uint32_t row, uint32_t chunk) {
  return row * 32u + ((chunk ^ ((row >> 2) & 1u)) << 4);
}

}  // namespace ws64

// kD: head dimension of Q, K and V (128 or 64).  It sets the number of 64-element steps of Q K^T,
// the bytes of a Q / K tile (128 rows of kD / 2 bytes: 64-byte-swizzled rows for 128, 32-byte for
// 64) and of a V tile (kD rows of 128 keys), and the width of O.  Shared and tensor memory are
// laid out for 128 either way.
// kGeneral adds sliding windows (the block range starts at the first block the window reaches, both
// limits are masked), the learnable sink (one more term of the row sum, in the epilogue) and the
// soft cap (tanh on the raw scores); a compile-time switch so that the plain instantiation carries
// none of it.  The window instantiation also serves KV-cache views (per-entry key counts, page
// tables); split-KV stays with attn_ws.cuh.
// (kWindow separates the two halves of it: the window changes the tile geometry and the masks of
// the hot loop, sink and soft cap do not -- a call with only those keeps the plain geometry code,
// which measured 16 % faster than carrying the window arithmetic along.)
// kCache: per-entry key counts and page tables without the window arithmetic.
template <int kD, bool kGeneral = false, bool kWindow = kGeneral, bool kCache = kWindow>
__global__ void __launch_bounds__(ws64::kThreads, 1)
attn_fwd_ws64_kernel(const __grid_constant__ CUtensorMap tm_q,
                     const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v,
                     const __grid_constant__ CUtensorMap tm_o, const KernelParams p) {
  using namespace ws64;
  using ws::rescale_accumulator;
  using ws::mask_scores_in_tmem;
  using ws::stage_accumulator_chunk;
  using ws::tile_of_round;
  using ws::wait_probed;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  const Bars bars(base + kOffBar);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + kOffMisc);
  volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(gbase + kOffMisc + 4);
  volatile float* s_hand = reinterpret_cast<volatile float*>(gbase + kOffHand);  // [4][128]
  volatile float* s_fin = reinterpret_cast<volatile float*>(gbase + kOffFin);    // [2][4][128][2]

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const WaitCtx wc{s_abort, p.status, p.budget_ns, p.epoch};
  const int num_tiles = p.num_m_blocks * p.Hq * p.B;
  const int ncta = gridDim.x, cta = blockIdx.x;

  if (tid == 0) {
    *s_abort = 0u;
    for (int b = 0; b < 2; ++b) {
      mbar_init(bars.at(Bars::kQFull + b), 1);
      mbar_init(bars.at(Bars::kQEmpty + b), 1);
    }
    for (int b = 0; b < 3; ++b) mbar_init(bars.at(Bars::kDrain + b), 1);
    for (int s = 0; s < kStagesK; ++s) {
      mbar_init(bars.at(Bars::kKFull + s), 1);
      mbar_init(bars.at(Bars::kKFree + s), 1);
      mbar_init(bars.at(Bars::kKsf + s), 1);
    }
    for (int s = 0; s < kStagesV; ++s) {
      mbar_init(bars.at(Bars::kVFull + s), 1);
      mbar_init(bars.at(Bars::kVFree + s), 1);
      mbar_init(bars.at(Bars::kVsf + s), 1);
    }
    for (int s = 0; s < kSBufs; ++s) {
      mbar_init(bars.at(Bars::kSFull + s), 1);
      mbar_init(bars.at(Bars::kSFree + s), 128);    // the softmax warpgroup that owns the buffer
      for (int q = 0; q < 4; ++q) mbar_init(bars.at(Bars::kHand + 4 * s + q), 32);  // per warp quarter
    }
    for (int s = 0; s < kPSlots; ++s) {
      mbar_init(bars.at(Bars::kPFull + s), 128);
      mbar_init(bars.at(Bars::kPvDone + s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bars.at(Bars::kFin + b), 512);      // the four softmax warpgroups
      mbar_init(bars.at(Bars::kFinFree + b), 128);  // the epilogue warpgroup
    }
    mbar_init(bars.at(Bars::kOFree), 128);
    mbar_init(bars.at(Bars::kEpi), 128);            // the epilogue warpgroup's own rendezvous
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
  static_assert(kD == 128 || kD == 64 || kD == 192, "head dimensions built: 128, 64 and (192, 128)");
  constexpr int kDv = kD == 192 ? 128 : kD;            // head dim of V and O
  constexpr uint32_t idesc_qk = make_idesc_nvf4(128, 128);
  constexpr uint32_t idesc_pv = make_idesc_nvf4(128, kDv);
  constexpr int kSteps = kD / 64;                      // 64-element steps of Q K^T
  constexpr uint32_t kQkBytes = 128u * kD / 2;         // bytes of a Q or K tile
  constexpr uint32_t kQkSfBytes = kSteps * 512u;       // its scale chunks (128 rows x kD / 16)
  constexpr uint32_t kVBytes = kDv * 64u;              // V tile: kDv rows of 128 keys
  // A Q / K tile in shared memory: one 64-byte-swizzled box for head dim 128; for 64 and 192 one or
  // three 32-byte-wide boxes (32-byte swizzle, 4 KB each), one per 64-element step.
  auto load_qk_tile = [&](uint32_t dst, const CUtensorMap* tm, uint32_t bar, int h, int row, int b) {
    if constexpr (kD == 128) {
      tma_load_4d(dst, tm, bar, 0, h, row, b);
    } else {
#pragma unroll
      for (int j = 0; j < kSteps; ++j) tma_load_4d(dst + 4096 * j, tm, bar, 32 * j, h, row, b);
    }
  };
  auto desc_qk = [&](uint32_t tile, int j) -> uint64_t {
    if constexpr (kD == 128) return make_desc_sw64(tile + 32 * j);
    return make_desc_sw32(tile + 4096 * j);
  };

#define FA4_FOR_EACH_TILE                                                                        \
  uint32_t gb = 0, ti = 0;                                                                       \
  bool ok = true;                                                                                \
  for (int it = 0, tile = tile_of_round(0, cta, ncta); ok && tile < num_tiles;                   \
       ++it, tile = tile_of_round(it, cta, ncta))

  if (warp >= kEpilogueWarp0) {
    // =========================================== epilogue warpgroup =============================
    // Thread = row.  Per tile: combine the four partial row sums, wait for the last P V, move O
    // from tensor memory to the staging tile (bf16, normalised), send it with TMA, write the LSE.
    // The softmax warpgroups meanwhile work on the next tile; only the P V issuer waits for the
    // accumulator to be read out.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsEpilogue));
    const int row = tid & 127;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const bool leader = (tid == kEpilogueWarp0 * 32);
    if (leader) tma_prefetch_desc(&tm_o);
    // rendezvous of the 128 epilogue threads on an mbarrier: unlike bar.sync the wait is bounded, so
    // a warp that gave up elsewhere cannot leave the others blocked
    uint32_t epi_phase = 0;
#define FA4_EPI_SYNC()                                                                              \
  mbar_arrive(bars.at(Bars::kEpi));                                                                 \
  ok = __all_sync(0xffffffffu, mbar_wait(bars.at(Bars::kEpi), epi_phase & 1, wc, kS64Epi));          \
  epi_phase += 1;                                                                                   \
  if (!ok) break;
    FA4_FOR_EACH_TILE {
      const Tile t = decode_tile<kWindow || kCache>(p, tile);
      const int n = t.n_blocks;
      const int q_idx = t.m_blk * kBlockM + row;
      if constexpr (kWindow || kCache) {
        // a tile past the end of a short sequence of a packed batch has no rows at all
        if (t.m_blk * kBlockM >= t.sq) continue;
      }
      float scale = 0.f, m_fin = kNegInf, l_tot = 0.f;
      if (n > 0) {
        const uint32_t fb = ti & 1;
        ok = __all_sync(0xffffffffu, mbar_wait_relaxed<kSlackNs>(bars.at(Bars::kFin + fb), (ti >> 1) & 1, wc, kS64Fin));
        if (!ok) break;
        volatile float* fin_slot = s_fin + fb * (4 * 128 * 2);
        float lw[4], mw[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          lw[w] = fin_slot[(w * 128 + row) * 2];
          mw[w] = fin_slot[(w * 128 + row) * 2 + 1];
          m_fin = fmaxf(m_fin, mw[w]);
        }
        mbar_arrive(bars.at(Bars::kFinFree + fb));
#pragma unroll
        for (int w = 0; w < 4; ++w) l_tot += lw[w] * reference_factor(mw[w], m_fin, p.sl2);
        if (m_fin == kNegInf) l_tot = 0.f;
        if constexpr (kGeneral) {
          // the sink joins the row sum, relative to the row's reference maximum
          if (p.sink != nullptr && m_fin != kNegInf) {
            l_tot += ex2_approx(static_cast<float>(kShift) + p.sink[t.h] * 1.4426950408889634f - m_fin * p.sl2);
          }
        }
        const uint32_t Jl = 2 * gb + 2 * n - 1;
        ok = __all_sync(0xffffffffu,
                        mbar_wait(bars.at(Bars::kPvDone + (Jl % kPSlots)), (Jl / kPSlots) & 1, wc, kS64FinalO));
        if (!ok) break;
        tc_fence_after_sync();
        scale = (l_tot > 0.f) ? p.out_scale / l_tot : 0.f;
      }
      // the staging tile is free once the previous store has read it
      if (it >= 1) {
        if (leader) bulk_wait_group_read0();
        FA4_EPI_SYNC()
      }
#pragma unroll 1
      for (int c = 0; c < kDv / 32; ++c) {
        uint8_t* box_row = gbase + kOffOut + (c >> 1) * (16 * 1024) + row * 128;
        uint32_t o[32];
        if (n > 0) {
          tmem_ld32(lane_addr + kTmO + 32 * c, o);
          tc_wait_ld();
          if (c == kDv / 32 - 1) {
            tc_fence_before_sync();
            mbar_arrive(bars.at(Bars::kOFree));  // the P V issuer may start the next tile
          }
        } else {
#pragma unroll
          for (int x = 0; x < 32; ++x) o[x] = 0u;
        }
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(o[8 * v + 0]) * scale, __uint_as_float(o[8 * v + 1]) * scale);
          w.y = pack_bf16x2(__uint_as_float(o[8 * v + 2]) * scale, __uint_as_float(o[8 * v + 3]) * scale);
          w.z = pack_bf16x2(__uint_as_float(o[8 * v + 4]) * scale, __uint_as_float(o[8 * v + 5]) * scale);
          w.w = pack_bf16x2(__uint_as_float(o[8 * v + 6]) * scale, __uint_as_float(o[8 * v + 7]) * scale);
          const int chunk = ((c & 1) * 4 + v) ^ (row & 7);
          *reinterpret_cast<uint4*>(box_row + chunk * 16) = w;
        }
      }
      fence_proxy_async_smem();
      FA4_EPI_SYNC()
      const int sq = query_len<kWindow || kCache>(p, t);
      const bool packed = (kWindow || kCache) && p.cu_seqlens_q != nullptr;
      if (packed && (t.m_blk + 1) * kBlockM > sq) {
        // last, partial tile of a packed sequence: a tiled store would run into the rows of the
        // next sequence (the tensor map only clips at the end of the whole batch), so every
        // thread copies its own row from the staging tile, if it has one
        if (q_idx < sq) {
          __nv_bfloat16* orow = p.out + (int64_t)(t.q0 + q_idx) * p.o_stride_s + (int64_t)t.h * p.o_stride_h;
#pragma unroll
          for (int c16 = 0; c16 < kDv / 8; ++c16) {
            const uint8_t* src = gbase + kOffOut + (c16 >> 3) * (16 * 1024) + row * 128 + (((c16 & 7) ^ (row & 7)) << 4);
            reinterpret_cast<uint4*>(orow)[c16] = *reinterpret_cast<const uint4*>(src);
          }
        }
      } else if (leader) {
#pragma unroll
        for (int bx = 0; bx < kDv / 64; ++bx) {
          tma_store_4d(&tm_o, base + kOffOut + bx * 16 * 1024, 64 * bx, t.h, t.q0 + t.m_blk * kBlockM,
                       packed ? 0 : t.b);
        }
        bulk_commit_group();
      }
      if (q_idx < sq && p.lse != nullptr) {
        float lse_v = finish_lse(m_fin, l_tot, p.sl2);
        if constexpr (kGeneral) {
          // a row without visible keys still has its sink: LSE = sink, output zero
          if (p.sink != nullptr && m_fin == kNegInf) lse_v = p.sink[t.h];
        }
        if (packed) {
          p.lse[(int64_t)t.h * p.total_q + t.q0 + q_idx] = lse_v;   // (Hq, total_q)
        } else {
          p.lse[((int64_t)t.b * p.Hq + t.h) * p.Sq + q_idx] = lse_v;
        }
      }
      gb += n;
      ti += (n > 0) ? 1u : 0u;
    }
#undef FA4_EPI_SYNC
    if (leader) bulk_wait_group0();
  } else if (warp >= kProducerWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
    if (warp == kProducerWarp && lane == 0) {
      // ========================================= TMA producer ===================================
      uint32_t issued_k = 0, issued_v = 0, issued_q = 0;
      FA4_FOR_EACH_TILE {
        const Tile t = decode_tile<kWindow || kCache, kWindow || kCache>(p, tile);
        const int n = t.n_blocks;
        if (n == 0) continue;
        if (status_poisoned(p.status, p.epoch)) {
          // another CTA of this launch failed: stop this one quickly.  Only this role polls the
          // status word (a global load at every tile start); the others see the abort flag in
          // their next wait, when the tiles stop coming
          *s_abort = 1u;
          break;
        }
        const uint32_t qb = ti & 1;
        if (ti >= 2) {
          ok = mbar_wait_relaxed<kSlackNs>(bars.at(Bars::kQEmpty + qb), ((ti - 2) >> 1) & 1, wc, kS64QEmpty);
          if (!ok) break;
        }
        mbar_arrive_expect_tx(bars.at(Bars::kQFull + qb), kQkBytes + kQkSfBytes);
        // a packed batch has no batch dimension: the sequence's first row is added to the row
        // coordinate instead (the scale tiles stay per sequence)
        const bool packed = (kWindow || kCache) && p.cu_seqlens_q != nullptr;
        load_qk_tile(base + kOffQ + qb * kQkSlot, &tm_q, bars.at(Bars::kQFull + qb), t.h,
                     t.q0 + t.m_blk * kBlockM, packed ? 0 : t.b);
        bulk_load(base + kOffSFQ + qb * kQkSfSlot,
                  p.q_sf + t.b * p.qsf_stride_b + t.h * p.qsf_stride_h + (int64_t)t.m_blk * kQkSfBytes,
                  kQkSfBytes, bars.at(Bars::kQFull + qb));
        issued_q = ti + 1;
        // where logical K/V block nb of this batch entry lives: the entry itself, or (window
        // instantiation, which also serves KV-cache views) a page of the pool and the block in it
        auto locate = [&](int nb, int& kb, int& nbl) {
          kb = t.b;
          nbl = nb;
          if constexpr (kWindow || kCache) {
            if (p.page_table != nullptr) {
              const int key0 = nb * kBlockN, pg = key0 / p.page_size;
              kb = p.page_table[(int64_t)t.b * p.pages_per_seq + pg];
              nbl = (key0 - pg * p.page_size) / kBlockN;
            }
          }
        };
        // K runs two blocks ahead of V
        for (int step = 0; ok && step < n + 2; ++step) {
          const int ik = step, iv = step - 2;
          if (ik < n) {
            const uint32_t G = gb + ik, st = G % kStagesK;
            const int nb = kWindow ? window_visit_block(ik, n, t.nb_top - n + 1, window_rotates(p, t)) : ik;  // ascending
            if (G >= kStagesK) {
              ok = mbar_wait_relaxed<kSlackNs>(bars.at(Bars::kKFree + st), ((G - kStagesK) / kStagesK) & 1, wc, kS64KFree);
              if (!ok) break;
            }
            mbar_arrive_expect_tx(bars.at(Bars::kKFull + st), kQkBytes + kQkSfBytes);
            int kb, nbl;
            locate(nb, kb, nbl);
            load_qk_tile(base + kOffK + st * kQkSlot, &tm_k, bars.at(Bars::kKFull + st), t.hk,
                         t.k0 + nbl * kBlockN, packed ? 0 : kb);
            bulk_load(base + kOffSFK + st * kQkSfSlot,
                      p.k_sf + kb * p.ksf_stride_b + t.hk * p.ksf_stride_h + (int64_t)nbl * kQkSfBytes,
                      kQkSfBytes, bars.at(Bars::kKFull + st));
            issued_k = G + 1;
          }
          if (iv >= 0 && iv < n) {
            const uint32_t G = gb + iv, st = G % kStagesV;
            const int nb = kWindow ? window_visit_block(iv, n, t.nb_top - n + 1, window_rotates(p, t)) : iv;
            if (G >= kStagesV) {
              ok = mbar_wait_relaxed<kSlackNs>(bars.at(Bars::kVFree + st), ((G - kStagesV) / kStagesV) & 1, wc, kS64VFree);
              if (!ok) break;
            }
            mbar_arrive_expect_tx(bars.at(Bars::kVFull + st), kVBytes + kSfBytes);
            int kb, nbl;
            locate(nb, kb, nbl);
            tma_load_4d(base + kOffV + st * kTileBytes, &tm_v, bars.at(Bars::kVFull + st),
                        (t.v0 + nbl * kBlockN) / 2, 0, t.hk, packed ? 0 : kb);
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
        const Tile t = decode_tile<kWindow || kCache, kWindow || kCache>(p, tile);
        const int n = t.n_blocks;
        if (n == 0) continue;
        const uint32_t qb = ti & 1;
        ok = mbar_wait(bars.at(Bars::kQFull + qb), (ti >> 1) & 1, wc, kS64QFull);
        if (!ok) break;
        tc_fence_after_sync();
        uint64_t dq[kSteps];
#pragma unroll
        for (int ks = 0; ks < kSteps; ++ks) {
          tc_cp_sf(tmem + kTmSFQ64 + 4 * ks, base + kOffSFQ + qb * kQkSfSlot + 512 * ks);
          dq[ks] = desc_qk(base + kOffQ + qb * kQkSlot, ks);
        }
        for (int i = 0; ok && i < n; ++i) {
          const uint32_t G = gb + i, st = G % kStagesK;
          // the K tile has landed (the copy warp saw k_full) and its scales are in tensor memory
          ok = mbar_wait(bars.at(Bars::kKsf + st), (G / kStagesK) & 1, wc, kS64Ksf);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t sfk = tmem + kTmSFK64 + 12 * st;
          const uint32_t kt = base + kOffK + st * kQkSlot;
          // one product of N = 128 fills the two neighbouring S buffers of sub-blocks 2G and 2G + 1
          // (keys 0-63 and 64-127 of the tile): half the tcgen05 instructions of two N = 64
          // products, and the in-order issue slots of this thread are scarce
          const uint32_t J0 = 2 * G, b0 = J0 % kSBufs;  // 0 or 2
          if (J0 >= kSBufs) {
            ok = mbar_wait(bars.at(Bars::kSFree + b0), ((J0 - kSBufs) / kSBufs) & 1, wc, kS64SFree) &&
                 mbar_wait(bars.at(Bars::kSFree + b0 + 1), ((J0 - kSBufs) / kSBufs) & 1, wc, kS64SFree);
            if (!ok) break;
            tc_fence_after_sync();
          }
#pragma unroll
          for (int ks = 0; ks < kSteps; ++ks) {
            mma_nvf4(tmem + kTmS64 + 64 * b0, dq[ks], desc_qk(kt, ks), idesc_qk,
                     tmem + kTmSFQ64 + 4 * ks, sfk + 4 * ks, ks > 0 ? 1u : 0u);
          }
          tc_commit(bars.at(Bars::kSFull + b0));  // both softmax warpgroups of the pair wait on it
          tc_commit(bars.at(Bars::kKFree + st));  // the K stage is free once both products have run
        }
        if (!ok) break;
        tc_commit(bars.at(Bars::kQEmpty + qb));
        gb += n;
        ti += 1;
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        tc_commit(bars.at(Bars::kDrain));
        while (!mbar_try_wait(bars.at(Bars::kDrain), 0) && globaltimer_ns() - t0 < 50ull * 1000 * 1000) {}
      }
    } else if (warp == kPvIssuerWarp && lane == 0) {
      // ========================================= P V issuer =====================================
      FA4_FOR_EACH_TILE {
        const Tile t = decode_tile<kWindow || kCache, kWindow || kCache>(p, tile);
        const int n = t.n_blocks;
        if (n == 0) continue;
        for (int i = 0; ok && i < n; ++i) {
          const uint32_t G = gb + i, st = G % kStagesV;
          ok = mbar_wait(bars.at(Bars::kVsf + st), (G / kStagesV) & 1, wc, kS64Vsf);
          if (!ok) break;
          const uint32_t vt = base + kOffV + st * kTileBytes;
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const uint32_t J = 2 * G + s, slot = J % kPSlots, tb = J % kSBufs;
            const uint32_t h64 = s;
            ok = mbar_wait(bars.at(Bars::kPFull + slot), (J / kPSlots) & 1, wc, kS64PFull);
            if (!ok) break;
            if (i == 0 && s == 0 && ti >= 1) {
              // O of the previous tile must have been copied out of tensor memory
              ok = mbar_wait(bars.at(Bars::kOFree), (ti - 1) & 1, wc, kS64OFree);
              if (!ok) break;
            }
            tc_fence_after_sync();
            const uint32_t sfp = tmem + kTmSFP64 + 4 * tb, sfv = tmem + kTmSFV64 + 8 * st + 4 * h64;
            tc_cp_sf(sfp, base + kOffSFP + slot * 512);
            mma_nvf4(tmem + kTmO, make_desc_sw32(base + kOffP + slot * kPTileBytes),
                     make_desc_sw64(vt + 32 * h64), idesc_pv, sfp, sfv, (i > 0 || s > 0) ? 1u : 0u);
            tc_commit(bars.at(Bars::kPvDone + slot));
          }
          if (!ok) break;
          tc_commit(bars.at(Bars::kVFree + st));
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
    } else if (warp == kCopyWarp && lane == 0) {
      // ========================================= scale copier ===================================
      // moves the K and V scale tiles of every stage into tensor memory as soon as they land, so
      // that the two issuers spend their (slow, in-order) tcgen05 issue slots on products only.
      // A stage's tensor-memory slot is free when its shared-memory stage is: the producer
      // reloads the stage only after the products that used it have completed.
      FA4_FOR_EACH_TILE {
        const Tile t = decode_tile<kWindow || kCache, kWindow || kCache>(p, tile);
        const int n = t.n_blocks;
        if (n == 0) continue;
        for (int step = 0; ok && step < n + 2; ++step) {
          const int ik = step, iv = step - 2;  // the producer's order
          if (ik < n) {
            const uint32_t G = gb + ik, st = G % kStagesK;
            ok = mbar_wait_relaxed<kSlackNs>(bars.at(Bars::kKFull + st), (G / kStagesK) & 1, wc, kS64KFull);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t ksf = base + kOffSFK + st * kQkSfSlot;
#pragma unroll
            for (int ks = 0; ks < kSteps; ++ks) tc_cp_sf(tmem + kTmSFK64 + 12 * st + 4 * ks, ksf + 512 * ks);
            tc_commit(bars.at(Bars::kKsf + st));
          }
          if (iv >= 0 && iv < n) {
            const uint32_t G = gb + iv, st = G % kStagesV;
            ok = mbar_wait_relaxed<kSlackNs>(bars.at(Bars::kVFull + st), (G / kStagesV) & 1, wc, kS64VFull);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t vsf = base + kOffSFV + st * kSfBytes;
            tc_cp_sf(tmem + kTmSFV64 + 8 * st, vsf);
            tc_cp_sf(tmem + kTmSFV64 + 8 * st + 4, vsf + 512);
            tc_commit(bars.at(Bars::kVsf + st));
          }
        }
        gb += n;
        ti += 1;
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        tc_commit(bars.at(Bars::kDrain + 2));
        while (!mbar_try_wait(bars.at(Bars::kDrain + 2), 0) && globaltimer_ns() - t0 < 50ull * 1000 * 1000) {}
      }
    }
  } else {
    // =========================================== softmax warpgroups =============================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    const int wg = warp >> 2;                 // 0..3: owns S buffer wg, i.e. the sub-blocks J % 4 == wg
    const int row = (warp & 3) * 32 + lane;   // tile row == tensor-memory lane
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const uint32_t s_addr = lane_addr + kTmS64 + 64 * wg;

    FA4_FOR_EACH_TILE {
      const Tile t = decode_tile<kWindow || kCache>(p, tile);
      const int n = t.n_blocks;
      float m_ref = kNegInf, l_sum = 0.f;

      for (int j = (wg - 2 * (int)gb) & 3; j < 2 * n; j += 4) {
        const uint32_t J = 2 * gb + j, slot = J % kPSlots;  // J % 4 == wg
        const int nb = kWindow ? window_visit_block(j >> 1, n, t.nb_top - n + 1, window_rotates(p, t)) : (j >> 1);
        const int h64 = j & 1;
        const uint32_t bar_s = bars.at(Bars::kSFull + (wg & 2)), par_s = (J / kSBufs) & 1;
        const uint32_t bar_p = bars.at(Bars::kPvDone + slot), par_p = ((J - kPSlots) / kPSlots) & 1;
        const bool r_p = (J >= kPSlots) ? mbar_test(bar_p, par_p) : true;

        // 1. the scores of this sub-block: the whole 64-key row of this thread
        ok = wait_probed(mbar_test(bar_s, par_s), bar_s, par_s, wc, kS64SFull);
        if (!ok) break;
        tc_fence_after_sync();
        if (block_needs_mask<kWindow || kCache, kWindow>(p, t, nb)) {
          if constexpr (kWindow) {
            ws::mask_scores_in_tmem_range(s_addr, lower_limit(p, t, row, nb) - 64 * h64,
                                          causal_limit<true>(p, t, row, nb) - 64 * h64);
          } else {
            mask_scores_in_tmem(s_addr, causal_limit<kWindow || kCache, kWindow>(p, t, row, nb) - 64 * h64);
          }
        }
        float s[64];
        tmem_ld32(s_addr, reinterpret_cast<uint32_t*>(&s[0]));
        tmem_ld32(s_addr + 32, reinterpret_cast<uint32_t*>(&s[32]));
        // While the scores travel (measured: 2.5 % of the kernel's time): the running reference,
        // handed from the warpgroup of sub-block J - 1 to this one through shared memory (one float
        // per row).  Every sub-block but the CTA's very first waits for its predecessor's hand-over,
        // also the first one of a tile (which ignores the value): the unbroken chain is what orders
        // the reuse of a slot -- the value of sub-block J is overwritten by J + 4, which follows
        // J + 3, J + 2 and J + 1, and J + 1 has read it -- and keeps a barrier from running two
        // phases ahead of its waiter.
        float m_prev = kNegInf;
        if (J > 0) {
          const uint32_t pw = (uint32_t)(wg + 3) & 3u;
          ok = __all_sync(0xffffffffu, mbar_wait(bars.at(Bars::kHand + 4 * pw + (warp & 3)), ((J - 1) / kSBufs) & 1, wc, kS64Hand));
          if (!ok) break;
          if (j > 0) m_prev = s_hand[pw * 128 + row];
        }
        tc_wait_ld();
        tc_fence_before_sync();
        mbar_arrive(bars.at(Bars::kSFree + wg));
        if constexpr (kGeneral) {
          if (p.softcap_c1 != 0.f) {
#pragma unroll
            for (int x = 0; x < 64; ++x) s[x] = soft_cap(s[x], p.softcap_c1);
          }
        }

        // 2. maxima of the four 16-key blocks, then the new reference
        float bm4[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float m0 = fmax3(s[16 * q], s[16 * q + 1], s[16 * q + 2]);
          float m1 = fmax3(s[16 * q + 3], s[16 * q + 4], s[16 * q + 5]);
          m0 = fmax3(m0, s[16 * q + 6], s[16 * q + 7]);
          m1 = fmax3(m1, s[16 * q + 8], s[16 * q + 9]);
          m0 = fmax3(m0, s[16 * q + 10], s[16 * q + 11]);
          m1 = fmax3(m1, s[16 * q + 12], s[16 * q + 13]);
          m0 = fmax3(m0, s[16 * q + 14], s[16 * q + 15]);
          bm4[q] = fmaxf(m0, m1);
        }
        const float m_loc = fmaxf(fmaxf(bm4[0], bm4[1]), fmaxf(bm4[2], bm4[3]));
        const float m_new = next_reference(m_prev, m_loc, p.sl2);
        s_hand[wg * 128 + row] = m_new;
        mbar_arrive(bars.at(Bars::kHand + 4 * wg + (warp & 3)));
        float noff4[4];
        uint32_t sbits4[4], sf_bytes;
#if FA4_P_SCALE_E4M3
        block_scales4_e4m3(bm4, m_new, p.sl2, noff4, sf_bytes, sbits4);
#else
        {
          uint32_t ue;
          block_exponents4(bm4, m_new, p.sl2, noff4, ue);
          sf_bytes = block_scale_bytes(ue);
#pragma unroll
          for (int b4 = 0; b4 < 4; ++b4) sbits4[b4] = __byte_perm(ue, 0u, 0x4440u + b4) << 23;  // 2^e as fp32
        }
#endif
        // own partial row sum follows the reference
        if (m_new != m_ref) l_sum *= reference_factor(m_ref, m_new, p.sl2);
        m_ref = m_new;

        // 3. exponentials and quantisation; P slot J % 8 is free once P V of sub-block J - 8 has run
        ok = wait_probed(r_p, bar_p, par_p, wc, kS64PvDone);
        if (!ok) break;
        uint8_t* p_tile = gbase + kOffP + slot * kPTileBytes;
        {
          uint32_t pk[8];
          float acc = 0.f;
#pragma unroll
          for (int b4 = 0; b4 < 4; ++b4) {
            const float bsum = quantize_block16(&s[16 * b4], noff4[b4], p.sl2, pk[2 * b4], pk[2 * b4 + 1]);
            acc = fmaf(bsum, __uint_as_float(sbits4[b4]), acc);   // times the block scale
          }
          l_sum += acc;
          *reinterpret_cast<uint4*>(p_tile + sw32_offset(row, 0)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          *reinterpret_cast<uint4*>(p_tile + sw32_offset(row, 1)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
        // the four scale bytes of this row: one word of the 512-byte chunk
        *reinterpret_cast<uint32_t*>(gbase + kOffSFP + slot * 512 + (row & 31) * 16 + (row >> 5) * 4) = sf_bytes;

        // 4. correction (rare, out of line): O holds the sub-blocks before this one relative to
        //    m_prev and must move to m_new before P V of this sub-block is issued; this thread
        //    owns its whole row of O
        //    (rows whose reference was -inf so far have an all-zero O: nothing to rescale)
        const bool fix = (m_new != m_prev) && (m_prev != kNegInf);
        if (j > 0 && __any_sync(0xffffffffu, fix)) {
          const uint32_t Jp = J - 1;
          ok = __all_sync(0xffffffffu, mbar_wait(bars.at(Bars::kPvDone + (Jp % kPSlots)),
                                                 (Jp / kPSlots) & 1, wc, kS64PvDone));
          if (!ok) break;
          tc_fence_after_sync();
          const float f = fix ? reference_factor(m_prev, m_new, p.sl2) : 1.f;
          rescale_accumulator(lane_addr + kTmO, f, kDv / 32);
          tc_wait_st();
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        mbar_arrive(bars.at(Bars::kPFull + slot));
      }
      if (!ok) break;

      // ---- tile end: hand the partial row sum and its reference to the epilogue warpgroup and
      //      go on with the next tile
      if (n > 0) {
        const uint32_t fb = ti & 1;
        if (ti >= 2) {
          ok = __all_sync(0xffffffffu,
                          mbar_wait(bars.at(Bars::kFinFree + fb), ((ti - 2) >> 1) & 1, wc, kS64FinFree));
          if (!ok) break;
        }
        volatile float* fin_slot = s_fin + fb * (4 * 128 * 2);
        // slot order = position of the warpgroup's first sub-block inside the tile: the summation
        // order of a row then depends on its tile only, not on what the CTA processed before
        const uint32_t fslot = (uint32_t)(wg - 2 * (int)gb) & 3u;
        fin_slot[(fslot * 128 + row) * 2] = l_sum;
        fin_slot[(fslot * 128 + row) * 2 + 1] = m_ref;
        mbar_arrive(bars.at(Bars::kFin + fb));
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
