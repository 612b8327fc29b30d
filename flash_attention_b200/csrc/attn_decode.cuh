// Decode / append kernel: a handful of query rows against a long key range (head dim 128).
//
// The prefill kernels put QUERY rows on the 128 lanes of the tensor-core tile; with one query
// token per sequence 127 of them are padding and the per-block latency chain (about 3000 clocks,
// two blocks in flight) sets the pace: 0.7 TB/s of K/V.  Here the products are transposed, as
// decode kernels usually do: the 128 KEYS of a block sit on the lanes and the query rows -- the
// Sq x (query heads per kv head) rows that share this kv head, at most 32 -- on the N side
// (N = 16, or 32 for more than 16 rows):
//
//   S^T (128 keys x N rows)  = K (A operand, the tile as it is loaded) . Q^T (B operand)
//   O^T (128 dv   x N rows) += V^T (A operand: V is stored key-contiguous, i.e. already as the
//                                   K-major (dv, keys) matrix) . P^T (B operand)
//
// so no lane is wasted, an S^T buffer is N tensor-memory columns, and tensor memory hands a
// softmax thread ONE key with its <= N scores.  The warp transposes that within groups of `rows`
// lanes, after which a thread owns one query ROW with `rows` neighbouring keys: the per-row work
// (mask limit, reference maximum, block exponent, running sum) is scalar per thread; block and
// warp maxima take zero to three shuffles, the CTA maximum one exchange through shared memory per
// block.  P is quantised exactly as in the prefill kernels (e2m1, power-of-two ue4m3 scale per
// row and 16 keys, lazy reference).
//
// One CTA = one (split, kv head, batch entry): a contiguous share of the entry's 128-key blocks,
// visited in ascending order; it writes a normalised fp32 partial O and a partial LSE for
// combine_splits_kernel, like the split-KV path of attn_ws.cuh.  Grid = (splits, Hkv, B).
//   warps 0-3  softmax / correction / epilogue (thread = key lane, after the transpose a row; in the
//              correction and the epilogue a dv lane)
//   warp 4     TMA producer of K (ring of three tiles, through the page table if there is one)
//   warp 5     MMA issuer (owns tensor memory)
//   warp 6     TMA producer of V (its own ring, independent of K's)
// Every wait is bounded, like everywhere else.
#pragma once
#include "attn_common.cuh"
#include "softmax.cuh"

namespace fa4 {
namespace dec {

constexpr int kThreads = 224;
// Three of everything: 70 KB of shared memory and 128 tensor-memory columns per CTA (256 in the
// 32-row form), so that THREE CTAs share an SM (two in the 32-row form).
constexpr int kStages = 3;   // K and V tiles in flight
constexpr int kSBufs = 3;    // S^T buffers (N columns each)
constexpr int kPSlots = 3;   // P^T tiles (N rows x 64 bytes) and their scale chunks
constexpr int kMaxRows = 32; // query rows per kv head: Sq * group

// shared memory
constexpr uint32_t kOffK = 0;
constexpr uint32_t kOffV = kOffK + kStages * kTileBytes;
constexpr uint32_t kOffSFK = kOffV + kStages * kTileBytes;
constexpr uint32_t kOffSFV = kOffSFK + kStages * kSfBytes;
constexpr uint32_t kQBytes = kMaxRows * 64;                // Q^T / P^T operand: up to 32 rows x 64 bytes
constexpr uint32_t kOffQ = kOffSFV + kStages * kSfBytes;   // rows x 64 bytes, 64-byte swizzle
constexpr uint32_t kOffSFQ = kOffQ + kQBytes;              // two 512-byte chunks
constexpr uint32_t kOffP = kOffSFQ + 1024;                 // kPSlots x kQBytes
constexpr uint32_t kOffSFP = kOffP + kPSlots * kQBytes;    // kPSlots x 2 chunks x 512
constexpr uint32_t kOffRed = kOffSFP + kPSlots * 1024;     // 2 x 4 warps x 32 floats
constexpr uint32_t kOffBar = kOffRed + 2 * 4 * kMaxRows * 4;
struct Bars {
  uint32_t base;
  static constexpr uint32_t kKFull = 0, kVFull = kKFull + kStages, kKFree = kVFull + kStages,
                            kVFree = kKFree + kStages, kSFull = kVFree + kStages,
                            kSFree = kSFull + kSBufs, kPFull = kSFree + kSBufs,
                            kPvDone = kPFull + kPSlots, kQReady = kPvDone + kPSlots,
                            kSync = kQReady + 1, kDrain = kSync + 1, kCount = kDrain + 1;
  __device__ explicit Bars(uint32_t b) : base(b) {}
  __device__ __forceinline__ uint32_t at(uint32_t idx) const { return base + 8u * idx; }
};
constexpr uint32_t kOffMisc = kOffBar + 8 * Bars::kCount;
constexpr uint32_t kSmemRequest = kOffMisc + 16 + 1024;
// The 32-row form allocates 256 tensor-memory columns: its request is padded so that only two CTAs
// fit an SM (a third would sit inside tcgen05.alloc until one of them ends).
constexpr uint32_t kSmemRequestWide = 100 * 1024;
static_assert(kSmemRequest <= kSmemRequestWide && 3 * kSmemRequest <= 227 * 1024, "decode kernel shared memory");

// tensor memory of the form with N columns per operand (N = 16: 128 columns allocated, N = 32:
// 256): S^T buffers, O^T, scale factors.  The K / V / P scale slots alternate between two copies:
// the copy and the product that reads it are issued by one thread to the in-order tensor pipe, the
// second copy keeps a copy from racing the product before.
template <int kN>
struct Tm {
  static constexpr uint32_t kCols = kN == 16 ? 128 : 256;
  static constexpr uint32_t kS = 0 /* 3 x N */, kO = 3 * kN, kSFQ = 4 * kN, kSFK = kSFQ + 8 /* 2 x 8 */,
                            kSFV = kSFK + 16 /* 2 x 8 */, kSFP = kSFV + 16 /* 2 x 8 */;
  static_assert(kSFP + 16 <= kCols, "tensor-memory map of the decode kernel");
};

enum Site { kDKFull = 80, kDVFull, kDKFree, kDVFree, kDSFull, kDSFree, kDPFull, kDPvDone, kDQReady, kDSync };

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
      "r"(r[15]), "r"(taddr)
      : "memory");
}

// One e2m1 byte from two values: `lo` goes to the low nibble (the even key).
__device__ __forceinline__ uint32_t pack2_e2m1(float lo, float hi) {
  uint16_t b;
  asm("{\n"
      ".reg .b8 t;\n"
      "cvt.rn.satfinite.e2m1x2.f32 t, %2, %1;\n"
      "cvt.u16.u8 %0, t;\n"
      "}\n"
      : "=h"(b)
      : "f"(lo), "f"(hi));
  return b;
}

// kN columns (4, 8 or 16) of this thread's tensor-memory lane.
template <int kN>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t* r) {
  if constexpr (kN == 4) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr)
                 : "memory");
  } else if constexpr (kN == 8) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
  } else if constexpr (kN == 16) {
    tmem_ld16(taddr, r);
  } else {
    tmem_ld32(taddr, r);
  }
}
template <int kN>
__device__ __forceinline__ void tmem_st_cols(uint32_t taddr, const uint32_t* r) {
  if constexpr (kN == 4) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%4], {%0, %1, %2, %3};"
                 ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(taddr)
                 : "memory");
  } else if constexpr (kN == 8) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%8], {%0, %1, %2, %3, %4, %5, %6, %7};"
                 ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                 "r"(taddr)
                 : "memory");
  } else if constexpr (kN == 16) {
    tmem_st16(taddr, r);
  } else {
    tmem_st32(taddr, r);
  }
}

// T x T transpose inside every group of T neighbouring lanes (T = 4, 8, 16, 32): before, lane i of a
// group holds x[0..T) = its own column; after, x[j] is what lane j of the group held in x[i].
// log2(T) butterfly rounds of T / 2 shuffles.
template <int T>
__device__ __forceinline__ void lane_group_transpose(float (&x)[T], int lane) {
#pragma unroll
  for (int bit = 1; bit < T; bit <<= 1) {
    const bool up = (lane & bit) != 0;
#pragma unroll
    for (int j = 0; j < T; ++j) {
      if ((j & bit) == 0) {
        const float send = up ? x[j] : x[j | bit];
        const float recv = __shfl_xor_sync(0xffffffffu, send, bit);
        if (up) x[j] = recv; else x[j | bit] = recv;
      }
    }
  }
}

// Exponent of one 16-key block of P from its maximum (the scalar form of block_exponents4):
// noff with p'/2^e = 2^(s * sl2 + noff), and the byte e + 127.
__device__ __forceinline__ void block_exponent1(float bm, float m_ref, float sl2, float& noff,
                                                uint32_t& ue) {
  constexpr float kMagic = 12582912.f + 127.f;
  const float msc = (m_ref == kNegInf) ? 0.f : m_ref * sl2;
  const float c_t = static_cast<float>(kShift) - kLog2Of6 + 0.4999995f - msc;
  const float c_off = static_cast<float>(kShift) - msc;
  float t = fmaf(bm, sl2, c_t);
  t = fmaxf(t, static_cast<float>(kEMin) - 0.4f);
  const float u = t + kMagic;
  ue = __float_as_uint(u) & 0xffu;
  noff = c_off - (u - kMagic);
}

}  // namespace dec

struct DecodeParams {
  const uint8_t* q;      // (B, Sq, Hq, 64) packed e2m1
  const uint8_t* q_sf;   // tiled (B, Hq, ceil(Sq/128), 2, 512)
  int64_t q_stride_b, q_stride_s, q_stride_h;
  int num_splits;
  float* o_partial;      // (splits, B, Sq, Hq, 128) fp32
  float* lse_partial;    // (splits, B, Hq, Sq) fp32
};

// kR: query rows the softmax code is built for (4, 8, 16 or 32 >= Sq * group): the size of the
// lane-group transpose and the number of keys a thread owns afterwards.  N (the MMA's N, the
// columns of an S^T buffer) is 16 up to sixteen rows and 32 above.
template <int kR>
__global__ void __launch_bounds__(dec::kThreads, kR <= 16 ? 3 : 2)
attn_decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const KernelParams p, const DecodeParams d) {
  using namespace dec;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  const Bars bars(base + kOffBar);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + kOffMisc);
  volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(gbase + kOffMisc + 4);
  volatile float* s_red = reinterpret_cast<volatile float*>(gbase + kOffRed);  // [2][4][32]
  constexpr int kN = kR <= 16 ? 16 : 32;
  using TM = Tm<kN>;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const WaitCtx wc{s_abort, p.status, p.budget_ns, p.epoch};
  const int R = p.Sq * p.group;  // live query rows (<= kR)

  // The query rows and their scale words go to registers first thing: their latency (a trip to
  // HBM while every CTA of the grid starts its K / V stream) then overlaps the set-up below
  // instead of following it.  Threads 0-127: row tid / 4, 16-byte chunk tid % 4; threads 0-63
  // also: row tid / 2, the scale word of 64-element step tid % 2.
  uint4 q_pref = make_uint4(0u, 0u, 0u, 0u);
  uint32_t qsf_pref = 0u;
  if (tid < 128) {
    const int r = tid >> 2, ch = tid & 3;
    if (r < R) {
      const int s = r / p.group, h = hk * p.group + r % p.group;
      q_pref = *reinterpret_cast<const uint4*>(d.q + b * d.q_stride_b + s * d.q_stride_s + h * d.q_stride_h +
                                               ch * 16);
    }
  }
  if (tid < 64) {
    const int r = tid >> 1, ks = tid & 1;
    if (r < R) {
      const int s = r / p.group, h = hk * p.group + r % p.group;
      const uint8_t* chunk = d.q_sf + b * p.qsf_stride_b + h * p.qsf_stride_h + ((int64_t)(s / 128) * 2 + ks) * 512;
      const int rr = s % 128;
      qsf_pref = *reinterpret_cast<const uint32_t*>(chunk + (rr % 32) * 16 + (rr / 32) * 4);
    }
  }

  // this CTA's share of the entry's K/V blocks (ascending, contiguous, ceil division like the
  // split-KV path of the prefill kernel)
  int sk = p.Sk;
  if (p.seqused_k != nullptr) {
    const int used = p.seqused_k[b];
    sk = used < 0 ? 0 : (used < p.Sk ? used : p.Sk);
  }
  const int n_total = (sk + kBlockN - 1) / kBlockN;
  const int per = (n_total + d.num_splits - 1) / d.num_splits;
  const int i0 = split * per < n_total ? split * per : n_total;
  const int i1 = i0 + per < n_total ? i0 + per : n_total;
  const int n = i1 - i0;

  if (tid == 0) {
    *s_abort = 0u;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bars.at(Bars::kKFull + s), 1);
      mbar_init(bars.at(Bars::kVFull + s), 1);
      mbar_init(bars.at(Bars::kKFree + s), 1);
      mbar_init(bars.at(Bars::kVFree + s), 1);
      mbar_init(bars.at(Bars::kSFull + s), 1);
      mbar_init(bars.at(Bars::kSFree + s), 128);
      mbar_init(bars.at(Bars::kPFull + s), 128);
      mbar_init(bars.at(Bars::kPvDone + s), 1);
    }
    mbar_init(bars.at(Bars::kQReady), 128);
    mbar_init(bars.at(Bars::kSync), 128);
    mbar_init(bars.at(Bars::kDrain), 1);
    fence_barrier_init();
  }
  if (warp == 4 && lane == 0) tma_prefetch_desc(&tm_k);
  if (warp == 6 && lane == 0) tma_prefetch_desc(&tm_v);
  if (warp == 5) {
    tmem_alloc(base + kOffMisc, TM::kCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  // the combine kernel is launched as a programmatic dependent: let its CTAs be scheduled while
  // this grid still runs (they wait for its completion before they read the partials)
  asm volatile("griddepcontrol.launch_dependents;");
  const uint32_t tmem = *tmem_slot;
  constexpr uint32_t idesc = make_idesc_nvf4(128, kN);
  bool ok = true;

  if (warp == 4 || warp == 6) {
    // ============================================ TMA producers =================================
    // Warp 4 streams K, warp 6 streams V, each as far ahead as its own ring allows.  (One thread
    // issuing K and V in turn tied the K stream to the P V products: K of block i + 1 went out
    // only when P V of block i - 3 had freed a V stage, one block time before Q K^T needs it, and
    // the kernel ran at one block per memory latency.)
    if (lane == 0) {
      const bool is_k = warp == 4;
      const uint32_t full0 = is_k ? Bars::kKFull : Bars::kVFull, free0 = is_k ? Bars::kKFree : Bars::kVFree;
      const uint32_t tile0 = base + (is_k ? kOffK : kOffV), sf0 = base + (is_k ? kOffSFK : kOffSFV);
      const uint8_t* sf_src = is_k ? p.k_sf + hk * p.ksf_stride_h : p.v_sf + hk * p.vsf_stride_h;
      const int64_t sf_stride_b = is_k ? p.ksf_stride_b : p.vsf_stride_b;
      uint32_t issued = 0;
      for (int li = 0; ok && li < n; ++li) {
        const int nb = i0 + li;
        const uint32_t st = li % kStages;
        int kb = b, nbl = nb;   // batch coordinate and block inside it (a page of the pool)
        if (p.page_table != nullptr) {
          const int key0 = nb * kBlockN, pg = key0 / p.page_size;
          kb = p.page_table[(int64_t)b * p.pages_per_seq + pg];
          nbl = (key0 - pg * p.page_size) / kBlockN;
        }
        if (li >= kStages) {
          ok = mbar_wait(bars.at(free0 + st), ((li - kStages) / kStages) & 1, wc, is_k ? kDKFree : kDVFree);
          if (!ok) break;
        }
        mbar_arrive_expect_tx(bars.at(full0 + st), kTileBytes + kSfBytes);
        if (is_k) {
          tma_load_4d(tile0 + st * kTileBytes, &tm_k, bars.at(full0 + st), 0, hk, nbl * kBlockN, kb);
        } else {
          tma_load_4d(tile0 + st * kTileBytes, &tm_v, bars.at(full0 + st), nbl * (kBlockN / 2), 0, hk, kb);
        }
        bulk_load(sf0 + st * kSfBytes, sf_src + kb * sf_stride_b + (int64_t)nbl * kSfBytes, kSfBytes,
                  bars.at(full0 + st));
        issued = li + 1;
      }
      if (!ok) {
        // bounded drain: let the copies already issued land before the CTA's memory is released
        const uint64_t t0 = globaltimer_ns();
        for (uint32_t i = issued > kStages ? issued - kStages : 0; i < issued; ++i) {
          while (!mbar_try_wait(bars.at(full0 + (i % kStages)), (i / kStages) & 1) &&
                 globaltimer_ns() - t0 < 50ull * 1000 * 1000) {}
        }
      }
    }
  } else if (warp == 5) {
    // ============================================ MMA issuer ====================================
    if (lane == 0 && n > 0) {
      ok = mbar_wait(bars.at(Bars::kQReady), 0, wc, kDQReady);
      uint64_t dq[2];
      if (ok) {
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
          tc_cp_sf(tmem + TM::kSFQ + 4 * ks, base + kOffSFQ + 512 * ks);
          dq[ks] = make_desc_sw64(base + kOffQ + 32 * ks);
        }
      }
      for (int step = 0; ok && step < n + 2; ++step) {
        if (step < n) {
          // S^T = K . Q^T of block step
          const uint32_t li = step, st = li % kStages, buf = li % kSBufs;
          ok = mbar_wait(bars.at(Bars::kKFull + st), (li / kStages) & 1, wc, kDKFull);
          if (!ok) break;
          if (li >= kSBufs) {
            ok = mbar_wait(bars.at(Bars::kSFree + buf), ((li - kSBufs) / kSBufs) & 1, wc, kDSFree);
            if (!ok) break;
          }
          tc_fence_after_sync();
          const uint32_t sfk = tmem + TM::kSFK + 8 * (li & 1);
          const uint32_t kt = base + kOffK + st * kTileBytes, ksf = base + kOffSFK + st * kSfBytes;
#pragma unroll
          for (int ks = 0; ks < 2; ++ks) tc_cp_sf(sfk + 4 * ks, ksf + 512 * ks);
#pragma unroll
          for (int ks = 0; ks < 2; ++ks) {
            mma_nvf4(tmem + TM::kS + kN * buf, make_desc_sw64(kt + 32 * ks), dq[ks], idesc, sfk + 4 * ks,
                     tmem + TM::kSFQ + 4 * ks, ks > 0 ? 1u : 0u);
          }
          tc_commit(bars.at(Bars::kSFull + buf));
          tc_commit(bars.at(Bars::kKFree + st));
        }
        if (step >= 2) {
          // O^T += V^T . P^T of block step - 2
          const uint32_t li = step - 2, st = li % kStages, slot = li % kPSlots;
          ok = mbar_wait(bars.at(Bars::kVFull + st), (li / kStages) & 1, wc, kDVFull);
          if (!ok) break;
          ok = mbar_wait(bars.at(Bars::kPFull + slot), (li / kPSlots) & 1, wc, kDPFull);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t sfv = tmem + TM::kSFV + 8 * (li & 1), sfp = tmem + TM::kSFP + 8 * (li & 1);
          const uint32_t vt = base + kOffV + st * kTileBytes, vsf = base + kOffSFV + st * kSfBytes;
          const uint32_t pt = base + kOffP + slot * kQBytes, psf = base + kOffSFP + slot * 1024;
#pragma unroll
          for (int ks = 0; ks < 2; ++ks) {
            tc_cp_sf(sfv + 4 * ks, vsf + 512 * ks);
            tc_cp_sf(sfp + 4 * ks, psf + 512 * ks);
          }
#pragma unroll
          for (int ks = 0; ks < 2; ++ks) {
            mma_nvf4(tmem + TM::kO, make_desc_sw64(vt + 32 * ks), make_desc_sw64(pt + 32 * ks), idesc,
                     sfv + 4 * ks, sfp + 4 * ks, (li > 0 || ks > 0) ? 1u : 0u);
          }
          tc_commit(bars.at(Bars::kPvDone + slot));
          tc_commit(bars.at(Bars::kVFree + st));
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        tc_commit(bars.at(Bars::kDrain));
        while (!mbar_try_wait(bars.at(Bars::kDrain), 0) && globaltimer_ns() - t0 < 50ull * 1000 * 1000) {}
      }
    }
  } else {
    // ============================================ softmax / epilogue warpgroup ==================
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    uint32_t sync_phase = 0;
    // rendezvous of the 128 threads on an mbarrier (bounded, unlike bar.sync)
#define FA4_DEC_SYNC()                                                                          \
  mbar_arrive(bars.at(Bars::kSync));                                                            \
  ok = __all_sync(0xffffffffu, mbar_wait(bars.at(Bars::kSync), sync_phase & 1, wc, kDSync));     \
  sync_phase += 1;

    // ---- set-up: Q^T operand (rows x 64 bytes, rows past R zero), its scale chunks, zeroed
    //      P^T tiles and scale chunks (rows past R are never written again)
    for (uint32_t i = tid; i < (kOffRed - kOffQ) / 16; i += 128) {
      *reinterpret_cast<uint4*>(gbase + kOffQ + i * 16) = make_uint4(0u, 0u, 0u, 0u);  // Q, SFQ, P, SFP are contiguous
    }
    ok = true;
    FA4_DEC_SYNC()
    if (ok) {
      const int r = tid >> 2, ch = tid & 3;
      if (r < R) *reinterpret_cast<uint4*>(gbase + kOffQ + sw64_offset(r, ch)) = q_pref;
    }
    if (ok && tid < 64) {
      // scale bytes of row r: two words (one per 64-element step) of the tiled layout
      const int r = tid >> 1, ks = tid & 1;
      if (r < R) *reinterpret_cast<uint32_t*>(gbase + kOffSFQ + 512 * ks + r * 16) = qsf_pref;
    }
    fence_proxy_async_smem();
    mbar_arrive(bars.at(Bars::kQReady));

    // After the transpose below a thread owns ONE query row (row = lane % kR) with kR neighbouring
    // keys of its warp's 32 (group = lane / kR), so everything per row -- mask limit, reference
    // maximum, block exponent, running sum -- is scalar per thread and runs once per block, where a
    // thread that kept "its key, all rows" ran it kR times.
    const int my_row = lane & (kR - 1), grp = lane / kR;
    const int key_in_blk = warp * 32 + grp * kR;   // first of this thread's kR keys inside the block
    float m_ref = kNegInf, l_sum = 0.f;
    // last visible key of the row (causal: bottom-right aligned on the entry's key count); rows
    // past R see nothing
    int lim = -1;
    if (my_row < R) {
      const int c = sk - p.Sq + my_row / p.group;
      lim = (p.causal && c < sk - 1) ? c : sk - 1;
    }

    for (int li = 0; ok && li < n; ++li) {
      const int nb = i0 + li;
      const uint32_t buf = li % kSBufs, slot = li % kPSlots;
      ok = __all_sync(0xffffffffu, mbar_wait(bars.at(Bars::kSFull + buf), (li / kSBufs) & 1, wc, kDSFull));
      if (!ok) break;
      tc_fence_after_sync();
      float x[kR];
      tmem_ld_cols<kR>(lane_addr + TM::kS + kN * buf, reinterpret_cast<uint32_t*>(x));
      tc_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(bars.at(Bars::kSFree + buf));

      // (key = lane, all rows) -> (row = lane % kR, kR keys): x[j] = score of key key_in_blk + j
      lane_group_transpose<kR>(x, lane);
      const int key0 = nb * kBlockN + key_in_blk;
      // kB 16-key blocks per thread: one (shared with neighbouring lanes) up to 16 rows, two of
      // its own in the 32-row form, where a thread owns all 32 keys of its warp
      constexpr int kB = kR <= 16 ? 1 : 2, kPer = kR / kB;
      float bm[kB];
#pragma unroll
      for (int q = 0; q < kB; ++q) {
        bm[q] = kNegInf;
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
          x[q * kPer + j] = (key0 + q * kPer + j <= lim) ? x[q * kPer + j] : kNegInf;
          bm[q] = fmaxf(bm[q], x[q * kPer + j]);
        }
      }
      // maximum of the row's 16-key block (kept for the P scale), then of the warp's 32 keys
      float wm;
      if constexpr (kB == 1) {
#pragma unroll
        for (int o = kR; o < 16; o <<= 1) bm[0] = fmaxf(bm[0], __shfl_xor_sync(0xffffffffu, bm[0], o));
        wm = fmaxf(bm[0], __shfl_xor_sync(0xffffffffu, bm[0], 16));
      } else {
        wm = fmaxf(bm[0], bm[kB - 1]);
      }
      volatile float* red = s_red + (li & 1) * (4 * kMaxRows);
      if (lane < kR) red[warp * kMaxRows + lane] = wm;
      FA4_DEC_SYNC()
      if (!ok) break;

      // reference maximum of the row (CTA-uniform per row: every warp computes the same value)
      const float m_loc = fmaxf(fmaxf(red[my_row], red[kMaxRows + my_row]),
                                fmaxf(red[2 * kMaxRows + my_row], red[3 * kMaxRows + my_row]));
      const float m_new = next_reference(m_ref, m_loc, p.sl2);
      float fac = 1.f;
      bool moved_row = false;
      if (m_new != m_ref) {
        fac = reference_factor(m_ref, m_new, p.sl2);
        moved_row = m_ref != kNegInf;
        l_sum *= fac;
        m_ref = m_new;
      }
      const bool moved = __any_sync(0xffffffffu, moved_row);   // every warp holds all rows

      // P slot free once P V of block li - kPSlots has run
      if (li >= kPSlots) {
        ok = __all_sync(0xffffffffu, mbar_wait(bars.at(Bars::kPvDone + slot), ((li - kPSlots) / kPSlots) & 1, wc,
                                               kDPvDone));
        if (!ok) break;
      }
      {
        float noff[kB];
        uint32_t ue[kB];
        float pv[kR];
#pragma unroll
        for (int q = 0; q < kB; ++q) {
          block_exponent1(bm[q], m_ref, p.sl2, noff[q], ue[q]);
          float psum = 0.f;
#pragma unroll
          for (int j = 0; j < kPer; ++j) {
            pv[q * kPer + j] = ex2_approx(fmaf(x[q * kPer + j], p.sl2, noff[q]));
            psum += pv[q * kPer + j];
          }
          l_sum = fmaf(psum, __uint_as_float(ue[q] << 23), l_sum);
        }
        if (my_row < R) {   // rows past R stay zero (written once at set-up)
          // kR keys = kR / 2 bytes of the row's 64, inside one 16-byte chunk of the swizzled tile
          const uint32_t col = static_cast<uint32_t>(key_in_blk) >> 1;
          uint8_t* dst = gbase + kOffP + slot * kQBytes + sw64_offset(my_row, col >> 4) + (col & 15);
          // scale byte of 16-key block blk = key_in_blk / 16: chunk blk / 4, the row's word, byte blk % 4
          uint8_t* sf_dst = gbase + kOffSFP + slot * 1024 + 512 * (key_in_blk >> 6) + my_row * 16 +
                            ((key_in_blk >> 4) & 3);
          if constexpr (kR == 4) {
            *reinterpret_cast<uint16_t*>(dst) =
                static_cast<uint16_t>(pack2_e2m1(pv[0], pv[1]) | (pack2_e2m1(pv[2], pv[3]) << 8));
          } else if constexpr (kR == 8) {
            *reinterpret_cast<uint32_t*>(dst) = pack8_e2m1(pv[0], pv[1], pv[2], pv[3], pv[4], pv[5], pv[6], pv[7]);
          } else if constexpr (kR == 16) {
            *reinterpret_cast<uint2*>(dst) =
                make_uint2(pack8_e2m1(pv[0], pv[1], pv[2], pv[3], pv[4], pv[5], pv[6], pv[7]),
                           pack8_e2m1(pv[8 % kR], pv[9 % kR], pv[10 % kR], pv[11 % kR], pv[12 % kR], pv[13 % kR],
                                      pv[14 % kR], pv[15 % kR]));
          } else {
            uint32_t w[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              w[c] = pack8_e2m1(pv[(8 * c) % kR], pv[(8 * c + 1) % kR], pv[(8 * c + 2) % kR], pv[(8 * c + 3) % kR],
                                pv[(8 * c + 4) % kR], pv[(8 * c + 5) % kR], pv[(8 * c + 6) % kR], pv[(8 * c + 7) % kR]);
            }
            *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
          }
          if constexpr (kB == 2) {
            // the thread's two blocks are neighbours in the scale word of its row
            *reinterpret_cast<uint16_t*>(sf_dst) =
                static_cast<uint16_t>(((ue[0] - 0x78u) << 3) | (((ue[kB - 1] - 0x78u) << 3) << 8));
          } else if ((key_in_blk & 15) == 0) {
            *sf_dst = static_cast<uint8_t>((ue[0] - 0x78u) << 3);
          }
        }
      }

      // correction (rare): O^T holds the earlier blocks relative to the old references; here a
      // thread is a dv lane with all rows in its columns, the factor of row r sits in lane r
      if (li > 0 && moved) {
        ok = __all_sync(0xffffffffu, mbar_wait(bars.at(Bars::kPvDone + ((li - 1) % kPSlots)),
                                               ((li - 1) / kPSlots) & 1, wc, kDPvDone));
        if (!ok) break;
        tc_fence_after_sync();
        float o[kR];
        tmem_ld_cols<kR>(lane_addr + TM::kO, reinterpret_cast<uint32_t*>(o));
        tc_wait_ld();
#pragma unroll
        for (int r = 0; r < kR; ++r) o[r] *= __shfl_sync(0xffffffffu, fac, r);
        tmem_st_cols<kR>(lane_addr + TM::kO, reinterpret_cast<const uint32_t*>(o));
        tc_wait_st();
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(bars.at(Bars::kPFull + slot));
    }

    // ---- epilogue: row sums over the 128 key lanes, then thread = dv lane of O^T --------------
    if (ok) {
      volatile float* red = s_red + (n & 1) * (4 * kMaxRows);
      float v = l_sum;   // this thread's share of its row; the lanes of one row are kR apart
#pragma unroll
      for (int o = kR; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane < kR) red[warp * kMaxRows + lane] = v;
      FA4_DEC_SYNC()
    }
    if (ok) {
      volatile float* red = s_red + (n & 1) * (4 * kMaxRows);
      float o[kR];
#pragma unroll
      for (int r = 0; r < kR; ++r) o[r] = 0.f;
      if (n > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(bars.at(Bars::kPvDone + ((n - 1) % kPSlots)),
                                               ((n - 1) / kPSlots) & 1, wc, kDPvDone));
        if (ok) {
          tc_fence_after_sync();
          tmem_ld_cols<kR>(lane_addr + TM::kO, reinterpret_cast<uint32_t*>(o));
          tc_wait_ld();
        }
      }
      if (ok) {
#pragma unroll
        for (int r = 0; r < kR; ++r) {
          if (r < R) {
            // fixed order over the four warps: the sum of a row does not depend on timing
            const float l_tot = ((red[r] + red[kMaxRows + r]) + red[2 * kMaxRows + r]) + red[3 * kMaxRows + r];
            const int s = r / p.group, h = hk * p.group + r % p.group;
            const float scale = (l_tot > 0.f && n > 0) ? p.out_scale / l_tot : 0.f;
            d.o_partial[((((int64_t)split * p.B + b) * p.Sq + s) * p.Hq + h) * 128 + tid] = o[r] * scale;
            if (tid == r) {   // thread r (warp 0, lane r) owns row r: its m_ref is the row's
              d.lse_partial[(((int64_t)split * p.B + b) * p.Hq + h) * p.Sq + s] =
                  finish_lse(m_ref, l_tot, p.sl2);
            }
          }
        }
      }
    }
#undef FA4_DEC_SYNC
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem, TM::kCols);
}

}  // namespace fa4
