// Serial variant: one warpgroup (128 threads) per 128-row tile does load -> QK^T -> softmax ->
// P.V one step after the other.  Nothing overlaps; it exists to bring the tensor-core contract
// up and to cross-check the warp-specialised kernel on the GPU at sizes the CPU oracle cannot
// reach.  Same math (softmax.cuh), same operand layouts, same tensor-memory map.
#pragma once
#include "attn_common.cuh"

namespace fa4 {

// tensor-memory column map (512 columns allocated), shared with the warp-specialised kernel
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmS0 = 0, kTmS1 = 128, kTmO = 256;
constexpr uint32_t kTmSFQ = 384;  // 8 columns: 2 MMA K-steps x 4
constexpr uint32_t kTmSFK = 392;  // 2 buffers x 8
constexpr uint32_t kTmSFV = 408;  // 2 buffers x 8
constexpr uint32_t kTmSFP = 424;  // 2 buffers x 8

constexpr uint32_t kTileBytes = 128 * 64;  // one 128-row x 128-element e2m1 tile
constexpr uint32_t kSfBytes = 1024;        // its scale factors: 2 chunks of 512

namespace serial {
constexpr uint32_t kOffQ = 0, kOffK = 8192, kOffV = 16384, kOffP = 24576;
constexpr uint32_t kOffSFQ = 32768, kOffSFK = 33792, kOffSFV = 34816, kOffSFP = 35840;
constexpr uint32_t kOffBar = 36864;  // 3 mbarriers, tmem slot, abort flag
constexpr uint32_t kSmemUsed = kOffBar + 64;
// Requested size is padded so that only one CTA fits per SM: every CTA allocates all 512
// tensor-memory columns, and a second resident CTA would block inside tcgen05.alloc.
constexpr uint32_t kSmemRequest = 120 * 1024;
enum Site { kSiteLoad = 1, kSiteMma = 2, kSiteCta = 3, kSiteDrain = 4 };
}  // namespace serial

__global__ void __launch_bounds__(128, 1)
attn_fwd_serial_kernel(const __grid_constant__ CUtensorMap tm_q,
                       const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const KernelParams p) {
  using namespace serial;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar_load = base + kOffBar, bar_mma = base + kOffBar + 8, bar_cta = base + kOffBar + 16;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + kOffBar + 24);
  volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(gbase + kOffBar + 28);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const WaitCtx wc{s_abort, p.status, p.budget_ns, p.epoch};

  if (tid == 0) {
    *s_abort = 0u;
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    mbar_init(bar_cta, 128);
    fence_barrier_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 0) {
    tmem_alloc(base + kOffBar + 24, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  // a CTA that starts after an earlier one failed does nothing
  const bool poisoned = status_poisoned(p.status, p.epoch);

  const Tile t = decode_tile(p, blockIdx.x);
  const int row = tid;  // tile row == tensor-memory lane
  const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
  constexpr uint32_t idesc = make_idesc_nvf4(128, 128);

  uint32_t ph_load = 0, ph_mma = 0, ph_cta = 0;
  bool load_pending = false, mma_pending = false;
  float m_ref = kNegInf, l_sum = 0.f;
  bool ok = !poisoned;

  if (ok && t.n_blocks > 0) {
    // ---- Q tile and its scales -------------------------------------------------------------
    if (tid == 0) {
      mbar_arrive_expect_tx(bar_load, kTileBytes + kSfBytes);
      tma_load_4d(base + kOffQ, &tm_q, bar_load, 0, t.h, t.m_blk * kBlockM, t.b);
      bulk_load(base + kOffSFQ,
                p.q_sf + t.b * p.qsf_stride_b + t.h * p.qsf_stride_h + (int64_t)t.m_blk * kSfBytes,
                kSfBytes, bar_load);
      load_pending = true;
    }
    ok = mbar_wait(bar_load, ph_load, wc, kSiteLoad);
    ph_load ^= 1;
    if (ok && tid == 0) {
      load_pending = false;
      tc_cp_sf(tmem + kTmSFQ, base + kOffSFQ);
      tc_cp_sf(tmem + kTmSFQ + 4, base + kOffSFQ + 512);
    }

    for (int i = 0; ok && i < t.n_blocks; ++i) {
      const int nb = t.n_blocks - 1 - i;  // last (diagonal) block first, like the reference
      // ---- K, V tiles and scales -----------------------------------------------------------
      if (tid == 0) {
        mbar_arrive_expect_tx(bar_load, 2 * (kTileBytes + kSfBytes));
        tma_load_4d(base + kOffK, &tm_k, bar_load, 0, t.hk, nb * kBlockN, t.b);
        bulk_load(base + kOffSFK,
                  p.k_sf + t.b * p.ksf_stride_b + t.hk * p.ksf_stride_h + (int64_t)nb * kSfBytes,
                  kSfBytes, bar_load);
        tma_load_4d(base + kOffV, &tm_v, bar_load, nb * (kBlockN / 2), 0, t.hk, t.b);
        bulk_load(base + kOffSFV,
                  p.v_sf + t.b * p.vsf_stride_b + t.hk * p.vsf_stride_h + (int64_t)nb * kSfBytes,
                  kSfBytes, bar_load);
        load_pending = true;
      }
      ok = mbar_wait(bar_load, ph_load, wc, kSiteLoad);
      ph_load ^= 1;
      if (!ok) break;
      // ---- S = Q K^T -------------------------------------------------------------------------
      if (tid == 0) {
        load_pending = false;
        tc_fence_after_sync();
        tc_cp_sf(tmem + kTmSFK, base + kOffSFK);
        tc_cp_sf(tmem + kTmSFK + 4, base + kOffSFK + 512);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const uint64_t da = make_smem_desc(base + kOffQ + 32 * j, 16, 512, kSwizzle64);
          const uint64_t db = make_smem_desc(base + kOffK + 32 * j, 16, 512, kSwizzle64);
          mma_nvf4(tmem + kTmS0, da, db, idesc, tmem + kTmSFQ + 4 * j, tmem + kTmSFK + 4 * j, j);
        }
        tc_commit(bar_mma);
        mma_pending = true;
      }
      ok = mbar_wait(bar_mma, ph_mma, wc, kSiteMma);
      ph_mma ^= 1;
      if (!ok) break;
      if (tid == 0) mma_pending = false;
      tc_fence_after_sync();

      // ---- softmax + quantisation of P --------------------------------------------------------
      float s[128];
#pragma unroll
      for (int c = 0; c < 4; ++c)
        tmem_ld32(lane_addr + kTmS0 + 32 * c, reinterpret_cast<uint32_t*>(&s[32 * c]));
      tc_wait_ld();
      if (block_needs_mask(p, t, nb)) mask_row(s, causal_limit(p, t, row, nb));
      float bm[8];
      const float m_loc = row_block_max(s, bm);
      const float m_new = next_reference(m_ref, m_loc, p.sl2);
      if (i > 0 && __any_sync(0xffffffffu, m_new != m_ref)) {
        // move the accumulator (and the row sum) to the new reference
        const float f = (m_new != m_ref) ? reference_factor(m_ref, m_new, p.sl2) : 1.f;
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
        l_sum *= f;
      }
      m_ref = m_new;
      float noff[8];
      uint32_t ue[2];
      block_exponents(bm, m_ref, p.sl2, noff, ue);
      l_sum += quantize_row(s, noff, ue, p.sl2, gbase + kOffP, row);
      const uint32_t sfw[2] = {block_scale_bytes(ue[0]), block_scale_bytes(ue[1])};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        *reinterpret_cast<uint32_t*>(gbase + kOffSFP + 512 * j + (row & 31) * 16 + (row >> 5) * 4) =
            sfw[j];
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(bar_cta);
      ok = mbar_wait(bar_cta, ph_cta, wc, kSiteCta);
      ph_cta ^= 1;
      if (!ok) break;

      // ---- O += P V ---------------------------------------------------------------------------
      if (tid == 0) {
        tc_fence_after_sync();
        tc_cp_sf(tmem + kTmSFP, base + kOffSFP);
        tc_cp_sf(tmem + kTmSFP + 4, base + kOffSFP + 512);
        tc_cp_sf(tmem + kTmSFV, base + kOffSFV);
        tc_cp_sf(tmem + kTmSFV + 4, base + kOffSFV + 512);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const uint64_t da = make_smem_desc(base + kOffP + 32 * j, 16, 512, kSwizzle64);
          const uint64_t db = make_smem_desc(base + kOffV + 32 * j, 16, 512, kSwizzle64);
          mma_nvf4(tmem + kTmO, da, db, idesc, tmem + kTmSFP + 4 * j, tmem + kTmSFV + 4 * j,
                   (i > 0 || j > 0) ? 1u : 0u);
        }
        tc_commit(bar_mma);
        mma_pending = true;
      }
      ok = mbar_wait(bar_mma, ph_mma, wc, kSiteMma);
      ph_mma ^= 1;
      if (!ok) break;
      if (tid == 0) mma_pending = false;
      tc_fence_after_sync();
    }
  }

  // ---- epilogue ---------------------------------------------------------------------------------
  if (ok) {
    const int q_idx = t.m_blk * kBlockM + row;
    const bool row_valid = q_idx < p.Sq;  // rows of a partial last tile are not stored
    __nv_bfloat16* orow = p.out + t.b * p.o_stride_b + (int64_t)q_idx * p.o_stride_s + t.h * p.o_stride_h;
    const bool empty = (t.n_blocks == 0) || !(l_sum > 0.f);
    const float scale = empty ? 0.f : p.out_scale / l_sum;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t o[32];
      if (t.n_blocks > 0) {
        tmem_ld32(lane_addr + kTmO + 32 * c, o);
        tc_wait_ld();
      }
      if (empty) {
#pragma unroll
        for (int x = 0; x < 32; ++x) o[x] = 0u;
      }
      if (row_valid) store_out_32(orow + 32 * c, o, scale);
    }
    if (p.lse != nullptr && row_valid) {
      p.lse[((int64_t)t.b * p.Hq + t.h) * p.Sq + q_idx] = finish_lse(m_ref, l_sum, p.sl2);
    }
  } else if (tid == 0 && !poisoned) {
    // give copies / MMAs still in flight a bounded chance to land before the CTA goes away
    const WaitCtx drain{s_abort, nullptr, 50ull * 1000 * 1000};
    const uint64_t t0 = globaltimer_ns();
    if (load_pending) {
      while (!mbar_try_wait(bar_load, ph_load ^ 1) && globaltimer_ns() - t0 < drain.budget_ns) {}
    }
    if (mma_pending) {
      while (!mbar_try_wait(bar_mma, ph_mma ^ 1) && globaltimer_ns() - t0 < drain.budget_ns) {}
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace fa4
