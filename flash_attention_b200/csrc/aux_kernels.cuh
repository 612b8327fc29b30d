// Small kernels around the attention forward: scale-factor layout conversion, the
// hardware-contract probe (one Q K^T tile) and the bounded-wait self test.
#pragma once
#include "attn_common.cuh"

namespace fa4 {

// ---------------------------------------------------------------------------------------------
// Scale factors, linear (rows x cols bytes, row stride given) -> 128 x 4 tiles of 512 bytes.
// One thread writes one 16-byte row of a tile chunk: destination offset (r % 32) * 16 holds
// the scales of rows r, r + 32, r + 64, r + 96 (4 bytes each = 4 consecutive columns).
// Grid: x = 32-row-group index over all tiles of all matrices; HBM-bound byte shuffling,
// reads are 4-byte per row (the linear layout offers no more), writes are 16-byte coalesced.
// ---------------------------------------------------------------------------------------------
__global__ void sf_linear_to_tiled_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                          int n_outer, int n_inner, int rows, int cols,
                                          int64_t stride_outer, int64_t stride_inner,
                                          int64_t stride_row, int col_tile_multiple) {
  const int row_tiles = (rows + 127) / 128;
  const int col_tiles = ((cols + 3) / 4 + col_tile_multiple - 1) / col_tile_multiple * col_tile_multiple;
  const int64_t total = (int64_t)n_outer * n_inner * row_tiles * col_tiles * 32;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int l = (int)(idx & 31);
    int64_t tile = idx >> 5;
    const int ct = (int)(tile % col_tiles);
    tile /= col_tiles;
    const int rt = (int)(tile % row_tiles);
    tile /= row_tiles;
    const int mi = (int)(tile % n_inner);
    const int mo = (int)(tile / n_inner);
    const uint8_t* m = src + mo * stride_outer + mi * stride_inner;
    uint32_t w[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int r = rt * 128 + c * 32 + l;
      uint32_t v = 0;
      if (r < rows) {
        const uint8_t* pr = m + (int64_t)r * stride_row + ct * 4;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (ct * 4 + k < cols) v |= (uint32_t)pr[k] << (8 * k);
        }
      }
      w[c] = v;
    }
    reinterpret_cast<uint4*>(dst)[idx] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// ---------------------------------------------------------------------------------------------
// The same conversion for a PACKED batch (sequences concatenated along the token axis, bounds in
// cu_seqlens on the device): every sequence gets its own tiles, padded with zeros to the longest
// sequence, so that a tile never mixes two sequences.
//   packed_rows = 1: the packed axis is the row axis (q / k scales, (total, H, cols)): matrix
//       (b, h) has rows cu[b] .. cu[b+1] at src + row * stride_row + h * stride_inner
//   packed_rows = 0: the packed axis is the column axis (v scales, (H, rows, total / 16)): matrix
//       (b, h) has `rows` rows at src + h * stride_inner + r * stride_row and the columns
//       cu[b] / 16 .. ceil(cu[b+1] / 16) (sequence starts are multiples of 16 keys)
// dst: (num_seqs, n_inner, ceil(max_rows / 128), col tiles of max_cols, 512).
// ---------------------------------------------------------------------------------------------
__global__ void sf_linear_to_tiled_packed_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                 const int32_t* __restrict__ cu, int num_seqs, int n_inner,
                                                 int max_rows, int max_cols, int64_t stride_inner,
                                                 int64_t stride_row, int col_tile_multiple, int packed_rows) {
  const int row_tiles = (max_rows + 127) / 128;
  const int col_tiles = ((max_cols + 3) / 4 + col_tile_multiple - 1) / col_tile_multiple * col_tile_multiple;
  const int64_t total = (int64_t)num_seqs * n_inner * row_tiles * col_tiles * 32;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int l = (int)(idx & 31);
    int64_t tile = idx >> 5;
    const int ct = (int)(tile % col_tiles);
    tile /= col_tiles;
    const int rt = (int)(tile % row_tiles);
    tile /= row_tiles;
    const int mi = (int)(tile % n_inner);
    const int mo = (int)(tile / n_inner);
    const int c0 = cu[mo], c1 = cu[mo + 1];
    const int rows = packed_rows ? (c1 - c0) : max_rows;
    const int cols = packed_rows ? max_cols : ((c1 - c0 + 15) >> 4);
    const uint8_t* m = src + mi * stride_inner + (packed_rows ? (int64_t)c0 * stride_row : (int64_t)(c0 >> 4));
    uint32_t w[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int r = rt * 128 + c * 32 + l;
      uint32_t v = 0;
      if (r < rows) {
        const uint8_t* pr = m + (int64_t)r * stride_row + ct * 4;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (ct * 4 + k < cols) v |= (uint32_t)pr[k] << (8 * k);
        }
      }
      w[c] = v;
    }
    reinterpret_cast<uint4*>(dst)[idx] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// ---------------------------------------------------------------------------------------------
// Probe: S (128 x 128 fp32) = Q tile x K tile^T, head dim 128, through exactly the descriptors
// the attention kernels use.  mode bit 0 = stage operands with plain stores (the path P takes)
// instead of TMA.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128, 1)
qk_tile_probe_kernel(const __grid_constant__ CUtensorMap tm_q,
                     const __grid_constant__ CUtensorMap tm_k, const uint8_t* q, const uint8_t* k,
                     const uint8_t* q_sf, const uint8_t* k_sf, float* s_out, int mode,
                     uint32_t* status, uint64_t budget_ns) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  constexpr uint32_t kOffQ = 0, kOffK = 8192, kOffSFQ = 16384, kOffSFK = 17408, kOffBar = 18432;
  const uint32_t bar_load = base + kOffBar, bar_mma = base + kOffBar + 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + kOffBar + 16);
  volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(gbase + kOffBar + 20);
  const int tid = threadIdx.x, warp = tid >> 5;
  const WaitCtx wc{s_abort, status, budget_ns};

  if (tid == 0) {
    *s_abort = 0u;
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(base + kOffBar + 16, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  bool ok = true;

  if (mode & 1) {
    // plain stores in the swizzled layout + scale chunks copied verbatim
    for (int c = 0; c < 4; ++c) {
      *reinterpret_cast<uint4*>(gbase + kOffQ + sw64_offset(tid, c)) =
          *reinterpret_cast<const uint4*>(q + tid * 64 + c * 16);
      *reinterpret_cast<uint4*>(gbase + kOffK + sw64_offset(tid, c)) =
          *reinterpret_cast<const uint4*>(k + tid * 64 + c * 16);
    }
    if (tid < 64) {
      *reinterpret_cast<uint4*>(gbase + kOffSFQ + tid * 16) = reinterpret_cast<const uint4*>(q_sf)[tid];
      *reinterpret_cast<uint4*>(gbase + kOffSFK + tid * 16) = reinterpret_cast<const uint4*>(k_sf)[tid];
    }
    fence_proxy_async_smem();
  } else {
    if (tid == 0) {
      mbar_arrive_expect_tx(bar_load, 2 * (kTileBytes + kSfBytes));
      tma_load_4d(base + kOffQ, &tm_q, bar_load, 0, 0, 0, 0);
      tma_load_4d(base + kOffK, &tm_k, bar_load, 0, 0, 0, 0);
      bulk_load(base + kOffSFQ, q_sf, kSfBytes, bar_load);
      bulk_load(base + kOffSFK, k_sf, kSfBytes, bar_load);
    }
    ok = __all_sync(0xffffffffu, mbar_wait(bar_load, 0, wc, 1));
  }
  tc_fence_before_sync();
  __syncthreads();
  if (ok) {
    if (tid == 0) {
      tc_fence_after_sync();
      tc_cp_sf(tmem + kTmSFQ, base + kOffSFQ);
      tc_cp_sf(tmem + kTmSFQ + 4, base + kOffSFQ + 512);
      tc_cp_sf(tmem + kTmSFK, base + kOffSFK);
      tc_cp_sf(tmem + kTmSFK + 4, base + kOffSFK + 512);
      constexpr uint32_t idesc = make_idesc_nvf4(128, 128);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint64_t da = make_smem_desc(base + kOffQ + 32 * j, 16, 512, kSwizzle64);
        const uint64_t db = make_smem_desc(base + kOffK + 32 * j, 16, 512, kSwizzle64);
        mma_nvf4(tmem + kTmS0, da, db, idesc, tmem + kTmSFQ + 4 * j, tmem + kTmSFK + 4 * j, j);
      }
      tc_commit(bar_mma);
    }
    ok = __all_sync(0xffffffffu, mbar_wait(bar_mma, 0, wc, 2));
    if (ok) {
      tc_fence_after_sync();
      const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(lane_addr + kTmS0 + 32 * c, r);
        tc_wait_ld();
#pragma unroll
        for (int x = 0; x < 32; ++x) s_out[tid * 128 + 32 * c + x] = __uint_as_float(r[x]);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

// ---------------------------------------------------------------------------------------------
// Split-KV combine (the reference's flash_fwd_combine.py; math of
// tests/cute/test_flash_attn_fast.py:295-300): per output row
//   lse = log sum_i exp(lse_i),   out = sum_i exp(lse_i - lse) * out_i
// over the splits' normalised fp32 partial outputs.  One thread = four neighbouring columns of
// one (batch, query, head) row; HBM-bound: reads num_splits * (Dv + 1) floats, writes Dv bf16.
// ---------------------------------------------------------------------------------------------
__global__ void combine_splits_kernel(const float* __restrict__ o_partial,
                                      const float* __restrict__ lse_partial,
                                      __nv_bfloat16* __restrict__ out, float* __restrict__ lse,
                                      int num_splits, int B, int Sq, int Hq, int Dv,
                                      int64_t o_stride_b, int64_t o_stride_s, int64_t o_stride_h) {
  const int per_row = Dv / 4;
  const int64_t rows = (int64_t)B * Sq * Hq;
  const int64_t split_o = rows * Dv, split_l = rows;
  // When launched as a programmatic dependent of the kernel that writes the partials (decode
  // path) the CTAs may start before that kernel has finished: wait for it here.  A plain launch
  // returns from this at once.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < rows * per_row;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(idx % per_row);
    const int64_t r = idx / per_row;  // (b, s, h) in the partial layout
    const int h = (int)(r % Hq);
    const int64_t bs = r / Hq;
    const int s = (int)(bs % Sq), b = (int)(bs / Sq);
    const int64_t l_idx = ((int64_t)b * Hq + h) * Sq + s;
    // loads in batches of eight, all in flight before the first is used: the partials come from L2
    // (the kernel before wrote them) and a chain of dependent round trips would set the pace
    constexpr int kBatch = 8;
    float m = -INFINITY;
    for (int i0 = 0; i0 < num_splits; i0 += kBatch) {
      float l[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) l[j] = (i0 + j < num_splits) ? lse_partial[(i0 + j) * split_l + l_idx] : -INFINITY;
#pragma unroll
      for (int j = 0; j < kBatch; ++j) m = fmaxf(m, l[j]);
    }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float sum = 0.f;
    if (m != -INFINITY) {
      for (int i0 = 0; i0 < num_splits; i0 += kBatch) {
        float l[kBatch];
        float4 v[kBatch];
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
          const bool live = i0 + j < num_splits;
          l[j] = live ? lse_partial[(i0 + j) * split_l + l_idx] : -INFINITY;
          v[j] = live ? *reinterpret_cast<const float4*>(o_partial + (i0 + j) * split_o + r * Dv + 4 * c)
                      : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {   // ascending split order, as before
          const float w = __expf(l[j] - m);  // exp(-inf) = 0 for the padding of the last batch
          sum += w;
          acc.x = fmaf(w, v[j].x, acc.x);
          acc.y = fmaf(w, v[j].y, acc.y);
          acc.z = fmaf(w, v[j].z, acc.z);
          acc.w = fmaf(w, v[j].w, acc.w);
        }
      }
      const float inv = 1.f / sum;
      acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    }
    __nv_bfloat16* dst = out + b * o_stride_b + (int64_t)s * o_stride_s + h * o_stride_h + 4 * c;
    uint2 pk;
    pk.x = pack_bf16x2(acc.x, acc.y);
    pk.y = pack_bf16x2(acc.z, acc.w);
    *reinterpret_cast<uint2*>(dst) = pk;
    if (c == 0 && lse != nullptr) lse[l_idx] = (m == -INFINITY) ? -INFINITY : m + __logf(sum);
  }
}

// ---------------------------------------------------------------------------------------------
// Tensor-pipe rate of the block-scaled e2m1 MMA (the denominator "measured FP4 peak"): every CTA
// (one per SM) fills one A and one B tile and their scale chunks with pseudo-random bytes, then
// one thread issues `iters` 128 x 128 x 64 instructions back to back, alternating between two
// accumulators, and the CTA reports the clocks from the first issue to the completion of the
// last.  Nothing is read from or written to HBM inside the timed part.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128, 1)
mma_rate_kernel(int iters, unsigned long long* clocks_out, uint32_t* status, uint64_t budget_ns) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  constexpr uint32_t kOffA = 0, kOffB = 8192, kOffSFA = 16384, kOffSFB = 17408, kOffBar = 18432;
  const uint32_t bar_mma = base + kOffBar;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + kOffBar + 16);
  volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(gbase + kOffBar + 20);
  const int tid = threadIdx.x, warp = tid >> 5;
  const WaitCtx wc{s_abort, status, budget_ns};

  if (tid == 0) {
    *s_abort = 0u;
    mbar_init(bar_mma, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(base + kOffBar + 16, kTmemCols);
    tmem_relinquish();
  }
  // operand bytes: any nibble is a valid e2m1; scale bytes 0x30..0x3f are ue4m3 values 2^-1..2
  uint32_t x = 0x9e3779b9u * (blockIdx.x * 128u + tid + 1u);
  for (int i = tid; i < 16384 / 4; i += 128) {
    x = x * 1664525u + 1013904223u;
    reinterpret_cast<uint32_t*>(gbase + kOffA)[i] = x ^ (x >> 13);
  }
  for (int i = tid; i < 2048 / 4; i += 128) {
    x = x * 1664525u + 1013904223u;
    reinterpret_cast<uint32_t*>(gbase + kOffSFA)[i] = 0x30303030u | ((x >> 8) & 0x0f0f0f0fu);
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  long long t0 = 0;
  if (tid == 0) {
    tc_cp_sf(tmem + kTmSFQ, base + kOffSFA);
    tc_cp_sf(tmem + kTmSFQ + 4, base + kOffSFA + 512);
    tc_cp_sf(tmem + kTmSFK, base + kOffSFB);
    tc_cp_sf(tmem + kTmSFK + 4, base + kOffSFB + 512);
    constexpr uint32_t idesc = make_idesc_nvf4(128, 128);
    const uint64_t da0 = make_smem_desc(base + kOffA, 16, 512, kSwizzle64);
    const uint64_t db0 = make_smem_desc(base + kOffB, 16, 512, kSwizzle64);
    const uint64_t da1 = make_smem_desc(base + kOffA + 32, 16, 512, kSwizzle64);
    const uint64_t db1 = make_smem_desc(base + kOffB + 32, 16, 512, kSwizzle64);
    t0 = clock64();
#pragma unroll 1
    for (int i = 0; i < iters; i += 4) {
      // a fresh accumulation every 4 instructions per accumulator keeps the sums finite
      mma_nvf4(tmem + kTmS0, da0, db0, idesc, tmem + kTmSFQ, tmem + kTmSFK, 0);
      mma_nvf4(tmem + kTmS1, da0, db0, idesc, tmem + kTmSFQ, tmem + kTmSFK, 0);
      mma_nvf4(tmem + kTmS0, da1, db1, idesc, tmem + kTmSFQ + 4, tmem + kTmSFK + 4, 1);
      mma_nvf4(tmem + kTmS1, da1, db1, idesc, tmem + kTmSFQ + 4, tmem + kTmSFK + 4, 1);
    }
    tc_commit(bar_mma);
  }
  const bool ok = __all_sync(0xffffffffu, mbar_wait(bar_mma, 0, wc, 3));
  if (tid == 0 && ok) clocks_out[blockIdx.x] = static_cast<unsigned long long>(clock64() - t0);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

// ---------------------------------------------------------------------------------------------
// Rate of the exponential unit (the denominator of the kernel's exponential roofline): every
// thread of 16 warps per CTA runs `iters` rounds of 16 independent ex2.approx, nothing else in
// the loop competes for the unit; the CTA reports its clocks.  exp2 per clock per SM =
// 512 threads * iters * 16 / clocks.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512, 1)
ex2_rate_kernel(int iters, unsigned long long* clocks_out, float* sink) {
  float x[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) x[i] = -1.f - 0.01f * (float)(threadIdx.x + i);
  __syncthreads();
  const long long t0 = clock64();
#pragma unroll 1
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < 16; ++i) x[i] = ex2_approx(x[i]) - 1.5f;   // stays in (-1.5, -0.5): no denormals
  }
  const long long t1 = clock64();
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) acc += x[i];
  if (acc == 12345.678f) *sink = acc;   // keeps the loop alive
  __syncthreads();
  if (threadIdx.x == 0) clocks_out[blockIdx.x] = static_cast<unsigned long long>(t1 - t0);
}

// ---------------------------------------------------------------------------------------------
// Bounded-wait self test: a barrier nothing arrives at.
// ---------------------------------------------------------------------------------------------
__global__ void wait_expiry_kernel(uint32_t* status, uint64_t budget_ns) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0u;
    mbar_init(smem_u32(&bar), 1);
    fence_barrier_init();
  }
  __syncthreads();
  const WaitCtx wc{&abort_flag, status, budget_ns};
  (void)mbar_wait(smem_u32(&bar), 0, wc, 99);
  __syncthreads();
}

}  // namespace fa4
