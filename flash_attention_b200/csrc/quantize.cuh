// Fused NVFP4 quantiser of the attention operands: bf16 -> packed e2m1 + ue4m3 block scales
// (linear and / or the tiled layout the attention kernel reads) in one pass over the tensor,
// after one amax pass.  The step directly in front of the attention forward; the reference has
// no quantiser for this path (flash_attn/cute/interface.py:370 rejects anything but fp16/bf16).
//
// Arithmetic (identical, bit for bit, to the CPU oracle's quantize_nvfp4):
//   tensor scale g = amax / (6 * 448)                      (1 when the tensor is all zero)
//   block scale    = e4m3_rne(min((block amax / 6) / g, 448))          per 16 elements
//   element        = e2m1_rne(x / (float(block scale) * g)), no negative zero
// every operation a correctly rounded fp32 one.
//
// All three kernels are HBM-bound byte movers: 2 B read per element in each pass, 9/16 B written.
#pragma once
#include "ptx.cuh"
#include <cuda_bf16.h>

namespace fa4 {

__device__ __forceinline__ float tensor_scale_of(float amax) {
  return amax > 0.f ? __fdiv_rn(amax, 6.f * 448.f) : 1.f;
}

// ue4m3 byte of a non-negative fp32 (round to nearest even, saturating at 448).
__device__ __forceinline__ uint32_t e4m3_byte(float v) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.f), "f"(v));
  return r & 0xffu;
}
__device__ __forceinline__ float e4m3_value(uint32_t byte) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(byte)));
  return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xffffu)));
}

// Clears the sign of nibbles whose magnitude is zero (the formats agree on "no negative zero").
__device__ __forceinline__ uint32_t drop_negative_zero(uint32_t n) {
  const uint32_t mag = n & 0x77777777u;
  const uint32_t nz = ((mag + 0x77777777u) | mag) & 0x88888888u;
  return n & (0x77777777u | nz);
}

// Rare path of quantize_block16: sixteen correctly rounded divisions.  Out of line so that the
// hot loop stays small (it was instruction-fetch bound with this inlined).
struct Block16 {
  float v[16];
};
__device__ __noinline__ uint2 quantize_block16_exact(Block16 x, float denom) {
  float y[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) y[i] = denom > 0.f ? __fdiv_rn(x.v[i], denom) : 0.f;
  return make_uint2(pack8_e2m1(y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7]),
                    pack8_e2m1(y[8], y[9], y[10], y[11], y[12], y[13], y[14], y[15]));
}

// Correctly rounded a / b from the correctly rounded reciprocal rb = RN(1 / b) and nb = -b: the
// product a rb is within 2 ulp of the quotient, one residual step (the residual a - y b is exact
// in an FMA) makes it faithful and a second one correctly rounded (Markstein's division theorem).
// Five FMA-pipe instructions where a library division takes a dozen and a branch.  Needs finite
// rb and residuals that do not underflow: callers keep operands near the bottom of the fp32
// range on the library path.
__device__ __forceinline__ float div_rn_by(float a, float nb, float rb) {
  const float y0 = __fmul_rn(a, rb);
  const float y1 = fmaf(fmaf(y0, nb, a), rb, y0);
  return fmaf(fmaf(y1, nb, a), rb, y1);
}
// The same for a pair (packed fp32 instructions: both lanes round like the scalar ones).
__device__ __forceinline__ float2 div_rn_by2(float2 a, float2 nb, float2 rb) {
  const float2 y0 = __fmul2_rn(a, rb);
  const float2 y1 = __ffma2_rn(__ffma2_rn(y0, nb, a), rb, y0);
  return __ffma2_rn(__ffma2_rn(y1, nb, a), rb, y1);
}

// Per-tensor constants of the quantisers: the tensor scale g, -g, RN(1 / g), and whether g is so
// small (below 1e-18) that the residual steps above could underflow where it matters: then the
// block scales take the library division.
struct TensorScale {
  float g, neg_g, rcp_g;
  bool tiny;
};
__device__ __forceinline__ TensorScale make_tensor_scale(float amax) {
  TensorScale t;
  t.g = tensor_scale_of(amax);
  t.neg_g = -t.g;
  t.tiny = !(t.g >= 1e-18f);
  t.rcp_g = t.tiny ? 0.f : __frcp_rn(t.g);
  return t;
}

// One block of 16 values -> 8 packed bytes (two words) and its scale byte.
__device__ __forceinline__ void quantize_block16(const float (&x)[16], const TensorScale& ts, uint32_t& lo,
                                                 uint32_t& hi, uint32_t& sf_byte) {
  const float g = ts.g;
  // |x| maxima of the block (two chains)
  float bm0 = fmaxf(fabsf(x[0]), fabsf(x[1])), bm1 = fmaxf(fabsf(x[2]), fabsf(x[3]));
#pragma unroll
  for (int i = 4; i < 16; i += 2) {
    bm0 = fmaxf(bm0, fabsf(x[i]));
    bm1 = fmaxf(bm1, fabsf(x[i + 1]));
  }
  const float bmax = fmaxf(bm0, bm1);
  // block scale = e4m3_rne(min((bmax / 6) / g, 448)).  With g >= 1e-18 every quotient that can
  // reach the first rounding boundary of e4m3 (2^-10) has exact residuals; smaller quotients give
  // the zero byte whatever their last bits are.
  constexpr float kRcp6 = 0.16666667163372039794921875f;   // RN(1 / 6)
  float t;
  if (ts.tiny) {
    t = __fdiv_rn(__fdiv_rn(bmax, 6.f), g);
  } else {
    t = div_rn_by(div_rn_by(bmax, -6.f, kRcp6), ts.neg_g, ts.rcp_g);
  }
  sf_byte = e4m3_byte(fminf(t, 448.f));
  const float denom = __fmul_rn(e4m3_value(sf_byte), g);
  // The element codes are those of the correctly rounded quotients x / denom.  Denominators near
  // the bottom of the fp32 range take the out-of-line exact path; quotients that small are far
  // below the first rounding boundary (0.25) whatever the residuals do.
  if (denom < 1e-30f) {
    Block16 blk;
#pragma unroll
    for (int i = 0; i < 16; ++i) blk.v[i] = x[i];
    const uint2 e = quantize_block16_exact(blk, denom);
    lo = e.x;
    hi = e.y;
  } else {
    const float r = __frcp_rn(denom);
    const float2 rr = make_float2(r, r), nd = make_float2(-denom, -denom);
    float2 y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = div_rn_by2(make_float2(x[2 * i], x[2 * i + 1]), nd, rr);
    lo = pack8_e2m1(y[0].x, y[0].y, y[1].x, y[1].y, y[2].x, y[2].y, y[3].x, y[3].y);
    hi = pack8_e2m1(y[4].x, y[4].y, y[5].x, y[5].y, y[6].x, y[6].y, y[7].x, y[7].y);
  }
  lo = drop_negative_zero(lo);
  hi = drop_negative_zero(hi);
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& v, float* out) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// ---------------------------------------------------------------------------------------------
// amax over a (n0, n1, n2, inner) bf16 tensor with contiguous last dimension.  A "row" is one
// (i0, i1) pair = n2 * inner / 8 chunks of 16 bytes; a CTA walks groups of rows with a grid
// stride, several independent 16-byte loads in flight per thread, and ends with ONE atomicMax on
// the bit pattern (values >= 0).  *amax must be zero before the first launch that contributes.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
amax_bf16_kernel(const __nv_bfloat16* __restrict__ x, int n1, int n2, int inner8, int64_t s0,
                 int64_t s1, int64_t s2, int rows, int rows_per_group, FastDiv div_per_row,
                 FastDiv div_inner8, FastDiv div_n1, float* __restrict__ amax) {
  __shared__ float warp_max[8];
  const int per_row = n2 * inner8;
  const int per_group = rows_per_group * per_row;
  const int groups = (rows + rows_per_group - 1) / rows_per_group;
  float m = 0.f;
  for (int grp = blockIdx.x; grp < groups; grp += gridDim.x) {
    const int row0 = grp * rows_per_group;
#pragma unroll 4
    for (int item = threadIdx.x; item < per_group; item += 256) {
      const int lr = fast_div(item, div_per_row), within = item - lr * per_row;
      const int row = row0 + lr;
      if (row < rows) {
        const int i2 = fast_div(within, div_inner8), c = within - i2 * inner8;
        const int i0 = fast_div(row, div_n1), i1 = row - i0 * n1;
        const uint4 v = *reinterpret_cast<const uint4*>(x + i0 * s0 + i1 * s1 + i2 * s2 + c * 8);
        // |bf16| maxima compare like their bit patterns with the sign cleared
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          m = fmaxf(m, __uint_as_float((w[i] << 16) & 0x7fffffffu));
          m = fmaxf(m, __uint_as_float(w[i] & 0x7fff0000u));
        }
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, warp_max[w]);
    if (m > 0.f) atomicMax(reinterpret_cast<int*>(amax), __float_as_int(m));
  }
}

// ---------------------------------------------------------------------------------------------
// Q / K: x (B, S, H, D) bf16, blocks along D.  One item = one block of 16 elements (two 16-byte
// loads, one 8-byte store); a CTA takes a group of (b, s) rows, H * D/16 blocks each, about
// eight items per thread.
// The row index runs over S padded to a multiple of 128 so that the tiled scale layout gets its
// zero padding from the same pass.
//   packed    (B, S, H, D/2)  contiguous
//   sf_lin    (B, S, H, D/16) contiguous, or null
//   sf_tiled  (B, H, ceil(S/128), ceil(D/64), 512), or null
// D is a multiple of 64 (four blocks = one 4-byte word of either scale layout); per_group is a
// multiple of 4, so the four lanes that assemble a word always sit in one warp iteration.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const __nv_bfloat16* __restrict__ x, int B, int S, int H, int D, int64_t sb,
                     int64_t ss, int64_t sh, const float* __restrict__ amax,
                     uint8_t* __restrict__ packed, uint8_t* __restrict__ sf_lin,
                     uint8_t* __restrict__ sf_tiled, float* __restrict__ scale_out,
                     int rows_per_group, FastDiv div_per_row, FastDiv div_nb, FastDiv div_spad) {
  const TensorScale g = make_tensor_scale(*amax);
  if (scale_out != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *scale_out = g.g;
  const int nb = D / 16, ct = D / 64;
  const int rt = (S + 127) / 128, s_pad = rt * 128;
  const int rows = B * s_pad;
  const int per_row = H * nb;
  const int per_group = rows_per_group * per_row;
  const int row0 = blockIdx.x * rows_per_group;
  // Every lane of a warp runs the same number of iterations (shuffles below).  kBatch items per
  // thread are loaded before any is processed (2 measured the same, 4 slower: the ALU and FMA
  // pipes are 55-66 % busy and two thirds of the issue slots are used; loads in flight are not
  // what limits it).
  constexpr int kBatch = 1;
  const int iters = (per_group + 256 * kBatch - 1) / (256 * kBatch);
  for (int it = 0; it < iters; ++it) {
    uint4 raw[kBatch][2];
    int s_of[kBatch], b_of[kBatch], h_of[kBatch], c_of[kBatch];
    bool in_range[kBatch];
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      const int item = (it * kBatch + k) * 256 + threadIdx.x;
      const int lr = fast_div(item, div_per_row), within = item - lr * per_row;
      const int row = row0 + lr;
      h_of[k] = fast_div(within, div_nb);
      c_of[k] = within - h_of[k] * nb;
      b_of[k] = fast_div(row, div_spad);
      s_of[k] = row - b_of[k] * s_pad;
      in_range[k] = item < per_group && row < rows;
      raw[k][0] = raw[k][1] = make_uint4(0u, 0u, 0u, 0u);
      if (in_range[k] && s_of[k] < S) {
        const __nv_bfloat16* src = x + b_of[k] * sb + s_of[k] * ss + h_of[k] * sh + c_of[k] * 16;
        raw[k][0] = *reinterpret_cast<const uint4*>(src);
        raw[k][1] = *reinterpret_cast<const uint4*>(src + 8);
      }
    }
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      const int s = s_of[k], b = b_of[k], h = h_of[k], c = c_of[k];
      uint32_t lo = 0, hi = 0, sfb = 0;
      if (in_range[k] && s < S) {
        float v[16];
        unpack_bf16x8(raw[k][0], v);
        unpack_bf16x8(raw[k][1], v + 8);
        quantize_block16(v, g, lo, hi, sfb);
        const int64_t orow = ((int64_t)b * S + s) * H + h;
        *reinterpret_cast<uint2*>(packed + (orow * nb + c) * 8) = make_uint2(lo, hi);
      }
      // four neighbouring lanes hold the four scale bytes of one word
      uint32_t word = sfb << (8 * (c & 3));
      word |= __shfl_xor_sync(0xffffffffu, word, 1);
      word |= __shfl_xor_sync(0xffffffffu, word, 2);
      if (in_range[k] && (c & 3) == 0) {
        if (sf_lin != nullptr && s < S) {
          const int64_t orow = ((int64_t)b * S + s) * H + h;
          *reinterpret_cast<uint32_t*>(sf_lin + orow * nb + c) = word;
        }
        if (sf_tiled != nullptr) {
          const int64_t chunk = (((int64_t)b * H + h) * rt + s / 128) * ct + c / 4;
          const int rr = s % 128;
          *reinterpret_cast<uint32_t*>(sf_tiled + chunk * 512 + (rr % 32) * 16 + (rr / 32) * 4) = word;
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// V: x (B, Sk, H, Dv) bf16 -> key-contiguous packed (B, H, Dv, Sk/2), blocks along the keys.
// One CTA transposes a tile of 128 keys x 128 d through shared memory (16-byte chunks swizzled
// by the key block so that both the row-wise fill and the column-wise reads are conflict free).
// One thread = two neighbouring d rows x one block of 16 keys.
//   sf_lin    (B, H, Dv, Sk/16) contiguous, or null
//   sf_tiled  (B, H, ceil(Dv/128), 2 * ceil(Sk/128), 512), or null
// Sk is a multiple of 16 and Dv a multiple of 8.  grid = (ceil(Sk/128), ceil(Dv/128), B * H).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
quantize_v_kernel(const __nv_bfloat16* __restrict__ x, int B, int Sk, int H, int Dv, int64_t sb,
                  int64_t ss, int64_t sh, const float* __restrict__ amax,
                  uint8_t* __restrict__ packed, uint8_t* __restrict__ sf_lin,
                  uint8_t* __restrict__ sf_tiled, float* __restrict__ scale_out) {
  __shared__ __align__(16) uint8_t tile[128 * 256];  // [key][16 chunks of 16 B], chunk ^ (key/16)
  const TensorScale g = make_tensor_scale(*amax);
  if (scale_out != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 &&
      threadIdx.x == 0)
    *scale_out = g.g;
  const int k0 = blockIdx.x * 128, d0 = blockIdx.y * 128;
  const int b = blockIdx.z / H, h = blockIdx.z % H;
  const int tid = threadIdx.x;

  // fill: 128 keys x 16 chunks of 8 d values; zero outside the tensor
#pragma unroll
  for (int i = tid; i < 128 * 16; i += 256) {
    const int key = i >> 4, ch = i & 15;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (k0 + key < Sk && d0 + ch * 8 < Dv)
      v = *reinterpret_cast<const uint4*>(x + b * sb + (int64_t)(k0 + key) * ss + h * sh + d0 + ch * 8);
    *reinterpret_cast<uint4*>(tile + key * 256 + ((ch ^ (key >> 4)) << 4)) = v;
  }
  __syncthreads();

  const int n_kb_total = Sk / 16;
  const int kt = (Sk + 127) / 128;  // 128-key tiles
  const int dt = (Dv + 127) / 128;
#pragma unroll 1
  for (int item = tid; item < 64 * 8; item += 256) {
    const int kb = item & 7, dp = item >> 3;  // key block inside the tile, d pair
    const int d = d0 + 2 * dp;
    const int ch = dp >> 2, within = (dp & 3) * 4;  // chunk and byte offset of the d pair
    float v0[16], v1[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int key = 16 * kb + j;
      const uint32_t w =
          *reinterpret_cast<const uint32_t*>(tile + key * 256 + ((ch ^ kb) << 4) + within);
      v0[j] = __uint_as_float(w << 16);
      v1[j] = __uint_as_float(w & 0xffff0000u);
    }
    uint32_t lo0, hi0, sf0, lo1, hi1, sf1;
    quantize_block16(v0, g, lo0, hi0, sf0);
    quantize_block16(v1, g, lo1, hi1, sf1);
    const bool key_ok = k0 + 16 * kb < Sk;
    const int64_t row0 = ((int64_t)b * H + h) * Dv + d;
    if (key_ok && d < Dv)
      *reinterpret_cast<uint2*>(packed + row0 * (Sk / 2) + (k0 + 16 * kb) / 2) = make_uint2(lo0, hi0);
    if (key_ok && d + 1 < Dv)
      *reinterpret_cast<uint2*>(packed + (row0 + 1) * (Sk / 2) + (k0 + 16 * kb) / 2) =
          make_uint2(lo1, hi1);
    // scale bytes: lanes kb = 4 q .. 4 q + 3 hold one word of either layout
    if (!key_ok) sf0 = sf1 = 0;
    uint32_t w0 = sf0 << (8 * (kb & 3)), w1 = sf1 << (8 * (kb & 3));
    w0 |= __shfl_xor_sync(0xffffffffu, w0, 1);
    w0 |= __shfl_xor_sync(0xffffffffu, w0, 2);
    w1 |= __shfl_xor_sync(0xffffffffu, w1, 1);
    w1 |= __shfl_xor_sync(0xffffffffu, w1, 2);
    if ((kb & 3) == 0) {
      const int kb_global = k0 / 16 + kb;
      if (sf_lin != nullptr && kb_global < n_kb_total) {
        // a word may run past the row's end when Sk/16 is not a multiple of 4: byte stores there
        uint8_t* p0 = sf_lin + row0 * n_kb_total + kb_global;
        const int nvalid = n_kb_total - kb_global < 4 ? n_kb_total - kb_global : 4;
        if (nvalid == 4 && (n_kb_total & 3) == 0) {
          if (d < Dv) *reinterpret_cast<uint32_t*>(p0) = w0;
          if (d + 1 < Dv) *reinterpret_cast<uint32_t*>(p0 + n_kb_total) = w1;
        } else {
          for (int q = 0; q < nvalid; ++q) {
            if (d < Dv) p0[q] = (uint8_t)(w0 >> (8 * q));
            if (d + 1 < Dv) p0[n_kb_total + q] = (uint8_t)(w1 >> (8 * q));
          }
        }
      }
      if (sf_tiled != nullptr) {
        // d rows past Dv inside the 128-row tile get their zero padding here as well
        const int64_t chunk =
            ((((int64_t)b * H + h) * dt + blockIdx.y) * (2 * kt) + 2 * blockIdx.x + kb / 4);
        const int r0 = 2 * dp, r1 = 2 * dp + 1;
        uint8_t* base = sf_tiled + chunk * 512;
        *reinterpret_cast<uint32_t*>(base + (r0 % 32) * 16 + (r0 / 32) * 4) = d < Dv ? w0 : 0u;
        *reinterpret_cast<uint32_t*>(base + (r1 % 32) * 16 + (r1 / 32) * 4) = d + 1 < Dv ? w1 : 0u;
      }
    }
  }
}

}  // namespace fa4
