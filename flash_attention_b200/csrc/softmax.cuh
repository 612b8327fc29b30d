// Per-row online softmax and re-quantisation of P to NVFP4, shared by every kernel variant.
//
// One thread owns one query row of a 128-key block (the 32x32b tensor-memory load gives a
// thread a whole row, as in the reference: flash_attn/cute/flash_fwd_sm100.py:1814-1818).
//
// Behaviour kept from the reference's SoftmaxSm100 (flash_attn/cute/softmax.py:169-279):
//   * the running row maximum is kept in raw score units and the scale
//     (softmax_scale * log2 e) is applied inside one FMA      (softmax.py:222-235)
//   * lazy rescale: the reference maximum only moves when the new maximum exceeds it by more
//     than a threshold in log2 units                          (softmax.py:203-209)
//   * a row that has seen no key uses 0 in place of -inf      (softmax.py:197-204)
//   * the row sum adds the un-rounded fp32 exponentials       (softmax.py:213-218)
//
// New here (the reference converts P to bf16/fp16, flash_fwd_sm100.py:2194-2196): P becomes
// e2m1 with one ue4m3 scale per 16 consecutive keys, the operand format of the block-scaled
// P.V tensor-core instruction.  The scale of a block is a power of two, 2^e with
//   e = clamp(ceil(log2(block max of p') - log2 6), -9, 8),    p' = 2^kShift * p,
// so that the block maximum lands in (3, 6] of the e2m1 grid, and p'/2^e is produced directly
// by the exponential (the exponent offset absorbs e), i.e. the quantisation costs no multiply.
#pragma once
#include "ptx.cuh"
#include <math.h>

namespace fa4 {

// Lazy-rescale threshold and the constant up-shift of P, both in log2 units.  A stale reference
// maximum lets p reach 2^kLazy; block scales are ue4m3 (max 448 >= 2^8), block maxima sit at
// <= 6 * 2^e, hence kLazy + kShift <= 10.  The smallest non-zero p is 2^-(10 + kShift)
// relative to the reference maximum.
constexpr int kLazy = 4;
constexpr int kShift = 6;
constexpr float kLog2Of6 = 2.5849625007f;
static_assert(kLazy + kShift <= 10, "P block scales would overflow ue4m3");

constexpr float kNegInf = -INFINITY;

// Block maxima (8 blocks of 16 keys) and the row maximum of one 128-key row.
__device__ __forceinline__ float row_block_max(const float (&s)[128], float (&bm)[8]) {
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    float m = fmax3(s[16 * b], s[16 * b + 1], s[16 * b + 2]);
#pragma unroll
    for (int j = 3; j < 15; j += 2) m = fmax3(m, s[16 * b + j], s[16 * b + j + 1]);
    bm[b] = fmaxf(m, s[16 * b + 15]);
  }
  float m01 = fmax3(bm[0], bm[1], bm[2]);
  float m23 = fmax3(bm[3], bm[4], bm[5]);
  return fmax3(fmaxf(m01, m23), bm[6], bm[7]);
}

// Next reference maximum given the previous one and this block's row maximum (raw units).
__device__ __forceinline__ float next_reference(float m_prev, float m_loc, float sl2) {
  const bool keep = (m_prev != kNegInf) && ((m_loc - m_prev) * sl2 <= static_cast<float>(kLazy));
  return keep ? m_prev : fmaxf(m_prev, m_loc);
}

// 2^((m_from - m_to) * sl2): the factor that moves a sum / accumulator from reference m_from
// to reference m_to (0 when nothing has been accumulated yet).
__device__ __forceinline__ float reference_factor(float m_from, float m_to, float sl2) {
  return (m_from == kNegInf) ? 0.f : ex2_approx((m_from - m_to) * sl2);
}

// Quantise one row of 128 scores against reference m_ref.
//   pk[16]  packed e2m1, 8 values per word, key order
//   sfw[2]  the 8 block scales as ue4m3 bytes, 4 per word (one word per 64-key MMA step)
//   returns the row's sum of p' (un-rounded), to be added to the running sum
__device__ __forceinline__ float quantize_row(const float (&s)[128], const float (&bm)[8],
                                              float m_ref, float sl2, uint32_t (&pk)[16],
                                              uint32_t (&sfw)[2]) {
  const float msc = (m_ref == kNegInf) ? 0.f : m_ref * sl2;
  float acc = 0.f;
  sfw[0] = 0u;
  sfw[1] = 0u;
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    // log2 of the block maximum of p'
    const float t = fmaf(bm[b], sl2, -msc) + static_cast<float>(kShift);
    const float ef = fminf(fmaxf(ceilf(t - kLog2Of6), -9.f), 8.f);
    const int e = static_cast<int>(ef);
    const float off = msc - static_cast<float>(kShift) + ef;
    float p[16];
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      p[j] = ex2_approx(fmaf(s[16 * b + j], sl2, -off));
      sum += p[j];
    }
    pk[2 * b] = pack8_e2m1(p[0], p[1], p[2], p[3], p[4], p[5], p[6], p[7]);
    pk[2 * b + 1] = pack8_e2m1(p[8], p[9], p[10], p[11], p[12], p[13], p[14], p[15]);
    acc = fmaf(sum, __int_as_float((e + 127) << 23), acc);
    // ue4m3 encoding of 2^e: normal for e >= -6 (exponent field e + 7), subnormal below
    const uint32_t byte = (e >= -6) ? (static_cast<uint32_t>(e + 7) << 3) : (1u << (e + 9));
    sfw[b >> 2] |= byte << (8 * (b & 3));
  }
  return acc;
}

// Causal / key-length mask of one row: keys with in-block index > limit become -inf.
__device__ __forceinline__ void mask_row(float (&s)[128], int limit) {
#pragma unroll
  for (int c = 0; c < 128; ++c) s[c] = (c <= limit) ? s[c] : kNegInf;
}

}  // namespace fa4
