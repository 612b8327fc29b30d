// Per-row online softmax and re-quantisation of P to NVFP4, shared by every kernel variant.
//
// One thread owns one query row of a 128-key block (the 32x32b tensor-memory load gives a
// thread a whole row, as in the reference: flash_attn/cute/flash_fwd_sm100.py:1814-1818).
//
// Behaviour kept from the reference's SoftmaxSm100 (flash_attn/cute/softmax.py:169-279):
//   * the running row maximum is kept in raw score units and the scale
//     (softmax_scale * log2 e) is applied inside one FMA      (softmax.py:222-235)
//   * packed two-wide fp32 FMA / ADD for the scale and the row sum (softmax.py:231)
//   * lazy rescale: the reference maximum only moves when the new maximum exceeds it by more
//     than a threshold in log2 units                          (softmax.py:203-209)
//   * a row that has seen no key uses 0 in place of -inf      (softmax.py:197-204)
//   * the row sum adds the un-rounded fp32 exponentials       (softmax.py:213-218)
//
// New here (the reference converts P to bf16/fp16, flash_fwd_sm100.py:2194-2196): P becomes
// e2m1 with one ue4m3 scale per 16 consecutive keys, the operand format of the block-scaled
// P.V tensor-core instruction.  The scale of a block is a power of two, 2^e with
//   e = clamp(ceil(log2(block max of p') - log2 6), kEMin, 8),    p' = 2^kShift * p,
// so that the block maximum lands in (3, 6] of the e2m1 grid, and p'/2^e is produced directly
// by the exponential (the exponent offset absorbs e), i.e. the quantisation costs no multiply.
//
// Pipe budget per 128x128 block on one SM (measured instruction rates on B200): 16 384
// ex2.approx at 16/clk = 1024 clk on the XU pipe and 8192 cvt.e2m1x2 at 16/clk = 512 clk (the
// two overlap: interleaved they take ~1100 clk, and the profiler's XU counter follows the
// exponentials alone); everything else is arranged to stay well below that on the FMA / ALU
// pipes and in issue slots (packed f32x2 arithmetic, 3-input max, block scales derived with a
// magic-number rounding instead of cvt / ceil, which run at the same low rate).
#pragma once
#include "ptx.cuh"
#include <math.h>

namespace fa4 {

// Lazy-rescale threshold and the constant up-shift of P, both in log2 units.  A stale reference
// maximum lets p reach 2^kLazy; block scales are ue4m3 normals 2^kEMin .. 2^8, block maxima sit
// at <= 6 * 2^e, hence kLazy + kShift <= 10.  The smallest non-zero p is 2^(kEMin - 2 - kShift)
// relative to the reference maximum.
constexpr int kLazy = 4;
constexpr int kShift = 6;
constexpr int kEMin = -6;
constexpr float kLog2Of6 = 2.5849625007f;
static_assert(kLazy + kShift <= 10, "P block scales would overflow ue4m3");

constexpr float kNegInf = -INFINITY;

// ---- packed two-wide fp32 arithmetic (one issue slot for two lanes): the sm_100 intrinsics
// __ffma2_rn / __fadd2_rn on float2 values.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}

// Block maxima (8 blocks of 16 keys) and the row maximum of one 128-key row.
__device__ __forceinline__ float row_block_max(const float (&s)[128], float (&bm)[8]) {
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    float m0 = fmax3(s[16 * b], s[16 * b + 1], s[16 * b + 2]);
    float m1 = fmax3(s[16 * b + 3], s[16 * b + 4], s[16 * b + 5]);
    m0 = fmax3(m0, s[16 * b + 6], s[16 * b + 7]);
    m1 = fmax3(m1, s[16 * b + 8], s[16 * b + 9]);
    m0 = fmax3(m0, s[16 * b + 10], s[16 * b + 11]);
    m1 = fmax3(m1, s[16 * b + 12], s[16 * b + 13]);
    m0 = fmax3(m0, s[16 * b + 14], s[16 * b + 15]);
    bm[b] = fmaxf(m0, m1);
  }
  const float m01 = fmax3(bm[0], bm[1], bm[2]);
  const float m23 = fmax3(bm[3], bm[4], bm[5]);
  return fmax3(fmaxf(m01, m23), bm[6], bm[7]);
}

// Soft cap of a raw score (reference: scores = softcap * tanh(scores / softcap),
// flash_attn/cute/testing.py:373-374; its kernel uses the same hardware approximation): the factor
// softcap is folded into sl2 by the host.  Masked scores stay -inf.
__device__ __forceinline__ float soft_cap(float s, float c1) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(s * c1));
  return (s == kNegInf) ? kNegInf : t;
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

// Per-block exponents of four neighbouring blocks of 16 keys (64 keys) from their maxima.
//   noff[b]  the exponent offset of block b:  p'/2^e = 2^(s * sl2 + noff[b])
//   ue[w]    4 bytes per word, byte k = e + 127 of block 4 w + k (e = block scale exponent)
//
// No cvt / ceil (both would sit on the XU pipe next to the exponentials): u = t + (1.5 * 2^23 +
// 127) rounds t to the nearest integer (t already carries the +0.5 that turns rounding into
// ceil) and leaves e + 127 in the low byte of u's bit pattern.
__device__ __forceinline__ void block_exponents4(const float* bm, float m_ref, float sl2,
                                                 float* noff, uint32_t& ue) {
  constexpr float kMagic = 12582912.f + 127.f;  // 1.5 * 2^23 + exponent bias
  const float msc = (m_ref == kNegInf) ? 0.f : m_ref * sl2;
  // t' = log2(block max of p') - log2 6 + (0.5 - tiny)
  const float c_t = static_cast<float>(kShift) - kLog2Of6 + 0.4999995f - msc;
  const float c_off = static_cast<float>(kShift) - msc;  // noff = c_off - e
  uint32_t ubits[4];
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    float t = fmaf(bm[b], sl2, c_t);
    t = fmaxf(t, static_cast<float>(kEMin) - 0.4f);  // also catches -inf (fully masked block)
    const float u = t + kMagic;
    ubits[b] = __float_as_uint(u);
    noff[b] = c_off - (u - kMagic);
  }
  uint32_t lo, hi;
  asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(lo) : "r"(ubits[0]), "r"(ubits[1]));
  asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(hi) : "r"(ubits[2]), "r"(ubits[3]));
  asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(ue) : "r"(lo), "r"(hi));
}

// The same for a whole row of 128 keys (8 blocks, two words of exponent bytes).
__device__ __forceinline__ void block_exponents(const float (&bm)[8], float m_ref, float sl2,
                                                float (&noff)[8], uint32_t (&ue)[2]) {
  block_exponents4(&bm[0], m_ref, sl2, &noff[0], ue[0]);
  block_exponents4(&bm[4], m_ref, sl2, &noff[4], ue[1]);
}

// The same with GENERAL ue4m3 block scales (three mantissa bits): scale = 2^e (1 + m / 8), the
// smallest such value that is >= (block max of p') / 6, so that the block maximum lands in
// (5.33, 6] of the e2m1 grid instead of (3, 6] -- a quarter less rounding error in O (rel-RMS
// against exact attention 0.10 instead of 0.134 on N(0,1) inputs).  The exponent offset still
// absorbs the scale, noff = c_off - log2(scale), so the exponentials cost nothing more; the price
// is ten more instructions per block here.  In the log2 domain, t = log2(block max / 6):
//   e = floor(t), fr = t - e                      (round-down add of 1.5 * 2^23)
//   m = ceil(8 (2^fr - 1)) in 0..8                (quadratic for 2^fr - 1, error < 0.025 of a
//                                                  step: a block maximum may exceed 6 by 0.3 %
//                                                  and saturate)
//   log2(1 + m / 8) from a nine-entry table
// k = 8 e + m is the scale in units of ue4m3 code steps: the scale byte is k + 56 (m = 8 carries
// into the exponent by itself) and the fp32 bits of the scale are (k + 1016) << 20.
//   noff[b]   exponent offset of block b
//   sf_bytes  the four ue4m3 scale bytes
//   sbits[b]  the scale of block b as fp32 bits (for the row sum)
__constant__ float kLog2OnePlusEighths[9] = {0.0f, 0.1699250042438507f, 0.32192808389663696f,
                                             0.45943161845207214f, 0.5849624872207642f,
                                             0.7004396915435791f, 0.8073549270629883f,
                                             0.9068905711174011f, 1.0f};
constexpr float kPow2m1C1 = 5.2904577f, kPow2m1C2 = 2.6854515f;   // 8 (2^x - 1) ~ x (C1 + C2 x) on [0, 1)
__device__ __forceinline__ void block_scales4_e4m3(const float* bm, float m_ref, float sl2, float* noff,
                                                   uint32_t& sf_bytes, uint32_t* sbits) {
  constexpr float kM = 12582912.f;  // 1.5 * 2^23
  const float msc = (m_ref == kNegInf) ? 0.f : m_ref * sl2;
  const float c_t = static_cast<float>(kShift) - kLog2Of6 - msc;
  const float c_off = static_cast<float>(kShift) - msc;
  uint32_t kb[4];
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    float t = fmaf(bm[b], sl2, c_t);
    t = fmaxf(t, static_cast<float>(kEMin));   // also catches -inf (fully masked block)
    float u;
    asm("add.rm.ftz.f32 %0, %1, %2;" : "=f"(u) : "f"(t), "f"(kM));
    const float e = u - kM;                     // floor(t)
    const float fr = t - e;
    const float g = fr * fmaf(fr, kPow2m1C2, kPow2m1C1);
    const float w = (g + 0.4999995f) + kM;      // round to nearest = ceil(g)
    const float m = w - kM;
    const float lm = kLog2OnePlusEighths[__float_as_uint(w) & 15u];
    noff[b] = (c_off - e) - lm;
    const float kf = fmaf(e, 8.f, m) + (kM + 56.f);   // low byte: 8 e + m + 56, the ue4m3 byte
    kb[b] = __float_as_uint(kf);
    sbits[b] = (kb[b] + 960u) << 20;            // (8 e + m + 1016) << 20: fp32 bits of the scale
  }
  uint32_t lo, hi;
  asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(lo) : "r"(kb[0]), "r"(kb[1]));
  asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(hi) : "r"(kb[2]), "r"(kb[3]));
  asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(sf_bytes) : "r"(lo), "r"(hi));
}

// Which rule the 64-key kernel uses for the P block scales: 0 = powers of two, 1 = general ue4m3.
#ifndef FA4_P_SCALE_E4M3
#define FA4_P_SCALE_E4M3 0
#endif

// ue4m3 bytes of the block scales 2^e from the packed (e + 127) bytes: (e + 7) << 3.
__device__ __forceinline__ uint32_t block_scale_bytes(uint32_t ue_word) {
  return (ue_word - 0x78787878u) << 3;
}

// Quantise two neighbouring key blocks (32 scores) of one row: the unit one 16-byte chunk of the
// P tile holds.  noff0/noff1 and e0/e1 (bytes e + 127) come from block_exponents().
//   out   packed e2m1 of the 32 values, key order
//   returns the sum of p' (un-rounded) over the 32 keys
__device__ __forceinline__ float quantize_pair(const float* s, float noff0, float noff1, uint32_t e0,
                                               uint32_t e1, float sl2, uint4& out) {
  float acc = 0.f;
  uint32_t pk[4];
  const float2 sl2_2 = make_float2(sl2, sl2);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float noff = h ? noff1 : noff0;
    const float2 noff2 = make_float2(noff, noff);
    float2 p[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float2 x = __ffma2_rn(make_float2(s[16 * h + 2 * j], s[16 * h + 2 * j + 1]), sl2_2, noff2);
      p[j] = make_float2(ex2_approx(x.x), ex2_approx(x.y));
    }
    float2 sum_a = __fadd2_rn(p[0], p[1]);
    float2 sum_b = __fadd2_rn(p[2], p[3]);
    sum_a = __fadd2_rn(sum_a, p[4]);
    sum_b = __fadd2_rn(sum_b, p[5]);
    sum_a = __fadd2_rn(sum_a, p[6]);
    sum_b = __fadd2_rn(sum_b, p[7]);
    sum_a = __fadd2_rn(sum_a, sum_b);
    pk[2 * h] = pack8_e2m1(p[0].x, p[0].y, p[1].x, p[1].y, p[2].x, p[2].y, p[3].x, p[3].y);
    pk[2 * h + 1] = pack8_e2m1(p[4].x, p[4].y, p[5].x, p[5].y, p[6].x, p[6].y, p[7].x, p[7].y);
    // 2^e as fp32: byte (e + 127) moved into the exponent field
    acc = fmaf(sum_a.x + sum_a.y, __uint_as_float((h ? e1 : e0) << 23), acc);
  }
  out = make_uint4(pk[0], pk[1], pk[2], pk[3]);
  return acc;
}

// 2^x for a pair on the FMA pipe instead of the exponential unit (the reference mixes the two the
// same way when the exponential unit bounds its kernel: flash_attn/cute/softmax.py:237-279, the
// arithmetic in flash_attn/cute/utils.py:703-737).  Input is NOT x but y = sat((x + 126) / 256),
// which one scalar FMA with the saturate modifier produces from the raw score: the clamp that
// keeps masked (-inf) and hopelessly small scores out of the exponent arithmetic costs no
// instruction of its own.  Steps, all packed two-wide:
//   t = rd(256 y + (M - 126))     M = 1.5 * 2^23: the low mantissa bits of t hold k = floor(x)
//   u = t - (M - 126)             = k + 126, exact
//   f = 256 y - u                 = x - k in [0, 1), one rounding
//   q = 1 + f (c1 + f (c2 + f c3))   minimax fit of 2^f on [0, 1), relative error 8.6e-5
//   result bits = q bits + (t bits << 23)   (k added to the exponent field; k is in [-126, 2])
// A clamped input gives 2^-126, which rounds to an e2m1 zero and adds nothing visible to a sum.
constexpr float kEx2C1 = 0.6951167583465576f, kEx2C2 = 0.22764499485492706f, kEx2C3 = 0.07706703990697861f;
constexpr float kEx2Magic = 12582912.f - 126.f;
__device__ __forceinline__ float ex2_arg_sat(float s, float sl2_256, float c) {
  float y;
  asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(s), "f"(sl2_256), "f"(c));
  return y;
}
__device__ __forceinline__ float2 ex2_emulated2(float2 y) {
  const float2 k256 = make_float2(256.f, 256.f);
  const float2 t = __ffma2_rd(y, k256, make_float2(kEx2Magic, kEx2Magic));
  const float2 u = __fadd2_rn(t, make_float2(-kEx2Magic, -kEx2Magic));
  const float2 f = __ffma2_rn(y, k256, make_float2(-u.x, -u.y));
  float2 q = __ffma2_rn(make_float2(kEx2C3, kEx2C3), f, make_float2(kEx2C2, kEx2C2));
  q = __ffma2_rn(q, f, make_float2(kEx2C1, kEx2C1));
  q = __ffma2_rn(q, f, make_float2(1.f, 1.f));
  uint32_t rx, ry;
  // multiply-add on the FMA pipe (a shift + add would go to the ALU pipe, which the e2m1
  // conversions already load)
  asm("mad.lo.u32 %0, %1, 8388608, %2;" : "=r"(rx) : "r"(__float_as_uint(t.x)), "r"(__float_as_uint(q.x)));
  asm("mad.lo.u32 %0, %1, 8388608, %2;" : "=r"(ry) : "r"(__float_as_uint(t.y)), "r"(__float_as_uint(q.y)));
  return make_float2(__uint_as_float(rx), __uint_as_float(ry));
}

// Which of the 8 pairs of a 16-key block take the FMA-pipe exponential (bit j = pair j, keys 2j and
// 2j + 1 of the block).  The share is a compile-time knob like the reference's ex2_emu_freq
// (flash_attn/cute/flash_fwd_sm100.py:71-90).
#ifndef FA4_EX2_EMU_MASK
#define FA4_EX2_EMU_MASK 0x00u
#endif
constexpr uint32_t kEx2EmuMask = FA4_EX2_EMU_MASK;

// Quantise one block of 16 scores of a row: 8 packed e2m1 bytes (two words); returns the block's
// sum of p' / 2^e (un-rounded; the caller multiplies by the block scale).
template <uint32_t kEmuMask = kEx2EmuMask>
__device__ __forceinline__ float quantize_block16(const float* s, float noff, float sl2,
                                                  uint32_t& pk0, uint32_t& pk1) {
  const float2 sl2_2 = make_float2(sl2, sl2);
  const float2 noff2 = make_float2(noff, noff);
  const float sl2_256 = sl2 * (1.f / 256.f);
  const float c_sat = fmaf(noff, 1.f / 256.f, 126.f / 256.f);
  float2 p[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if ((kEmuMask >> j) & 1u) {
      p[j] = ex2_emulated2(make_float2(ex2_arg_sat(s[2 * j], sl2_256, c_sat),
                                       ex2_arg_sat(s[2 * j + 1], sl2_256, c_sat)));
    } else {
      const float2 x = __ffma2_rn(make_float2(s[2 * j], s[2 * j + 1]), sl2_2, noff2);
      p[j] = make_float2(ex2_approx(x.x), ex2_approx(x.y));
    }
  }
  float2 sum_a = __fadd2_rn(p[0], p[1]);
  float2 sum_b = __fadd2_rn(p[2], p[3]);
  sum_a = __fadd2_rn(sum_a, p[4]);
  sum_b = __fadd2_rn(sum_b, p[5]);
  sum_a = __fadd2_rn(sum_a, p[6]);
  sum_b = __fadd2_rn(sum_b, p[7]);
  sum_a = __fadd2_rn(sum_a, sum_b);
  pk0 = pack8_e2m1(p[0].x, p[0].y, p[1].x, p[1].y, p[2].x, p[2].y, p[3].x, p[3].y);
  pk1 = pack8_e2m1(p[4].x, p[4].y, p[5].x, p[5].y, p[6].x, p[6].y, p[7].x, p[7].y);
  return sum_a.x + sum_a.y;
}

// Quantise one row of 128 scores with the exponents from block_exponents() and store it as one
// row of the P tile (K-major, 64-byte rows, 64-byte swizzle), one 16-byte chunk at a time.
// Returns the row's sum of p' (un-rounded), to be added to the running sum.
__device__ __forceinline__ float quantize_row(const float (&s)[128], const float (&noff)[8],
                                              const uint32_t (&ue)[2], float sl2, uint8_t* p_tile,
                                              uint32_t row) {
  float acc = 0.f;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 chunk;
    acc += quantize_pair(&s[32 * c], noff[2 * c], noff[2 * c + 1],
                         __byte_perm(ue[c >> 1], 0u, 0x4440u + ((2 * c) & 3)),
                         __byte_perm(ue[c >> 1], 0u, 0x4440u + ((2 * c + 1) & 3)), sl2, chunk);
    *reinterpret_cast<uint4*>(p_tile + sw64_offset(row, c)) = chunk;
  }
  return acc;
}

// Causal / key-length mask of one row: keys with in-block index > limit become -inf.
__device__ __forceinline__ void mask_row(float (&s)[128], int limit) {
#pragma unroll
  for (int c = 0; c < 128; ++c) s[c] = (c <= limit) ? s[c] : kNegInf;
}

}  // namespace fa4
