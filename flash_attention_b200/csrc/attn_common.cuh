// Parameters and tile bookkeeping shared by the attention kernels (head dim 128 family).
#pragma once
#include "ptx.cuh"
#include "softmax.cuh"
#include <cuda_bf16.h>

namespace fa4 {

constexpr int kBlockM = 128;  // query rows per CTA tile (= tensor-memory lanes)
constexpr int kBlockN = 128;  // keys per K/V block

// tensor-memory column map (512 columns allocated) shared by the 128-key kernel, the decode
// kernel and the probes; the 64-key kernel has its own map
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmS0 = 0, kTmS1 = 128, kTmO = 256;
constexpr uint32_t kTmSFQ = 384;  // 8 columns: 2 MMA K-steps x 4
constexpr uint32_t kTmSFK = 392;  // 2 buffers x 8
constexpr uint32_t kTmSFV = 408;  // 2 buffers x 8
constexpr uint32_t kTmSFP = 424;  // 2 buffers x 8

constexpr uint32_t kTileBytes = 128 * 64;  // one 128-row x 128-element e2m1 tile
constexpr uint32_t kSfBytes = 1024;        // its scale factors: 2 chunks of 512

// Shared memory the single-tile probes request: padded so that only one CTA fits per SM (every
// CTA allocates all 512 tensor-memory columns, and a second resident CTA would block inside
// tcgen05.alloc).
constexpr uint32_t kProbeSmemRequest = 120 * 1024;

struct KernelParams {
  const uint8_t* q_sf;  // tiled scale factors, see fa4_nvfp4.h
  const uint8_t* k_sf;
  const uint8_t* v_sf;
  __nv_bfloat16* out;
  float* lse;
  uint32_t* status;
  int64_t o_stride_b, o_stride_s, o_stride_h;  // elements
  int64_t qsf_stride_b, qsf_stride_h;          // bytes between batches / heads of tiled SFs
  int64_t ksf_stride_b, ksf_stride_h;
  int64_t vsf_stride_b, vsf_stride_h;
  int B, Sq, Sk, Hq, Hkv, group;
  // divisors of the tile-list arithmetic, as multiply-high + shift: every warp decodes every tile
  FastDiv div_tiles_per_m;   // Hq * B
  FastDiv div_hq, div_group, div_splits;
  int num_m_blocks, num_n_blocks;
  int causal;
  float sl2;        // softmax_scale * q_scale * k_scale * log2(e)
  float out_scale;  // v_scale
  uint64_t budget_ns;
  uint32_t epoch;   // launch epoch (0..255): a failure in the status word stops only the launch that recorded it
  // split-KV (num_splits > 1): every (tile, split) pair is a work item that visits a contiguous
  // share of the tile's K/V blocks and writes a normalised fp32 partial O and a partial LSE;
  // combine_splits_kernel merges them (flash_attn/cute/interface.py:494-510,804-812 and
  // flash_fwd_combine.py in the reference)
  int num_splits;
  float* o_partial;    // (num_splits, B, Sq, Hq, Dv) fp32
  float* lse_partial;  // (num_splits, B, Hq, Sq) fp32
  int Dv;
  // local (sliding-window) attention, general instantiation only: query row i sees keys j with
  //   i + Sk - Sq - win_left <= j <= i + Sk - Sq + win_right        (-1 = no limit on that side)
  // (flash_attn/cute/testing.py:249-288 construct_local_mask; mask.py:487-527).  `causal` is set
  // whenever the right limit exists; plain causal is win_right == 0, win_left == -1.
  int win_left, win_right;
  // learnable sink (general instantiation only): one extra logit per query head, in natural-log
  // units of the scaled scores, that takes part in the normalisation and in the LSE but has no
  // value row (flash_attn/cute/flash_fwd_sm100.py:2383-2394, testing.py:406-416); null = none
  const float* sink;
  // soft cap (general instantiation only): 0 = off; otherwise the raw products s become
  // tanh(s * softcap_c1) with softcap_c1 = softmax_scale * q_scale * k_scale / softcap, and sl2 is
  // softcap * log2(e) instead of the product of the scales
  float softcap_c1;
  // KV cache (general instantiation only).  seqused_k: per batch entry the number of valid keys
  // (<= Sk; causal alignment and masks then use it in place of Sk); NULL = Sk for all.
  // page_table: K / V / their scales live in a pool of pages of page_size keys (a multiple of
  // 128) and logical key block nb of batch entry b sits in page page_table[b * pages_per_seq +
  // nb * 128 / page_size]; the K / V tensor maps and scale strides then describe the POOL
  // (their batch dimension is the page).  NULL = contiguous operands.
  const int32_t* seqused_k;
  const int32_t* page_table;
  int page_size, pages_per_seq;
  // Packed variable-length batch (general instantiation only; the reference's cu_seqlens_q /
  // cu_seqlens_k, flash_attn/cute/interface.py:1795-1840): q, k, v, out are packed along the token
  // axis without a batch dimension, sequence b owns query rows cu_seqlens_q[b] .. cu_seqlens_q[b+1]
  // and keys cu_seqlens_k[b] .. cu_seqlens_k[b+1] (B = number of sequences; Sq / Sk = the longest
  // sequence, which sizes the tile grid -- tiles past a sequence's end visit nothing).  The tiled
  // scales stay per sequence, padded to that longest length.  LSE is (Hq, total_q).  NULL = dense.
  const int32_t* cu_seqlens_q;
  const int32_t* cu_seqlens_k;
  const int32_t* cu_seqlens_v;   // starts of the sequences inside V (multiples of 32); null: cu_seqlens_k
  int total_q;
};

// Work tile of a CTA.  Tiles are ordered so that, for causal problems, the m-blocks with the
// most K/V blocks come first (longest-processing-time-first, the idea of the reference's
// SingleTileLPTScheduler, flash_attn/cute/tile_scheduler.py:386-618) and the query heads of one
// kv head are neighbours, so that their K/V tiles are shared through L2.
struct Tile {
  int m_blk, h, b, hk;
  int n_blocks;  // number of K/V blocks this work item visits (0: nothing visible / empty split)
  int nb_top;    // K/V block index of the first visited block; the i-th visited is nb_top - i
  int split;
  int sk;        // valid keys of this batch entry (general instantiation; p.Sk otherwise)
  int sq;        // query rows of this batch entry (packed batches; p.Sq otherwise)
  int q0, k0;    // first packed query row / key of this entry (packed batches; 0 otherwise)
  int v0;        // first key of this entry inside V (packed batches: V pads every sequence to 32 keys)
};

// Query length that masks, block ranges and stores see.
template <bool kGeneral>
__device__ __forceinline__ int query_len(const KernelParams& p, const Tile& t) {
  if constexpr (kGeneral) return t.sq;
  return p.Sq;
}

// Key length that masks and block ranges see.
template <bool kGeneral>
__device__ __forceinline__ int key_len(const KernelParams& p, const Tile& t) {
  if constexpr (kGeneral) return t.sk;
  return p.Sk;
}

// kGeneral = false: the work list is the tile list (num_splits == 1) and the only masks are
// causal / key length; kept as a compile-time switch so that the common case carries none of the
// split or window arithmetic or registers.
// kFast: the three divisions of the tile index as multiply-high + shift instead of the hardware's
// division sequence (about 35 instructions each).  Every warp decodes every tile, so for tiles of
// a few K/V blocks the divisions are a visible share of the work: 1024-token sequences and
// 1024-key windows run 8-20 % faster with them.  Measured as well: the single-lane service warps
// of the 64-key kernel (producer, issuers, scale copier) are better left on the slow form in the
// plain instantiation -- with the fast form there the long-tile workloads lose 1-2 % (the warps
// reach their next wait sooner and spend the difference polling), while the softmax and epilogue
// warps gain 1 % from it.
template <bool kGeneral = false, bool kFast = true>
__device__ __forceinline__ Tile decode_tile(const KernelParams& p, int tile_idx) {
  Tile t;
  t.split = 0;
  if constexpr (kGeneral) {
    const int whole = fast_div(tile_idx, p.div_splits);   // the splits of one tile are neighbours in the work list
    t.split = tile_idx - whole * p.num_splits;
    tile_idx = whole;
  }
  const int per_m = p.Hq * p.B;
  const int m_rev = kFast ? fast_div(tile_idx, p.div_tiles_per_m) : tile_idx / per_m;
  const int rem = tile_idx - m_rev * per_m;
  t.b = kFast ? fast_div(rem, p.div_hq) : rem / p.Hq;
  t.h = rem - t.b * p.Hq;
  t.hk = kFast ? fast_div(t.h, p.div_group) : t.h / p.group;
  t.m_blk = p.causal ? (p.num_m_blocks - 1 - m_rev) : m_rev;
  t.sk = p.Sk;
  t.sq = p.Sq;
  t.q0 = 0;
  t.k0 = 0;
  t.v0 = 0;
  int n = p.num_n_blocks;
  if constexpr (kGeneral) {
    if (p.cu_seqlens_q != nullptr) {
      t.q0 = p.cu_seqlens_q[t.b];
      t.sq = p.cu_seqlens_q[t.b + 1] - t.q0;
      t.k0 = p.cu_seqlens_k[t.b];
      t.sk = p.cu_seqlens_k[t.b + 1] - t.k0;
      t.v0 = p.cu_seqlens_v != nullptr ? p.cu_seqlens_v[t.b] : t.k0;
      n = (t.sk + kBlockN - 1) / kBlockN;
    }
    if (p.seqused_k != nullptr) {
      const int used = p.seqused_k[t.b];
      t.sk = used < 0 ? 0 : (used < t.sk ? used : t.sk);
      n = (t.sk + kBlockN - 1) / kBlockN;
    }
    if (t.m_blk * kBlockM >= t.sq) n = 0;   // a tile past the end of a short sequence
  }
  const int sk = key_len<kGeneral>(p, t);
  const int sq = query_len<kGeneral>(p, t);
  if (p.causal) {
    // last visible key of the tile's last row: (m_blk + 1) * 128 - 1 + Sk - Sq
    // (block range of flash_attn/cute/block_info.py:23-55, bottom-right aligned)
    const int last = (t.m_blk + 1) * kBlockM + sk - sq + (kGeneral ? p.win_right : 0);  // exclusive
    int nb = (last + kBlockN - 1) / kBlockN;
    if (last <= 0) nb = 0;
    n = nb < n ? nb : n;
  }
  if constexpr (kGeneral) {
    // first block that holds a visible key of the tile's first row (left window limit)
    int n_min = 0;
    if (p.win_left >= 0) {
      const int first = t.m_blk * kBlockM + sk - sq - p.win_left;
      n_min = first > 0 ? first / kBlockN : 0;
      if (n_min > n) n_min = n;
    }
    const int cnt = n - n_min;
    // visit order is last block first; split s takes visits [s * per, (s + 1) * per)
    const int per = fast_div(cnt + p.num_splits - 1, p.div_splits);
    const int i0 = t.split * per < cnt ? t.split * per : cnt;
    const int i1 = i0 + per < cnt ? i0 + per : cnt;
    t.n_blocks = i1 - i0;
    t.nb_top = n - 1 - i0;
  } else {
    t.n_blocks = n;
    t.nb_top = n - 1;
  }
  return t;
}

// In-block index of the last visible key for query row `row_in_tile` of tile t in K/V block
// `nb` (>= 127 when the block needs no mask for that row).  Two limits combine: the causal one
// (bottom-right aligned, flash_attn/cute/mask.py:369-527) and the key length (keys >= Sk of the
// last, partial block are zero-filled by TMA and must not count; the reference masks them on the
// first-processed block only, flash_fwd_sm100.py:1997-2004).
// (kWindow = false with kGeneral = true: the entry's own key count, no window arithmetic -- what
// split-KV and KV-cache calls without a window use.)
template <bool kGeneral = false, bool kWindow = kGeneral>
__device__ __forceinline__ int causal_limit(const KernelParams& p, const Tile& t, int row_in_tile,
                                            int nb) {
  const int sk = key_len<kGeneral>(p, t);
  const int len_limit = sk - 1 - nb * kBlockN;
  if (!p.causal) return len_limit;
  const int c = t.m_blk * kBlockM + row_in_tile + sk - query_len<kGeneral>(p, t) + (kWindow ? p.win_right : 0) - nb * kBlockN;
  return c < len_limit ? c : len_limit;
}
// In-block index of the FIRST visible key (left window limit); <= 0 when nothing is cut.
__device__ __forceinline__ int lower_limit(const KernelParams& p, const Tile& t, int row_in_tile,
                                           int nb) {
  if (p.win_left < 0) return -(1 << 30);
  return t.m_blk * kBlockM + row_in_tile + t.sk - t.sq - p.win_left - nb * kBlockN;
}
template <bool kGeneral = false, bool kWindow = kGeneral>
__device__ __forceinline__ bool block_needs_mask(const KernelParams& p, const Tile& t, int nb) {
  const int sk = key_len<kGeneral>(p, t);
  const bool partial = (nb + 1) * kBlockN > sk;
  const int off = t.m_blk * kBlockM + sk - query_len<kGeneral>(p, t);
  bool need = partial || (p.causal && (nb * kBlockN + kBlockN - 1 > off + (kWindow ? p.win_right : 0)));
  if constexpr (kWindow) {
    // the last row of the tile has the highest left limit
    need = need || (p.win_left >= 0 && nb * kBlockN < off + kBlockM - 1 - p.win_left);
  }
  return need;
}

// Final scaling and bf16 store of 32 consecutive output columns of one row.
__device__ __forceinline__ void store_out_32(__nv_bfloat16* dst, const uint32_t (&acc)[32],
                                             float scale) {
  uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    uint4 w;
    w.x = pack_bf16x2(__uint_as_float(acc[8 * v + 0]) * scale, __uint_as_float(acc[8 * v + 1]) * scale);
    w.y = pack_bf16x2(__uint_as_float(acc[8 * v + 2]) * scale, __uint_as_float(acc[8 * v + 3]) * scale);
    w.z = pack_bf16x2(__uint_as_float(acc[8 * v + 4]) * scale, __uint_as_float(acc[8 * v + 5]) * scale);
    w.w = pack_bf16x2(__uint_as_float(acc[8 * v + 6]) * scale, __uint_as_float(acc[8 * v + 7]) * scale);
    d4[v] = w;
  }
}

// Natural-log LSE of the scaled scores from the reference maximum (raw units) and the sum of
// p' = 2^kShift * p (flash_attn/cute/flash_fwd_sm100.py:2481-2501).
__device__ __forceinline__ float finish_lse(float m_ref, float l_sum, float sl2) {
  if (!(l_sum > 0.f) || m_ref == kNegInf) return kNegInf;
  return (m_ref * sl2 + lg2_approx(l_sum) - static_cast<float>(kShift)) * 0.6931471805599453f;
}

}  // namespace fa4
