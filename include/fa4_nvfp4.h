/*
 * fa4_nvfp4.h -- C ABI of the B200 (sm_100a) NVFP4 fused attention forward.
 *
 * One shared library (libfa4_nvfp4.so), plain C types only.  Every buffer is
 * owned by the caller and lives in device memory unless stated otherwise; the
 * library allocates nothing per call.  All entry points return 0 on success,
 * a negative FA4_E_* code when an argument is rejected on the host (nothing is
 * launched), or a positive CUDA error code (cudaError_t) when a CUDA runtime
 * call fails.  Device-side failures (a bounded wait that ran out) are reported
 * through the caller's `status` word, see fa4_nvfp4_params::status.
 *
 * Reference interface this boundary replaces (paths inside the reference
 * project, graphcore-research/flash-attention):
 *   flash_attn/cute/interface.py:279-813   _flash_attn_fwd  (validation, output
 *       conventions, launch on the current stream)
 *   flash_attn/cute/interface.py:785-803   the compiled-kernel call
 *       fn(q, k, v, out, lse, softmax_scale, ...)  -> fa4_nvfp4_fwd
 *   flash_attn/cute/flash_fwd_sm100.py:336-728  FlashAttentionForwardSm100.__call__
 *       (TMA descriptors, grid, shared-memory opt-in) -> done inside fa4_nvfp4_fwd
 * The reference has no NVFP4 signature (inputs are asserted fp16/bf16 at
 * interface.py:370), so the operand formats below are defined here.
 *
 * Operand formats
 *   q   (B, Sq, Hq,  D/2)  bytes, two e2m1 values per byte, low nibble = even index
 *   k   (B, Sk, Hkv, D/2)  bytes
 *   v   (B, Hkv, Dv, Skp/2) bytes: V is stored key-contiguous ("V transposed")
 *                           because 4-bit tensor-core operands must be K-major; its key axis
 *                           is padded to Skp = Sk rounded up to a multiple of 32, the padding
 *                           holds zero values and zero scales (Sk itself is free)
 *   *_sf  e4m3 (unsigned use: scales are >= 0) scale of each block of 16
 *         consecutive elements (along D for q and k, along the key axis for v),
 *         in the 128x4 TILED layout described at fa4_nvfp4_sf_linear_to_tiled
 *   q_scale, k_scale, v_scale  fp32 per-tensor scales; a value is
 *         e2m1 * e4m3_block_scale * per_tensor_scale
 *   out (B, Sq, Hq, Dv) bf16;  lse (B, Hq, Sq) fp32, natural log of the sum of
 *         exp(softmax_scale * q.k) over the visible keys, -inf for a row that
 *         sees no key (same conventions as interface.py:413-433 and
 *         flash_fwd_sm100.py:2481-2501)
 *   causal: key j visible to query i iff j <= i + Sk - Sq (bottom-right aligned,
 *         flash_attn/cute/testing.py:276)
 *   GQA: query head h reads kv head h / (Hq / Hkv)  (testing.py:362-363)
 */
#ifndef FA4_NVFP4_H_
#define FA4_NVFP4_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FA4_NVFP4_ABI_VERSION 1

/* host-side argument errors (returned negated) */
enum {
  FA4_E_NULL = 1,        /* a required pointer is NULL */
  FA4_E_SHAPE = 2,       /* unsupported shape or divisibility */
  FA4_E_STRIDE = 3,      /* stride not a multiple of 16 bytes / not contiguous where required */
  FA4_E_ALIGN = 4,       /* base pointer not 16-byte aligned */
  FA4_E_VARIANT = 5,     /* unknown kernel variant */
  FA4_E_TENSORMAP = 6,   /* the driver rejected a TMA tensor map */
  FA4_E_STRUCT = 7,      /* struct_size does not match this ABI */
  FA4_E_TOO_LARGE = 8,   /* problem exceeds a fixed capacity of the entry point */
  FA4_E_BUILD = 9        /* the library was compiled with a register count its kernels cannot run with */
};

/* device status word: 0 = ok; otherwise
 *     (code << 24) | (site << 16) | (launch epoch << 8) | (blockIdx.x & 0xff).
 * The word is sticky for REPORTING: the first failure stays until the host reads and clears it.
 * It is not sticky for EXECUTION: every launch carries an epoch (the library counts launches
 * modulo 256) and only CTAs of the launch that recorded the failure stop early, so a stale word
 * does not disturb later calls.  A launch that gave up leaves (part of) its outputs unwritten
 * and the entry point has long returned 0 by then, as with any asynchronous CUDA failure: read
 * the word wherever results are consumed on the host. */
enum {
  FA4_S_OK = 0,
  FA4_S_WAIT_EXPIRED = 1 /* a bounded mbarrier wait ran out; `site` names the wait */
};

/* kernel variants */
enum {
  FA4_VARIANT_AUTO = 0,   /* WS64 unless the call splits the keys (then WS) */
  /* 1: retired (a one-warpgroup bring-up kernel); -FA4_E_VARIANT */
  FA4_VARIANT_WS = 2,     /* warp-specialised pipeline, steps of 128 keys from the last visible
                             block down; every feature, D = 128 and 64 */
  FA4_VARIANT_WS64 = 3,   /* warp-specialised pipeline, steps of 64 keys upwards, four score
                             buffers, separate epilogue warpgroup; D = 128, 64 and (192, 128);
                             windows, sinks, the soft cap and KV-cache views, but no split-KV
                             (-FA4_E_SHAPE) */
  FA4_VARIANT_DECODE = 4  /* transposed products for a handful of query rows: keys on the tile's
                             lanes, the Sq * (Hq / Hkv) <= 32 query rows of a kv head on the N
                             side; D = Dv = 128, causal or unmasked, seqused_k / page_table allowed;
                             through fa4_nvfp4_fwd_ex with num_splits >= 1 and the split-KV
                             workspace (grid = splits x Hkv x B) */
};

typedef struct fa4_nvfp4_params {
  uint32_t struct_size;   /* = sizeof(fa4_nvfp4_params) */
  int32_t variant;        /* FA4_VARIANT_* */

  const void* q;          /* packed e2m1 */
  const void* k;
  const void* v;
  const void* q_sf;       /* e4m3, tiled: (B, Hq,  ceil(Sq/128), D/64,  512) bytes */
  const void* k_sf;       /* e4m3, tiled: (B, Hkv, ceil(Sk/128), D/64,  512) bytes */
  const void* v_sf;       /* e4m3, tiled: (B, Hkv, ceil(Dv/128), 2*ceil(Sk/128), 512) bytes (zero past Sk) */
  void* out;              /* bf16 (B, Sq, Hq, Dv) */
  float* lse;             /* fp32 (B, Hq, Sq) or NULL */
  uint32_t* status;       /* one device word, zeroed by the caller; NULL = not reported */

  /* strides in BYTES for the packed operands, in ELEMENTS for out */
  int64_t q_stride_b, q_stride_s, q_stride_h;    /* innermost (D/2 bytes) is contiguous */
  int64_t k_stride_b, k_stride_s, k_stride_h;
  int64_t v_stride_b, v_stride_h, v_stride_d;    /* innermost (Sk/2 bytes) is contiguous */
  int64_t o_stride_b, o_stride_s, o_stride_h;    /* innermost (Dv) is contiguous */

  int32_t B, Sq, Sk, Hq, Hkv, D, Dv;
  int32_t causal;
  float q_scale, k_scale, v_scale;
  float softmax_scale;
  uint64_t wait_budget_ns; /* limit of every device-side wait; 0 = default (2 s) */
} fa4_nvfp4_params;

/*
 * NVFP4 attention forward.  Replaces the compiled-kernel call of the reference
 * (flash_attn/cute/interface.py:785-803).  Asynchronous on `cuda_stream`
 * (a cudaStream_t; NULL = legacy default stream), no host synchronisation.
 * Shapes built: (D, Dv) = (128, 128), (64, 64) or (192, 128) (the reference's table is
 * flash_attn/cute/interface.py:84-99; fa4_nvfp4_query lists D), any Sq, any Sk (the reference's
 * ragged shapes, tests/cute/test_flash_attn.py:91-119; V's key axis padded as above),
 * Hq a multiple of Hkv; everything else returns -FA4_E_SHAPE.  (192, 128) runs on the 64-key
 * kernel only (no split-KV, no decode variant).
 */
int fa4_nvfp4_fwd(const fa4_nvfp4_params* p, void* cuda_stream);

/*
 * The same forward with the K/V sequence split `num_splits` ways (1..128): the reference's
 * num_splits path (flash_attn/cute/interface.py:494-510 heuristics, :804-812 combine call,
 * flash_attn/cute/flash_fwd_combine.py).  Every (query tile, split) pair becomes a work item that
 * visits a contiguous share of the tile's K/V blocks and writes a normalised fp32 partial output
 * and a partial LSE into `workspace`; a second kernel on the same stream merges them
 * (lse = log sum exp(lse_i), out = sum exp(lse_i - lse) out_i) into p->out / p->lse.  For short
 * Sq (decode) this is what fills the GPU: without it there are only B * Hq * ceil(Sq/128) work
 * items.  `workspace`: caller-owned device memory, 16-byte aligned, at least
 * fa4_nvfp4_splitkv_workspace_bytes(p, num_splits) bytes (= num_splits * B * Sq * Hq * (Dv + 1)
 * floats; 0 for num_splits = 1, in which case this is fa4_nvfp4_fwd).  Split calls run the
 * 128-key kernel (FA4_VARIANT_WS) or the decode kernel; D = 128 and 64.
 */
int64_t fa4_nvfp4_splitkv_workspace_bytes(const fa4_nvfp4_params* p, int32_t num_splits);
int fa4_nvfp4_fwd_splitkv(const fa4_nvfp4_params* p, int32_t num_splits, void* workspace,
                          uint64_t workspace_bytes, void* cuda_stream);

/*
 * Extended forward: split-KV and / or local (sliding-window) attention, the reference's
 * window_size_left / window_size_right (flash_attn/cute/interface.py:256-276,293-294; mask
 * semantics flash_attn/cute/testing.py:249-288, mask.py:487-527): query row i sees keys j with
 *     i + Sk - Sq - window_left <= j <= i + Sk - Sq + window_right,     -1 = no limit.
 * p->causal is the right limit 0 (an explicit window_right >= 0 takes its place).  Tiles skip
 * the K/V blocks that lie wholly outside the window of all their rows.  Windows, sinks, the soft
 * cap and KV-cache views run on the 64-key kernel (every head dim) when the call does not split
 * the keys, and on the 128-key kernel (D = 128, 64) when it does.
 */
typedef struct fa4_nvfp4_ext {
  uint32_t struct_size;     /* = sizeof(fa4_nvfp4_ext) */
  int32_t num_splits;       /* 0 or 1: no split; k > 1 needs the workspace of fa4_nvfp4_fwd_splitkv */
  void* workspace;
  uint64_t workspace_bytes;
  int32_t window_left;      /* -1: unlimited */
  int32_t window_right;     /* -1: unlimited (or 0 when p->causal) */
  const float* sink;        /* learnable sink: Hq fp32 logits on the device (natural-log units of the
                               scaled scores) that join every row's normalisation and LSE without a
                               value row (flash_attn/cute/flash_fwd_sm100.py:2383-2394); NULL = none */
  float softcap;            /* > 0: scores = softcap * tanh(scores / softcap) on the scaled scores
                               before masking (flash_attn/cute/interface.py:528-530,
                               testing.py:373-374), with the hardware tanh approximation; 0 = off */
  uint32_t reserved;        /* 0 */
  /* KV cache, the reference's seqused_k / page_table (flash_attn/cute/interface.py:296-300,
   * paged_kv.py): */
  const int32_t* seqused_k; /* B counts on the device: batch entry b attends to its first
                               seqused_k[b] keys (clamped to 0..Sk); causal and window limits align
                               to that length.  NULL = Sk for every entry.  Scale bytes of the
                               unused slots must not be NaN encodings (a zero-filled cache is fine) */
  const int32_t* page_table;/* (B, pages_per_seq) page numbers on the device, or NULL.  With a table
                               p->k / p->v / p->k_sf / p->v_sf describe a POOL of num_pages pages of
                               page_size keys: k (num_pages, page_size, Hkv, D/2), v (num_pages, Hkv,
                               Dv, page_size/2), tiled scales per page; k_stride_b / v_stride_b are
                               page strides; p->Sk is the logical key length, at most
                               pages_per_seq * page_size */
  int32_t page_size;        /* keys per page, a multiple of 128 */
  int32_t pages_per_seq;
  int32_t num_pages;
  int32_t reserved2;        /* 0 */
} fa4_nvfp4_ext;
int fa4_nvfp4_fwd_ex(const fa4_nvfp4_params* p, const fa4_nvfp4_ext* x, void* cuda_stream);

/*
 * Packed variable-length batches in ONE launch: the reference's flash_attn_varlen_func
 * (flash_attn/cute/interface.py:1795-1840; its persistent varlen scheduler is
 * flash_attn/cute/tile_scheduler.py:755-1087).  q, k, v, out of `p` have no batch dimension:
 *   q (total_q, Hq, D/2), k (total_k, Hkv, D/2), v (Hkv, Dv, total_kp/2) with total_kp = total_k
 *   rounded up to a multiple of 32, out (total_q, Hq, Dv), lse (Hq, total_q);
 * p->q_stride_s / q_stride_h etc. are the token and head strides (the batch strides must still be
 * positive multiples of 16 and are not used), p->B / Sq / Sk are ignored.  Sequence b owns query
 * rows cu_seqlens_q[b] .. cu_seqlens_q[b+1] and keys cu_seqlens_k[b] .. cu_seqlens_k[b+1] (device
 * arrays of num_seqs + 1 int32; no host read-back anywhere).  V is key-contiguous and blocked by 16
 * keys with 16-byte rows, so inside V (and v_sf) every sequence starts on a multiple of 32 keys:
 * cu_seqlens_v gives those starts (slot i = cu_seqlens_v[i] .. cu_seqlens_v[i+1], at least as long
 * as sequence i, a multiple of 32, its tail zero), total_v the length of V's key axis; with
 * cu_seqlens_v = NULL V uses cu_seqlens_k, whose starts must then be multiples of 32 themselves.
 * K is packed without padding in either case.  `seqused_k` (optional) gives the valid keys of
 * each slot.  The tile grid is (sequence, m-block of the LONGEST sequence, head):
 * pass max_seqlen_q / max_seqlen_k as the reference's call does; tiles past a sequence's end
 * cost a few instructions.  The tiled scale factors are per sequence, padded to the longest:
 *   q_sf (num_seqs, Hq, ceil(max_seqlen_q/128), D/64, 512), k_sf (num_seqs, Hkv,
 *   ceil(max_seqlen_k/128), D/64, 512), v_sf (num_seqs, Hkv, ceil(Dv/128),
 *   2*ceil(max_seqlen_k/128), 512): fa4_nvfp4_sf_linear_to_tiled_packed builds them from the
 * packed linear layouts.  Causal and window limits align bottom-right per sequence.  Runs the
 * 64-key kernel (no split-KV).
 */
typedef struct fa4_nvfp4_varlen {
  uint32_t struct_size;          /* = sizeof(fa4_nvfp4_varlen) */
  int32_t num_seqs;
  const int32_t* cu_seqlens_q;   /* device, num_seqs + 1 */
  const int32_t* cu_seqlens_k;   /* device, num_seqs + 1 */
  const int32_t* seqused_k;      /* device, num_seqs, or NULL */
  int32_t total_q, total_k;
  int32_t max_seqlen_q, max_seqlen_k;
  int32_t window_left, window_right;   /* -1: unlimited (right: 0 when p->causal) */
  const float* sink;             /* Hq logits or NULL */
  float softcap;                 /* 0 = off */
  uint32_t reserved;             /* 0 */
  const int32_t* cu_seqlens_v;   /* device, num_seqs + 1, multiples of 32, or NULL (= cu_seqlens_k) */
  int32_t total_v;               /* keys along V's axis (a multiple of 32); 0 with cu_seqlens_v = NULL */
  int32_t reserved2;             /* 0 */
} fa4_nvfp4_varlen;
int fa4_nvfp4_fwd_varlen(const fa4_nvfp4_params* p, const fa4_nvfp4_varlen* v, void* cuda_stream);

/*
 * Linear -> tiled scale factors of a packed batch (see fa4_nvfp4_varlen): per-sequence tiles,
 * padded with zeros to max_rows x max_cols.  packed_rows = 1: src is (total, n_inner, cols) with
 * the packed axis on the rows (q / k scales; stride_row = n_inner * cols, stride_inner = cols);
 * packed_rows = 0: src is (n_inner, rows, total / 16) with the packed axis on the columns
 * (v scales; cu_seqlens in keys -- the starts inside V, i.e. cu_seqlens_v when that is given --
 * stride_inner = rows * row length, stride_row = row length).
 * No counterpart in the reference (it has no scale factors).
 */
int fa4_nvfp4_sf_linear_to_tiled_packed(const void* src, void* dst, const int32_t* cu_seqlens,
                                        int32_t num_seqs, int32_t n_inner, int32_t max_rows,
                                        int32_t max_cols, int64_t stride_inner, int64_t stride_row,
                                        int32_t col_tile_multiple, int32_t packed_rows,
                                        void* cuda_stream);

/*
 * Scale-factor layout conversion, linear -> tiled.
 *   src: rows x cols e4m3 bytes; element (r, c) of matrix m at
 *        src + m_outer*stride_outer + m_inner*stride_inner + r*stride_row + c
 *        (n_outer x n_inner matrices; for q_sf given as (B, S, H, D/16):
 *        outer = batch, inner = head, stride_row = H*D/16)
 *   dst: (n_outer, n_inner, ceil(rows/128), CT, 512) bytes, CT = ceil(cols/4) rounded up to a
 *        multiple of col_tile_multiple (1 for q_sf / k_sf; 2 for v_sf, whose 128-key blocks
 *        are read as two 64-key column tiles even when the last block is partial); inside a
 *        512-byte tile the scale of row r, column c sits at
 *        (r % 32) * 16 + (r / 32) * 4 + c   -- the 32x4x4 chunk that one
 *        `tcgen05.cp 32x128b.warpx4` moves to tensor memory.  Padding rows and
 *        columns are written as zero.
 * The reference has no scale-factor operand at all; this layout is the one the
 * block-scaled tensor-core instruction consumes (flash_attn/cute/mma_sm100_desc.py
 * documents only the non-scaled kinds).
 */
int fa4_nvfp4_sf_linear_to_tiled(const void* src, void* dst,
                                 int32_t n_outer, int32_t n_inner,
                                 int32_t rows, int32_t cols,
                                 int64_t stride_outer, int64_t stride_inner,
                                 int64_t stride_row, int32_t col_tile_multiple,
                                 void* cuda_stream);

/*
 * Version / capability query (host only, never touches a GPU).
 *   what = 0: ABI version; 1: number of supported head dims; 2+i: i-th supported
 *   head dim; 100: default dynamic shared memory per CTA of the WS variant; 101: which of the 8
 *   pairs of a 16-key block take the FMA-pipe exp2 in this build (bit mask, 0 = none; the
 *   compile-time knob that corresponds to the reference's ex2_emu_freq,
 *   flash_attn/cute/flash_fwd_sm100.py:71-90).
 * Mirrors the head-dim validation of flash_attn/cute/interface.py:84-99.
 */
int fa4_nvfp4_query(int32_t what);

/*
 * Fused NVFP4 quantiser: bf16 operands in the reference's layout ((batch, seqlen, heads,
 * head_dim), flash_attn/cute/interface.py:227-228, last dimension contiguous, strides in
 * ELEMENTS and multiples of 8) -> the operands of fa4_nvfp4_fwd.  No counterpart in the
 * reference, which takes fp16/bf16 only (interface.py:370); this is the step a caller runs
 * directly before the forward.  Arithmetic, every step a correctly rounded fp32 operation:
 *     tensor scale = amax / (6 * 448)               (1 for an all-zero tensor)
 *     block scale  = e4m3_rne(min(block_amax / 6 / tensor scale, 448))   per 16 elements
 *     element      = e2m1_rne(x / (block scale * tensor scale)), never negative zero
 *
 * fa4_nvfp4_amax_bf16: *amax = max(*amax, max |x|) over an (n0, n1, n2, inner) tensor; the
 *     caller zeroes *amax (device memory) first.  inner % 8 == 0.
 * fa4_nvfp4_quantize_qk_bf16: x (B, S, H, D), blocks along D (D % 64 == 0).  Writes
 *     packed (B, S, H, D/2); sf_linear (B, S, H, D/16) and / or sf_tiled
 *     (B, H, ceil(S/128), D/64, 512), either may be NULL; *scale_out (device, may be NULL)
 *     receives the tensor scale.  `amax` is device memory (the result of the call above, or any
 *     caller-chosen value: the tensor scale is derived from it).
 * fa4_nvfp4_quantize_v_bf16: x (B, Sk, H, Dv), blocks along the KEY axis (Sk % 16 == 0,
 *     Dv % 8 == 0, B * H <= 65535).  Writes packed (B, H, Dv, Sk/2) -- V key-contiguous --,
 *     sf_linear (B, H, Dv, Sk/16) and / or sf_tiled (B, H, ceil(Dv/128), 2*ceil(Sk/128), 512).
 * All outputs are fully contiguous and 16-byte aligned; nothing is allocated; the kernels run on
 * `cuda_stream` in call order.
 */
int fa4_nvfp4_amax_bf16(const void* x, int64_t n0, int32_t n1, int32_t n2, int32_t inner,
                        int64_t s0, int64_t s1, int64_t s2, float* amax, void* cuda_stream);
int fa4_nvfp4_quantize_qk_bf16(const void* x, int32_t B, int32_t S, int32_t H, int32_t D,
                               int64_t stride_b, int64_t stride_s, int64_t stride_h,
                               const float* amax, void* packed, void* sf_linear, void* sf_tiled,
                               float* scale_out, void* cuda_stream);
int fa4_nvfp4_quantize_v_bf16(const void* x, int32_t B, int32_t Sk, int32_t H, int32_t Dv,
                              int64_t stride_b, int64_t stride_s, int64_t stride_h,
                              const float* amax, void* packed, void* sf_linear, void* sf_tiled,
                              float* scale_out, void* cuda_stream);

/*
 * Hardware-contract probe: one 128x128xD block-scaled tile S = A * B^T with
 * A = q tile, B = k tile (same operand formats as above, one head, one batch,
 * Sq = Sk = 128), written as fp32 (128,128) to `s_out`.  `mode` bit 0: stage the
 * operands with plain shared-memory stores instead of TMA.  Used by the GPU
 * tests to pin the descriptor and scale-factor layouts; no counterpart in the
 * reference (its tests never look inside a tile).
 */
int fa4_nvfp4_debug_qk_tile(const void* q, const void* k, const void* q_sf,
                            const void* k_sf, float* s_out, int32_t D,
                            int32_t mode, uint32_t* status, void* cuda_stream);

/*
 * Tensor-pipe rate probe: `num_ctas` CTAs (one per SM when num_ctas = SM count) each issue
 * `iters` (a multiple of 4) block-scaled 128x128x64 e2m1 MMAs back to back on operands that
 * stay in shared memory, and write the clocks from first issue to last completion to
 * clocks_out[cta] (device memory, num_ctas entries).  The caller times the launch; FLOPs =
 * num_ctas * iters * 2 * 128 * 128 * 64.  This is the measured dense-FP4 ceiling the benchmark
 * reports beside the nominal one; no counterpart in the reference (its benchmark hard-codes a
 * nominal peak, benchmarks/benchmark_attn.py:200).
 */
int fa4_nvfp4_debug_mma_rate(int32_t iters, int32_t num_ctas, uint64_t* clocks_out,
                             uint32_t* status, void* cuda_stream);

/*
 * Exponential-unit rate probe: `num_ctas` CTAs of 512 threads each run `iters` rounds of 16
 * independent ex2.approx per thread and write their clocks to clocks_out[cta]; exp2 per clock per
 * SM = 512 * iters * 16 / clocks.  `scratch`: one float of device memory (never written in
 * practice).  The denominator of the benchmark's exponential roofline (one exp2 per score); the
 * reference's tuning script states the same limit in words (benchmarks/tune_ex2_emu.py:1-30) and
 * has no probe.
 */
int fa4_nvfp4_debug_ex2_rate(int32_t iters, int32_t num_ctas, uint64_t* clocks_out, float* scratch,
                             void* cuda_stream);

/*
 * Bounded-wait self test: launches one CTA that waits on a barrier nothing
 * arrives at, with a limit of `budget_ns`; the kernel must give up, record
 * FA4_S_WAIT_EXPIRED in *status and return normally.  No counterpart in the
 * reference, whose device waits are unbounded (flash_attn/cute/blackwell_helpers.py:519-526).
 */
int fa4_nvfp4_debug_wait_expiry(uint32_t* status, uint64_t budget_ns, void* cuda_stream);

/*
 * Forward from LINEAR scale factors for hosts that cannot allocate device memory.
 * No counterpart in the reference (which allocates its outputs with torch and has no scale
 * factors at all).
 *
 * Same contract as fa4_nvfp4_fwd except that p->q_sf, p->k_sf, p->v_sf are the linear, fully
 * contiguous layouts (B, Sq, Hq, D/16), (B, Sk, Hkv, D/16), (B, Hkv, Dv, Skp/16), Skp = Sk rounded up
 * to a multiple of 32.  The tiled copies
 * the kernel reads are staged in a fixed 16 MiB array that is part of the library image on every
 * GPU the library is loaded on (FA4_NVFP4_STATIC_SCRATCH_BYTES), so the call performs no
 * cudaMalloc / cudaFree and needs no workspace argument.  Meant for callers whose device memory
 * is entirely owned by their own arena, or whose steady-state loop must not call the allocator.
 *
 * Limits and rules:
 *  - the three tiled scale-factor tensors together must fit: sum over q, k, v of
 *    matrices * ceil(rows/128) * column tiles * 512 bytes <= 16 MiB, else -FA4_E_TOO_LARGE
 *    (B=4, Hq=32, Hkv=8, S=8192, D=128 needs 12 MiB);
 *  - the call is validated exactly like fa4_nvfp4_fwd BEFORE anything is launched: a negative
 *    return means no kernel ran and the array was not touched.  FA4_VARIANT_DECODE is refused
 *    (it needs a caller-owned workspace);
 *  - every call asks the runtime for the array's device address on the current device
 *    (cudaGetSymbolAddress; no pointer is kept across calls, so a cudaDeviceReset in between is
 *    harmless).  The first call on a device also loads the library image there: make that first
 *    call outside any stream capture;
 *  - all calls on a device share the one array, and it keeps whatever the previous call left
 *    there.  Each call rewrites every byte it later reads (padding included), so nothing has to
 *    be cleared, but two calls that overlap on the GPU (different streams without an ordering
 *    between them) race on it: serialise them.
 */
#define FA4_NVFP4_STATIC_SCRATCH_BYTES (16u << 20)
int fa4_nvfp4_fwd_linear_sf_noalloc(const fa4_nvfp4_params* p, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* FA4_NVFP4_H_ */
