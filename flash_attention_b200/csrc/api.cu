// C ABI of the NVFP4 attention forward (see include/fa4_nvfp4.h): argument validation, TMA
// tensor maps, launch configuration.  Host code only; the kernels live in the .cuh files.
#include "../../include/fa4_nvfp4.h"

#include "attn_common.cuh"
#include "attn_ws.cuh"
#include "attn_ws64.cuh"
#include "attn_decode.cuh"
#include "aux_kernels.cuh"
#include "quantize.cuh"

#include <cudaTypedefs.h>
#include <atomic>
#include <map>
#include <mutex>
#include <utility>

namespace {

using namespace fa4;

constexpr uint64_t kDefaultBudgetNs = 2000ull * 1000 * 1000;

PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    }
  });
  return fn;
}

// Byte tensor of rank 4, innermost dimension contiguous; box = {box0, box1, box2, box3} bytes /
// rows; 64-byte swizzle when the innermost box is 64 bytes.
// bf16 output tensor (B, Sq, Hq, Dv) as {Dv, Hq, Sq, B}; box = 64 columns x 128 rows, 128-byte
// swizzle (the staging layout of the warp-specialised kernel's epilogue).
bool encode_out_4d(CUtensorMap* m, void* base, const uint64_t (&dims)[4], const uint64_t (&strides)[3]) {
  auto fn = get_encode();
  if (fn == nullptr) return false;
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const cuuint32_t box[4] = {64, 1, 128, 1};
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool encode_u8_4d(CUtensorMap* m, const void* base, const uint64_t (&dims)[4],
                  const uint64_t (&strides)[3], const uint32_t (&box)[4], CUtensorMapSwizzle sw) {
  auto fn = get_encode();
  if (fn == nullptr) return false;
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Launch epoch recorded with a device-side failure (see ptx.cuh): launches modulo 256.
uint32_t next_launch_epoch() {
  static std::atomic<uint32_t> counter{0};
  return counter.fetch_add(1, std::memory_order_relaxed) & 0xffu;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Per-kernel launch preparation, done once per (kernel, device) and remembered: the opt-in to
// `smem_bytes` of dynamic shared memory and -- for the warp-specialised kernels, which re-partition
// registers with setmaxnreg -- the check that the build kept the register count the budget in the
// source assumes (an increase blocks for ever when the CTA was launched with fewer registers per
// thread; such a build is refused with -FA4_E_BUILD instead of being launched).
// expected_regs = 0: no register check.
int prepare_kernel(const void* kernel, uint32_t smem_bytes, int expected_regs) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, int> seen;   // -> result of the first preparation
  int dev = 0;
  const cudaError_t ge = cudaGetDevice(&dev);
  if (ge != cudaSuccess) return (int)ge;
  std::lock_guard<std::mutex> lock(mu);
  const auto key = std::make_pair(kernel, dev);
  const auto it = seen.find(key);
  if (it != seen.end()) return it->second;
  int rc = 0;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
  if (e != cudaSuccess) return (int)e;          // not remembered: the caller may retry
  if (expected_regs > 0) {
    cudaFuncAttributes attr;
    e = cudaFuncGetAttributes(&attr, kernel);
    if (e != cudaSuccess) return (int)e;
    if (attr.numRegs < expected_regs) rc = -FA4_E_BUILD;
  }
  seen[key] = rc;
  return rc;
}
template <class Kernel>
int ensure_smem(Kernel kernel, uint32_t bytes) {
  return prepare_kernel(reinterpret_cast<const void*>(kernel), bytes, 0);
}
template <class Kernel>
int ensure_kernel(Kernel kernel, uint32_t bytes, int expected_regs) {
  return prepare_kernel(reinterpret_cast<const void*>(kernel), bytes, expected_regs);
}

}  // namespace

extern "C" int fa4_nvfp4_query(int32_t what) {
  static const int dims[] = {128, 64, 192};   // 192 pairs with a V / O head dim of 128
  switch (what) {
    case 0: return FA4_NVFP4_ABI_VERSION;
    case 1: return (int)(sizeof(dims) / sizeof(dims[0]));
    case 100: return (int)fa4::ws::kSmemRequest;
    case 101: return (int)fa4::kEx2EmuMask;
    case 102: return FA4_P_SCALE_E4M3;
    default:
      if (what >= 2 && what < 2 + (int)(sizeof(dims) / sizeof(dims[0]))) return dims[what - 2];
      return -FA4_E_SHAPE;
  }
}

namespace {
int64_t splitkv_bytes(const fa4_nvfp4_params* p, int num_splits) {
  // partial O (num_splits, B, Sq, Hq, Dv) fp32, then partial LSE (num_splits, B, Hq, Sq) fp32
  return (int64_t)num_splits * p->B * p->Sq * p->Hq * ((int64_t)p->Dv + 1) * 4;
}
// KV-cache view of K / V: per-entry key counts and / or a page pool (see fa4_nvfp4_ext).
struct CacheView {
  const int32_t* seqused_k = nullptr;
  const int32_t* page_table = nullptr;
  int page_size = 0, pages_per_seq = 0, num_pages = 0;
  // packed variable-length batch (see fa4_nvfp4_varlen)
  const int32_t* cu_seqlens_q = nullptr;
  const int32_t* cu_seqlens_k = nullptr;
  const int32_t* cu_seqlens_v = nullptr;   // starts inside V (multiples of 32); null: cu_seqlens_k
  int total_q = 0, total_k = 0, total_v = 0;
};
int launch_fwd(const fa4_nvfp4_params* p, int num_splits, void* workspace, uint64_t workspace_bytes,
               int win_left, int win_right, const float* sink, float softcap, const CacheView& cache,
               void* cuda_stream);
}  // namespace

extern "C" int fa4_nvfp4_fwd(const fa4_nvfp4_params* p, void* cuda_stream) {
  return launch_fwd(p, 1, nullptr, 0, -1, -1, nullptr, 0.f, CacheView{}, cuda_stream);
}

extern "C" int fa4_nvfp4_fwd_ex(const fa4_nvfp4_params* p, const fa4_nvfp4_ext* x, void* cuda_stream) {
  if (x == nullptr) return -FA4_E_NULL;
  if (x->struct_size != sizeof(fa4_nvfp4_ext)) return -FA4_E_STRUCT;
  const int splits = x->num_splits == 0 ? 1 : x->num_splits;
  if (splits < 1 || splits > 128 || x->window_left < -1 || x->window_right < -1) return -FA4_E_SHAPE;
  if (!(x->softcap >= 0.f) || x->softcap > 3.0e38f || x->reserved != 0u) return -FA4_E_SHAPE;
  CacheView cache;
  cache.seqused_k = x->seqused_k;
  if (x->page_table != nullptr) {
    // pages hold whole 128-key blocks; the table must cover the logical key length
    if (x->page_size <= 0 || x->page_size % 128 != 0 || x->num_pages <= 0 || x->pages_per_seq <= 0)
      return -FA4_E_SHAPE;
    if (p != nullptr && (int64_t)x->pages_per_seq * x->page_size < p->Sk) return -FA4_E_SHAPE;
    cache.page_table = x->page_table;
    cache.page_size = x->page_size;
    cache.pages_per_seq = x->pages_per_seq;
    cache.num_pages = x->num_pages;
  }
  return launch_fwd(p, splits, x->workspace, x->workspace_bytes, x->window_left, x->window_right,
                    x->sink, x->softcap, cache, cuda_stream);
}

extern "C" int fa4_nvfp4_fwd_varlen(const fa4_nvfp4_params* p, const fa4_nvfp4_varlen* v, void* cuda_stream) {
  if (p == nullptr || v == nullptr) return -FA4_E_NULL;
  if (v->struct_size != sizeof(fa4_nvfp4_varlen) || p->struct_size != sizeof(fa4_nvfp4_params)) return -FA4_E_STRUCT;
  if (v->cu_seqlens_q == nullptr || v->cu_seqlens_k == nullptr) return -FA4_E_NULL;
  if (v->num_seqs <= 0 || v->total_q <= 0 || v->total_k <= 0 || v->max_seqlen_q <= 0 || v->max_seqlen_k <= 0 ||
      v->max_seqlen_q > v->total_q || v->max_seqlen_k > v->total_k)
    return -FA4_E_SHAPE;
  if (v->window_left < -1 || v->window_right < -1 || !(v->softcap >= 0.f) || v->softcap > 3.0e38f || v->reserved != 0u ||
      v->reserved2 != 0)
    return -FA4_E_SHAPE;
  if (v->cu_seqlens_v != nullptr ? (v->total_v < v->total_k || v->total_v % 32 != 0) : v->total_v != 0)
    return -FA4_E_SHAPE;
  if (p->variant != FA4_VARIANT_AUTO && p->variant != FA4_VARIANT_WS64) return -FA4_E_VARIANT;
  // one launch over (sequence, m-block of the longest sequence, head): the grid of the dense call
  // with B = number of sequences and Sq / Sk = the longest ones
  fa4_nvfp4_params q = *p;
  q.B = v->num_seqs;
  q.Sq = v->max_seqlen_q;
  q.Sk = v->max_seqlen_k;
  q.variant = FA4_VARIANT_WS64;
  CacheView cache;
  cache.seqused_k = v->seqused_k;
  cache.cu_seqlens_q = v->cu_seqlens_q;
  cache.cu_seqlens_k = v->cu_seqlens_k;
  cache.total_q = v->total_q;
  cache.total_k = v->total_k;
  cache.cu_seqlens_v = v->cu_seqlens_v;
  cache.total_v = v->cu_seqlens_v != nullptr ? v->total_v : v->total_k;
  return launch_fwd(&q, 1, nullptr, 0, v->window_left, v->window_right, v->sink, v->softcap, cache, cuda_stream);
}

extern "C" int fa4_nvfp4_sf_linear_to_tiled_packed(const void* src, void* dst, const int32_t* cu_seqlens,
                                                   int32_t num_seqs, int32_t n_inner, int32_t max_rows,
                                                   int32_t max_cols, int64_t stride_inner, int64_t stride_row,
                                                   int32_t col_tile_multiple, int32_t packed_rows,
                                                   void* cuda_stream) {
  if (!src || !dst || !cu_seqlens) return -FA4_E_NULL;
  if (num_seqs <= 0 || n_inner <= 0 || max_rows <= 0 || max_cols <= 0 || col_tile_multiple <= 0)
    return -FA4_E_SHAPE;
  if (!aligned16(dst)) return -FA4_E_ALIGN;
  const int64_t ct = ((max_cols + 3) / 4 + col_tile_multiple - 1) / col_tile_multiple * col_tile_multiple;
  const int64_t total = (int64_t)num_seqs * n_inner * ((max_rows + 127) / 128) * ct * 32;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = 148 * 16;
  if (blocks > cap) blocks = cap;
  sf_linear_to_tiled_packed_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), cu_seqlens, num_seqs, n_inner, max_rows,
      max_cols, stride_inner, stride_row, col_tile_multiple, packed_rows ? 1 : 0);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int64_t fa4_nvfp4_splitkv_workspace_bytes(const fa4_nvfp4_params* p, int32_t num_splits) {
  if (p == nullptr || p->struct_size != sizeof(fa4_nvfp4_params)) return -FA4_E_STRUCT;
  if (num_splits < 1 || num_splits > 128 || p->B <= 0 || p->Sq <= 0 || p->Hq <= 0 || p->Dv <= 0)
    return -FA4_E_SHAPE;
  return num_splits == 1 ? 0 : splitkv_bytes(p, num_splits);
}

extern "C" int fa4_nvfp4_fwd_splitkv(const fa4_nvfp4_params* p, int32_t num_splits, void* workspace,
                                     uint64_t workspace_bytes, void* cuda_stream) {
  if (num_splits < 1 || num_splits > 128) return -FA4_E_SHAPE;
  return launch_fwd(p, num_splits, workspace, workspace_bytes, -1, -1, nullptr, 0.f, CacheView{}, cuda_stream);
}

namespace {
// What a call resolves to once its arguments have been accepted.
struct FwdPlan {
  int variant = 0;
  int win_left = -1, win_right = -1;
  bool decode = false, d192 = false, local = false, general = false, cached = false;
  int dec_rows = 0;
};

// Every host-side check of a forward call.  Touches no CUDA API: a call that fails here has
// launched nothing and has not made a device current.  `linear_sf`: the three scale pointers are
// the caller's LINEAR layouts (the allocation-free entry point), which need no 16-byte alignment.
int validate_fwd(const fa4_nvfp4_params* p, int num_splits, const void* workspace, uint64_t workspace_bytes,
                 int win_left, int win_right, const float* sink, float softcap, const CacheView& cache,
                 bool linear_sf, FwdPlan* plan) {
  if (p == nullptr) return -FA4_E_NULL;
  if (p->struct_size != sizeof(fa4_nvfp4_params)) return -FA4_E_STRUCT;
  if (!p->q || !p->k || !p->v || !p->q_sf || !p->k_sf || !p->v_sf || !p->out) return -FA4_E_NULL;
  if (p->B <= 0 || p->Sq <= 0 || p->Sk <= 0 || p->Hq <= 0 || p->Hkv <= 0) return -FA4_E_SHAPE;
  if (p->Hq % p->Hkv != 0) return -FA4_E_SHAPE;
  // head dims built: (128, 128), (64, 64) and (192, 128), the last on the 64-key kernel only
  const bool d192 = p->D == 192 && p->Dv == 128;
  if (!d192 && (p->D != p->Dv || (p->D != 128 && p->D != 64))) return -FA4_E_SHAPE;
  // Sq and Sk are free.  V is stored key-contiguous with its key axis padded to a multiple of 32
  // (zero values, zero scales): keys are blocked by 16 along that axis and the 16-byte stride rule
  // of TMA (checked below) needs whole 32-key groups per row; keys >= Sk are masked
  if ((int64_t)((p->Sq + kBlockM - 1) / kBlockM) * p->Hq * p->B > 0x7fffffffLL) return -FA4_E_SHAPE;
  if (!(p->softmax_scale > 0.f) || !(p->q_scale > 0.f) || !(p->k_scale > 0.f)) return -FA4_E_SHAPE;
  const void* ptrs[] = {p->q, p->k, p->v, p->out};
  for (const void* q : ptrs)
    if (!aligned16(q)) return -FA4_E_ALIGN;
  if (!linear_sf && (!aligned16(p->q_sf) || !aligned16(p->k_sf) || !aligned16(p->v_sf))) return -FA4_E_ALIGN;
  const int64_t bstr[] = {p->q_stride_b, p->q_stride_s, p->q_stride_h, p->k_stride_b, p->k_stride_s,
                          p->k_stride_h, p->v_stride_b, p->v_stride_h, p->v_stride_d};
  for (int64_t s : bstr)
    if (s <= 0 || (s & 15) != 0) return -FA4_E_STRIDE;
  if ((p->o_stride_b & 7) || (p->o_stride_s & 7) || (p->o_stride_h & 7)) return -FA4_E_STRIDE;
  // automatic choice: the 64-key kernel where it applies (no split-KV), the 128-key kernel
  // otherwise
  const bool cached = cache.seqused_k != nullptr || cache.page_table != nullptr || cache.cu_seqlens_q != nullptr;
  const bool takes64 = num_splits == 1;   // what the 64-key kernel can run
  int variant = p->variant;
  if (variant == FA4_VARIANT_AUTO) variant = takes64 ? FA4_VARIANT_WS64 : FA4_VARIANT_WS;
  if (variant != FA4_VARIANT_WS && variant != FA4_VARIANT_WS64 && variant != FA4_VARIANT_DECODE)
    return -FA4_E_VARIANT;
  const bool decode = variant == FA4_VARIANT_DECODE;
  if (decode) {
    // a handful of query rows per kv head, head dim 128, causal or unmasked; always through the
    // partial-output workspace and the combine kernel
    if (p->D != 128 || p->Dv != 128 || (int64_t)p->Sq * (p->Hq / p->Hkv) > dec::kMaxRows) return -FA4_E_SHAPE;
    if (win_left >= 0 || win_right > 0 || sink != nullptr || softcap > 0.f) return -FA4_E_SHAPE;
    if (workspace == nullptr || !aligned16(workspace)) return -FA4_E_NULL;
    if (workspace_bytes < (uint64_t)splitkv_bytes(p, num_splits)) return -FA4_E_TOO_LARGE;
  }
  if (variant == FA4_VARIANT_WS64 && !takes64) return -FA4_E_SHAPE;
  if (d192 && variant != FA4_VARIANT_WS64) return -FA4_E_SHAPE;
  // window limits: `causal` is the right limit 0; an explicit right limit overrides it
  if (p->causal && win_right < 0) win_right = 0;
  const bool local = win_left >= 0 || win_right > 0;
  if (num_splits > 1) {
    if (workspace == nullptr) return -FA4_E_NULL;
    if (!aligned16(workspace)) return -FA4_E_ALIGN;
    if (workspace_bytes < (uint64_t)splitkv_bytes(p, num_splits)) return -FA4_E_TOO_LARGE;
    if ((int64_t)((p->Sq + kBlockM - 1) / kBlockM) * p->Hq * p->B * num_splits > 0x7fffffffLL)
      return -FA4_E_SHAPE;
  }
  plan->variant = variant;
  plan->win_left = win_left;
  plan->win_right = win_right;
  plan->decode = decode;
  plan->d192 = d192;
  plan->local = local;
  plan->cached = cached;
  plan->general = local || num_splits > 1 || sink != nullptr || softcap > 0.f || cached;
  plan->dec_rows = p->Sq * (p->Hq / p->Hkv);
  return 0;
}

int launch_fwd(const fa4_nvfp4_params* p, int num_splits, void* workspace, uint64_t workspace_bytes,
               int win_left, int win_right, const float* sink, float softcap, const CacheView& cache,
               void* cuda_stream) {
  FwdPlan plan;
  if (int e = validate_fwd(p, num_splits, workspace, workspace_bytes, win_left, win_right, sink, softcap, cache,
                           false, &plan))
    return e;
  const int variant = plan.variant;
  const bool decode = plan.decode, local = plan.local, general = plan.general, cached = plan.cached;
  const int dec_rows = plan.dec_rows;
  win_left = plan.win_left;
  win_right = plan.win_right;

  CUtensorMap tm_q, tm_k, tm_v;
  {
    // a packed batch is one long sequence for the tensor maps: the kernel adds each sequence's
    // first row to the row coordinate
    const bool packed = cache.cu_seqlens_q != nullptr;
    const uint64_t dq[4] = {(uint64_t)p->D / 2, (uint64_t)p->Hq, packed ? (uint64_t)cache.total_q : (uint64_t)p->Sq,
                            packed ? 1u : (uint64_t)p->B};
    const uint64_t sq[3] = {(uint64_t)p->q_stride_h, (uint64_t)p->q_stride_s, (uint64_t)p->q_stride_b};
    // a Q / K tile row is D / 2 bytes: one 64-byte-swizzled box for D = 128; 32-byte-wide boxes
    // (32-byte swizzle), one per 64-element step, for D = 64 and 192
    const uint32_t qk_box = p->D == 128 ? 64u : 32u;
    const uint32_t bq[4] = {qk_box, 1, (uint32_t)kBlockM, 1};
    // with a page table K / V describe the pool: "batch" = page, "Sk" = keys per page
    const uint64_t k_rows = cache.page_table ? (uint64_t)cache.page_size
                                             : (packed ? (uint64_t)cache.total_k : (uint64_t)p->Sk);
    const uint64_t k_batch = cache.page_table ? (uint64_t)cache.num_pages : (packed ? 1u : (uint64_t)p->B);
    const uint64_t dk[4] = {(uint64_t)p->D / 2, (uint64_t)p->Hkv, k_rows, k_batch};
    const uint64_t sk[3] = {(uint64_t)p->k_stride_h, (uint64_t)p->k_stride_s, (uint64_t)p->k_stride_b};
    const uint32_t bk[4] = {qk_box, 1, (uint32_t)kBlockN, 1};
    const uint64_t v_keys = packed ? (uint64_t)cache.total_v : k_rows;   // a packed V has its own, padded key axis
    const uint64_t dv[4] = {(v_keys + 31) / 32 * 16, (uint64_t)p->Dv, (uint64_t)p->Hkv, k_batch};   // padded key axis
    const uint64_t sv[3] = {(uint64_t)p->v_stride_d, (uint64_t)p->v_stride_h, (uint64_t)p->v_stride_b};
    const uint32_t bv[4] = {64, (uint32_t)p->Dv, 1, 1};
    // a Q / K tile row is D / 2 bytes: 64-byte swizzle for D = 128, 32-byte for D = 64
    const CUtensorMapSwizzle sw_qk = p->D == 128 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
    if (!encode_u8_4d(&tm_q, p->q, dq, sq, bq, sw_qk) ||
        !encode_u8_4d(&tm_k, p->k, dk, sk, bk, sw_qk) ||
        !encode_u8_4d(&tm_v, p->v, dv, sv, bv, CU_TENSOR_MAP_SWIZZLE_64B))
      return -FA4_E_TENSORMAP;
  }

  KernelParams kp;
  kp.q_sf = static_cast<const uint8_t*>(p->q_sf);
  kp.k_sf = static_cast<const uint8_t*>(p->k_sf);
  kp.v_sf = static_cast<const uint8_t*>(p->v_sf);
  kp.out = static_cast<__nv_bfloat16*>(p->out);
  kp.lse = p->lse;
  kp.status = p->status;
  kp.epoch = next_launch_epoch();
  kp.o_stride_b = p->o_stride_b;
  kp.o_stride_s = p->o_stride_s;
  kp.o_stride_h = p->o_stride_h;
  kp.B = p->B; kp.Sq = p->Sq; kp.Sk = p->Sk; kp.Hq = p->Hq; kp.Hkv = p->Hkv;
  kp.group = p->Hq / p->Hkv;
  kp.div_tiles_per_m = make_fastdiv((uint32_t)p->Hq * (uint32_t)p->B);
  kp.div_hq = make_fastdiv((uint32_t)p->Hq);
  kp.div_group = make_fastdiv((uint32_t)kp.group);
  kp.div_splits = make_fastdiv((uint32_t)num_splits);
  kp.num_m_blocks = (p->Sq + kBlockM - 1) / kBlockM;
  kp.num_n_blocks = (p->Sk + kBlockN - 1) / kBlockN;
  kp.causal = win_right >= 0 ? 1 : 0;
  kp.win_left = win_left;
  kp.win_right = win_right;
  kp.sink = sink;
  // tiled scale factors: (B, H, row tiles, col tiles, 512)
  kp.qsf_stride_h = (int64_t)kp.num_m_blocks * (p->D / 64) * 512;
  kp.qsf_stride_b = kp.qsf_stride_h * p->Hq;
  // (per page when K / V are a page pool: the tiled scales of a page are laid out like those of
  // a batch entry of page_size keys)
  const int64_t kv_blocks = cache.page_table ? cache.page_size / kBlockN : kp.num_n_blocks;
  kp.ksf_stride_h = kv_blocks * (p->D / 64) * 512;
  kp.ksf_stride_b = kp.ksf_stride_h * p->Hkv;
  // V scales: two 64-key column tiles per 128-key block, the last block padded with zeros
  kp.vsf_stride_h = (int64_t)((p->Dv + 127) / 128) * (2 * kv_blocks) * 512;
  kp.vsf_stride_b = kp.vsf_stride_h * p->Hkv;
  kp.seqused_k = cache.seqused_k;
  kp.page_table = cache.page_table;
  kp.page_size = cache.page_size;
  kp.pages_per_seq = cache.pages_per_seq;
  kp.cu_seqlens_q = cache.cu_seqlens_q;
  kp.cu_seqlens_k = cache.cu_seqlens_k;
  kp.cu_seqlens_v = cache.cu_seqlens_v;
  kp.total_q = cache.total_q;
  kp.sl2 = p->softmax_scale * p->q_scale * p->k_scale * 1.4426950408889634f;
  kp.softcap_c1 = 0.f;
  if (softcap > 0.f) {
    // the kernel caps the raw products and then works in units of softcap * log2(e)
    kp.softcap_c1 = p->softmax_scale * p->q_scale * p->k_scale / softcap;
    kp.sl2 = softcap * 1.4426950408889634f;
  }
  kp.out_scale = p->v_scale;
  kp.budget_ns = p->wait_budget_ns ? p->wait_budget_ns : kDefaultBudgetNs;
  kp.num_splits = num_splits;
  kp.Dv = p->Dv;
  kp.o_partial = static_cast<float*>(workspace);
  kp.lse_partial = (num_splits > 1 || decode)
                       ? kp.o_partial + (int64_t)num_splits * p->B * p->Sq * p->Hq * p->Dv
                       : nullptr;

  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  const unsigned tiles = (unsigned)(kp.num_m_blocks * p->Hq * p->B * num_splits);
  if (decode) {
    DecodeParams dp;
    dp.q = static_cast<const uint8_t*>(p->q);
    dp.q_sf = kp.q_sf;
    dp.q_stride_b = p->q_stride_b;
    dp.q_stride_s = p->q_stride_s;
    dp.q_stride_h = p->q_stride_h;
    dp.num_splits = num_splits;
    dp.o_partial = kp.o_partial;
    dp.lse_partial = kp.lse_partial;
    auto launch_dec = [&](auto kernel, uint32_t smem) -> int {
      if (int e = ensure_smem(kernel, smem)) return e;
      kernel<<<dim3((unsigned)num_splits, (unsigned)p->Hkv, (unsigned)p->B), dec::kThreads, smem, stream>>>(
          tm_k, tm_v, kp, dp);
      return 0;
    };
    const int rc = dec_rows <= 4    ? launch_dec(attn_decode_kernel<4>, dec::kSmemRequest)
                   : dec_rows <= 8  ? launch_dec(attn_decode_kernel<8>, dec::kSmemRequest)
                   : dec_rows <= 16 ? launch_dec(attn_decode_kernel<16>, dec::kSmemRequest)
                                    : launch_dec(attn_decode_kernel<32>, dec::kSmemRequestWide);
    if (rc != 0) return rc;
  } else {
    // persistent: one CTA per SM walks the tile list
    int dev = 0, sms = 0;
    cudaError_t ce = cudaGetDevice(&dev);
    if (ce == cudaSuccess) ce = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (ce != cudaSuccess) return (int)ce;
    const unsigned grid = tiles < (unsigned)sms ? tiles : (unsigned)sms;
    CUtensorMap tm_o;
    {
      const bool packed = cache.cu_seqlens_q != nullptr;
      const uint64_t d_o[4] = {(uint64_t)p->Dv, (uint64_t)p->Hq, packed ? (uint64_t)cache.total_q : (uint64_t)p->Sq,
                               packed ? 1u : (uint64_t)p->B};
      const uint64_t s_o[3] = {(uint64_t)p->o_stride_h * 2, (uint64_t)p->o_stride_s * 2,
                               (uint64_t)p->o_stride_b * 2};
      if (!encode_out_4d(&tm_o, p->out, d_o, s_o)) return -FA4_E_TENSORMAP;
    }
    auto launch = [&](auto kernel) -> int {
      if (int e = ensure_kernel(kernel, ws::kSmemRequest, ws::kRegsLaunch)) return e;
      kernel<<<grid, ws::kThreads, ws::kSmemRequest, stream>>>(tm_q, tm_k, tm_v, tm_o, kp);
      return 0;
    };
    int rc;
    if (variant == FA4_VARIANT_WS64) {
      auto launch64 = [&](auto kernel) -> int {
        if (int e = ensure_kernel(kernel, ws64::kSmemRequest, ws64::kRegsLaunch)) return e;
        kernel<<<grid, ws64::kThreads, ws64::kSmemRequest, stream>>>(tm_q, tm_k, tm_v, tm_o, kp);
        return 0;
      };
      if (general && local) {   // window (with or without sink / softcap / cache view)
        rc = p->D == 128 ? launch64(attn_fwd_ws64_kernel<128, true>)
                         : (p->D == 64 ? launch64(attn_fwd_ws64_kernel<64, true>)
                                       : launch64(attn_fwd_ws64_kernel<192, true>));
      } else if (general && cached) {   // KV-cache view without a window
        rc = p->D == 128 ? launch64(attn_fwd_ws64_kernel<128, true, false, true>)
                         : (p->D == 64 ? launch64(attn_fwd_ws64_kernel<64, true, false, true>)
                                       : launch64(attn_fwd_ws64_kernel<192, true, false, true>));
      } else if (general) {     // sink / softcap only: plain tile geometry
        rc = p->D == 128 ? launch64(attn_fwd_ws64_kernel<128, true, false>)
                         : (p->D == 64 ? launch64(attn_fwd_ws64_kernel<64, true, false>)
                                       : launch64(attn_fwd_ws64_kernel<192, true, false>));
      } else {
        rc = p->D == 128 ? launch64(attn_fwd_ws64_kernel<128>)
                         : (p->D == 64 ? launch64(attn_fwd_ws64_kernel<64>) : launch64(attn_fwd_ws64_kernel<192>));
      }
    } else if (p->D == 128) {
      rc = !general ? launch(attn_fwd_ws_kernel<128, false>)
                    : (local ? launch(attn_fwd_ws_kernel<128, true>) : launch(attn_fwd_ws_kernel<128, true, false>));
    } else {
      rc = !general ? launch(attn_fwd_ws_kernel<64, false>)
                    : (local ? launch(attn_fwd_ws_kernel<64, true>) : launch(attn_fwd_ws_kernel<64, true, false>));
    }
    if (rc != 0) return rc;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (num_splits > 1 || decode) {
    const int64_t items = (int64_t)p->B * p->Sq * p->Hq * (p->Dv / 4);
    int64_t blocks = (items + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (decode) {
      // programmatic dependent launch: the launch latency of the combine kernel overlaps the
      // decode kernel (the combine CTAs wait on griddepcontrol.wait)
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)blocks);
      cfg.blockDim = dim3(256);
      cfg.dynamicSmemBytes = 0;
      cfg.stream = stream;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      const cudaError_t le = cudaLaunchKernelEx(
          &cfg, combine_splits_kernel, (const float*)kp.o_partial, (const float*)kp.lse_partial, kp.out, kp.lse,
          num_splits, p->B, p->Sq, p->Hq, p->Dv, kp.o_stride_b, kp.o_stride_s, kp.o_stride_h);
      if (le != cudaSuccess) return (int)le;
    } else {
      combine_splits_kernel<<<(unsigned)blocks, 256, 0, stream>>>(
          kp.o_partial, kp.lse_partial, kp.out, kp.lse, num_splits, p->B, p->Sq, p->Hq, p->Dv,
          kp.o_stride_b, kp.o_stride_s, kp.o_stride_h);
    }
    e = cudaGetLastError();
  }
  return e == cudaSuccess ? 0 : (int)e;
}
}  // namespace

extern "C" int fa4_nvfp4_sf_linear_to_tiled(const void* src, void* dst, int32_t n_outer,
                                            int32_t n_inner, int32_t rows, int32_t cols,
                                            int64_t stride_outer, int64_t stride_inner,
                                            int64_t stride_row, int32_t col_tile_multiple,
                                            void* cuda_stream) {
  if (!src || !dst) return -FA4_E_NULL;
  if (n_outer <= 0 || n_inner <= 0 || rows <= 0 || cols <= 0 || col_tile_multiple <= 0)
    return -FA4_E_SHAPE;
  if (!aligned16(dst)) return -FA4_E_ALIGN;
  const int64_t ct = ((cols + 3) / 4 + col_tile_multiple - 1) / col_tile_multiple * col_tile_multiple;
  const int64_t total = (int64_t)n_outer * n_inner * ((rows + 127) / 128) * ct * 32;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = 148 * 16;  // grid-stride beyond a few waves
  if (blocks > cap) blocks = cap;
  sf_linear_to_tiled_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), n_outer, n_inner, rows, cols,
      stride_outer, stride_inner, stride_row, col_tile_multiple);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}

// ---------------------------------------------------------------------------------------------
// Fused NVFP4 quantiser (bf16 operands in the reference layout -> what fa4_nvfp4_fwd reads)
// ---------------------------------------------------------------------------------------------
extern "C" int fa4_nvfp4_amax_bf16(const void* x, int64_t n0, int32_t n1, int32_t n2, int32_t inner,
                                   int64_t s0, int64_t s1, int64_t s2, float* amax,
                                   void* cuda_stream) {
  if (!x || !amax) return -FA4_E_NULL;
  if (n0 <= 0 || n1 <= 0 || n2 <= 0 || inner <= 0 || inner % 8 != 0) return -FA4_E_SHAPE;
  if (s0 % 8 != 0 || s1 % 8 != 0 || s2 % 8 != 0) return -FA4_E_STRIDE;
  if (!aligned16(x)) return -FA4_E_ALIGN;
  if (n0 * n1 > 0x7fffffffll || (int64_t)n2 * (inner / 8) > (1 << 24)) return -FA4_E_TOO_LARGE;
  const int rows = (int)(n0 * n1);
  const int per_row = n2 * (inner / 8);
  // a group of rows gives every thread about 8 independent 16-byte loads
  int rows_per_group = (256 * 8 + per_row - 1) / per_row;
  if (rows_per_group > rows) rows_per_group = rows;
  const int groups = (rows + rows_per_group - 1) / rows_per_group;
  const int grid = groups < 148 * 8 ? groups : 148 * 8;
  amax_bf16_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const __nv_bfloat16*>(x), n1, n2, inner / 8, s0, s1, s2, rows, rows_per_group,
      make_fastdiv(per_row), make_fastdiv(inner / 8), make_fastdiv(n1), amax);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int fa4_nvfp4_quantize_qk_bf16(const void* x, int32_t B, int32_t S, int32_t H, int32_t D,
                                          int64_t stride_b, int64_t stride_s, int64_t stride_h,
                                          const float* amax, void* packed, void* sf_linear,
                                          void* sf_tiled, float* scale_out, void* cuda_stream) {
  if (!x || !amax || !packed) return -FA4_E_NULL;
  if (B <= 0 || S <= 0 || H <= 0 || D <= 0 || D % 64 != 0) return -FA4_E_SHAPE;
  if (stride_b % 8 != 0 || stride_s % 8 != 0 || stride_h % 8 != 0) return -FA4_E_STRIDE;
  if (!aligned16(x) || !aligned16(packed) || (sf_linear && !aligned16(sf_linear)) ||
      (sf_tiled && !aligned16(sf_tiled)))
    return -FA4_E_ALIGN;
  const int64_t rows64 = (int64_t)B * ((S + 127) / 128) * 128;
  const int64_t per_row64 = (int64_t)H * (D / 16);
  if (rows64 > 0x7fffffffll || per_row64 > (1 << 24)) return -FA4_E_TOO_LARGE;
  const int per_row = (int)per_row64;
  // about eight blocks of 16 per thread: the per-thread set-up (tensor scale and its reciprocal,
  // index constants) is paid once per CTA, and a CTA streams 64 KB
  int rows_per_group = per_row >= 2048 ? 1 : 2048 / per_row;
  const int64_t groups = (rows64 + rows_per_group - 1) / rows_per_group;
  if (groups > 0x7fffffffll) return -FA4_E_TOO_LARGE;
  quantize_rows_kernel<<<(unsigned)groups, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const __nv_bfloat16*>(x), B, S, H, D, stride_b, stride_s, stride_h, amax,
      static_cast<uint8_t*>(packed), static_cast<uint8_t*>(sf_linear),
      static_cast<uint8_t*>(sf_tiled), scale_out, rows_per_group, make_fastdiv(per_row),
      make_fastdiv(D / 16), make_fastdiv(((S + 127) / 128) * 128));
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int fa4_nvfp4_quantize_v_bf16(const void* x, int32_t B, int32_t Sk, int32_t H, int32_t Dv,
                                         int64_t stride_b, int64_t stride_s, int64_t stride_h,
                                         const float* amax, void* packed, void* sf_linear,
                                         void* sf_tiled, float* scale_out, void* cuda_stream) {
  if (!x || !amax || !packed) return -FA4_E_NULL;
  if (B <= 0 || Sk <= 0 || H <= 0 || Dv <= 0 || Sk % 16 != 0 || Dv % 8 != 0) return -FA4_E_SHAPE;
  if ((int64_t)B * H > 65535) return -FA4_E_TOO_LARGE;
  if (stride_b % 8 != 0 || stride_s % 8 != 0 || stride_h % 8 != 0) return -FA4_E_STRIDE;
  if (!aligned16(x) || !aligned16(packed) || (sf_linear && !aligned16(sf_linear)) ||
      (sf_tiled && !aligned16(sf_tiled)))
    return -FA4_E_ALIGN;
  const dim3 grid((Sk + 127) / 128, (Dv + 127) / 128, B * H);
  quantize_v_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const __nv_bfloat16*>(x), B, Sk, H, Dv, stride_b, stride_s, stride_h, amax,
      static_cast<uint8_t*>(packed), static_cast<uint8_t*>(sf_linear),
      static_cast<uint8_t*>(sf_tiled), scale_out);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int fa4_nvfp4_debug_qk_tile(const void* q, const void* k, const void* q_sf,
                                       const void* k_sf, float* s_out, int32_t D, int32_t mode,
                                       uint32_t* status, void* cuda_stream) {
  if (!q || !k || !q_sf || !k_sf || !s_out) return -FA4_E_NULL;
  if (D != 128) return -FA4_E_SHAPE;
  if (!aligned16(q) || !aligned16(k) || !aligned16(q_sf) || !aligned16(k_sf)) return -FA4_E_ALIGN;
  CUtensorMap tm_q, tm_k;
  const uint64_t d[4] = {64, 1, 128, 1};
  const uint64_t s[3] = {64, 64, 64 * 128};
  const uint32_t b[4] = {64, 1, 128, 1};
  if (!encode_u8_4d(&tm_q, q, d, s, b, CU_TENSOR_MAP_SWIZZLE_64B) ||
      !encode_u8_4d(&tm_k, k, d, s, b, CU_TENSOR_MAP_SWIZZLE_64B))
    return -FA4_E_TENSORMAP;
  if (int e = ensure_smem(qk_tile_probe_kernel, kProbeSmemRequest)) return e;
  qk_tile_probe_kernel<<<1, 128, kProbeSmemRequest, static_cast<cudaStream_t>(cuda_stream)>>>(
      tm_q, tm_k, static_cast<const uint8_t*>(q), static_cast<const uint8_t*>(k),
      static_cast<const uint8_t*>(q_sf), static_cast<const uint8_t*>(k_sf), s_out, mode, status,
      kDefaultBudgetNs);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int fa4_nvfp4_debug_mma_rate(int32_t iters, int32_t num_ctas, uint64_t* clocks_out,
                                        uint32_t* status, void* cuda_stream) {
  if (!clocks_out) return -FA4_E_NULL;
  if (iters < 4 || iters % 4 != 0 || iters > (1 << 22) || num_ctas < 1 || num_ctas > 1024)
    return -FA4_E_SHAPE;
  if (int e = ensure_smem(mma_rate_kernel, kProbeSmemRequest)) return e;
  mma_rate_kernel<<<num_ctas, 128, kProbeSmemRequest, static_cast<cudaStream_t>(cuda_stream)>>>(
      iters, reinterpret_cast<unsigned long long*>(clocks_out), status, kDefaultBudgetNs);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int fa4_nvfp4_debug_ex2_rate(int32_t iters, int32_t num_ctas, uint64_t* clocks_out, float* scratch,
                                        void* cuda_stream) {
  if (!clocks_out || !scratch) return -FA4_E_NULL;
  if (iters < 1 || iters > (1 << 22) || num_ctas < 1 || num_ctas > 1024) return -FA4_E_SHAPE;
  ex2_rate_kernel<<<num_ctas, 512, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      iters, reinterpret_cast<unsigned long long*>(clocks_out), scratch);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int fa4_nvfp4_debug_wait_expiry(uint32_t* status, uint64_t budget_ns, void* cuda_stream) {
  if (!status) return -FA4_E_NULL;
  if (budget_ns == 0 || budget_ns > kDefaultBudgetNs) return -FA4_E_SHAPE;
  wait_expiry_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(status, budget_ns);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}

// ---------------------------------------------------------------------------------------------
// Forward from LINEAR scale factors without any allocation.
//
// The regular route for linear scale factors needs scratch memory: three tiled copies of the
// scales that the caller (the Python wrapper) allocates before calling
// fa4_nvfp4_sf_linear_to_tiled and fa4_nvfp4_fwd.  Some hosts cannot do that: a serving
// process that handed every byte of device memory to its own arena at start-up, or a
// steady-state loop that runs under a "no cudaMalloc" rule because the call synchronises the
// device.  For them the scratch lives in the library image instead: one fixed array per GPU,
// resident from the moment the library is loaded on that GPU until the process exits.
//
// The array name below is only a host-side handle; every call asks the runtime for the device
// address on the current device (cudaGetSymbolAddress), so a pointer from before a
// cudaDeviceReset is never reused.
// ---------------------------------------------------------------------------------------------
#define FA4_STATIC_SCRATCH_BYTES (16u << 20)
static __device__ __align__(256) uint8_t g_sf_scratch[FA4_STATIC_SCRATCH_BYTES];

namespace {
inline int64_t tiled_sf_bytes(int64_t n_mats, int64_t rows, int64_t cols, int64_t ct_multiple) {
  const int64_t ct = ((cols + 3) / 4 + ct_multiple - 1) / ct_multiple * ct_multiple;
  return n_mats * ((rows + 127) / 128) * ct * 512;
}
}  // namespace

extern "C" int fa4_nvfp4_fwd_linear_sf_noalloc(const fa4_nvfp4_params* p, void* cuda_stream) {
  // 1. every host-side check of the forward itself, before anything touches the GPU or the
  //    shared array: a negative return means nothing was launched and nothing was overwritten
  FwdPlan plan;
  if (int e = validate_fwd(p, 1, nullptr, 0, -1, -1, nullptr, 0.f, CacheView{}, /*linear_sf=*/true, &plan))
    return e;
  if (plan.variant == FA4_VARIANT_DECODE) return -FA4_E_VARIANT;   // needs a caller-owned workspace
  // 2. capacity of the array
  const int64_t q_bytes = tiled_sf_bytes((int64_t)p->B * p->Hq, p->Sq, p->D / 16, 1);
  const int64_t k_bytes = tiled_sf_bytes((int64_t)p->B * p->Hkv, p->Sk, p->D / 16, 1);
  const int64_t skp = ((int64_t)p->Sk + 31) / 32 * 32;   // V's padded key axis
  const int64_t v_bytes = tiled_sf_bytes((int64_t)p->B * p->Hkv, p->Dv, skp / 16, 2);
  if (q_bytes + k_bytes + v_bytes > (int64_t)FA4_STATIC_SCRATCH_BYTES) return -FA4_E_TOO_LARGE;

  // 3. device address of the array on the current device
  void* sym = nullptr;
  const cudaError_t se = cudaGetSymbolAddress(&sym, g_sf_scratch);
  if (se != cudaSuccess) return (int)se;
  uint8_t* q_t = static_cast<uint8_t*>(sym);
  uint8_t* k_t = q_t + q_bytes;   // multiples of 512: every region stays 256-byte aligned
  uint8_t* v_t = k_t + k_bytes;

  const int64_t cq = p->D / 16, cv = skp / 16;
  // q_sf (B, Sq, Hq, D/16) and k_sf (B, Sk, Hkv, D/16): matrix (b, h) has row stride H * D/16
  if (int e = fa4_nvfp4_sf_linear_to_tiled(p->q_sf, q_t, p->B, p->Hq, p->Sq, (int)cq,
                                           (int64_t)p->Sq * p->Hq * cq, cq, (int64_t)p->Hq * cq, 1,
                                           cuda_stream))
    return e;
  if (int e = fa4_nvfp4_sf_linear_to_tiled(p->k_sf, k_t, p->B, p->Hkv, p->Sk, (int)cq,
                                           (int64_t)p->Sk * p->Hkv * cq, cq, (int64_t)p->Hkv * cq, 1,
                                           cuda_stream))
    return e;
  // v_sf (B, Hkv, Dv, Sk/16): matrix (b, h) is contiguous
  if (int e = fa4_nvfp4_sf_linear_to_tiled(p->v_sf, v_t, p->B, p->Hkv, p->Dv, (int)cv,
                                           (int64_t)p->Hkv * p->Dv * cv, (int64_t)p->Dv * cv, cv, 2,
                                           cuda_stream))
    return e;
  fa4_nvfp4_params tiled = *p;
  tiled.q_sf = q_t;
  tiled.k_sf = k_t;
  tiled.v_sf = v_t;
  return fa4_nvfp4_fwd(&tiled, cuda_stream);
}
