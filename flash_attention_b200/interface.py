"""Python call surface of the NVFP4 attention forward.

Mirrors ``flash_attn.cute.flash_attn_func`` of the reference
(flash_attn/cute/interface.py:1753-1792 -> FlashAttnFunc.forward :1576-1633 -> _flash_attn_fwd
:279-813): same positional surface, same tensor conventions ((batch, seqlen, heads, head_dim),
GQA map ``h_kv = h // (Hq // Hkv)``, ``softmax_scale=None -> 1/sqrt(D)``, bottom-right aligned
``causal``, returns ``(out, lse)`` with ``lse`` fp32 ``(B, Hq, Sq)`` or ``None``), same error
behaviour (``AssertionError`` for malformed tensors, ``NotImplementedError`` for features that are
not built), launch on the current CUDA stream with no host synchronisation.

The reference asserts fp16/bf16 inputs (interface.py:370); this module is the branch an NVFP4
overload takes before that assert.  Operands arrive either as :class:`NVFP4Tensor` triples through
:func:`flash_attn_func`, or as raw tensors through :func:`flash_attn_fp4_func` whose scale
arguments follow the descale convention of the reference's FP8 path
(hopper/flash_attn_interface.py:81-83).  Output is bf16, as for the reference's quantised inputs
(hopper/flash_api.cpp:859-863).
"""
from __future__ import annotations

import ctypes
import math
from typing import Callable, Optional, Tuple

import torch

from . import _lib
from .quant import NVFP4Tensor, sf_to_tiled

VARIANT_AUTO, VARIANT_WS, VARIANT_WS64, VARIANT_DECODE = 0, 2, 3, 4


def _validate_tensor(t, name, expected_shape, expected_dtype, expected_device):
    # same checks and messages as flash_attn/cute/interface.py:231-236
    assert t.shape == expected_shape, f"{name} shape {t.shape} != expected {expected_shape}"
    assert t.dtype == expected_dtype, f"{name} dtype {t.dtype} != expected {expected_dtype}"
    assert t.device == expected_device, f"{name} device {t.device} != expected {expected_device}"
    assert t.is_cuda, f"{name} must be on CUDA"


def _as_u8(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype == torch.uint8:
        return t
    if t.dtype in (torch.float8_e4m3fn, getattr(torch, "float4_e2m1fn_x2", torch.uint8)):
        return t.view(torch.uint8)
    raise AssertionError(f"{name} must be uint8 / float8_e4m3fn / float4_e2m1fn_x2, got {t.dtype}")


def _scalar(x, name: str) -> float:
    if isinstance(x, torch.Tensor):
        assert x.numel() == 1, f"{name} must be a python float or a 1-element tensor"
        return float(x)  # reads the value (synchronises if it lives on the device)
    return float(x)


class DeviceStatus:
    """One device word per CUDA device that the kernels report bounded-wait expiry into.

    The word is checked lazily: :func:`check_status` reads it back (one small copy, which
    synchronises) and raises if a kernel gave up; the attention call itself never synchronises.
    A launch whose wait ran out leaves its outputs unwritten and returns normally, like any
    asynchronous CUDA failure: call :func:`check_status` wherever results are consumed on the host.
    The word keeps the first failure until it is read, but only the launch that recorded it stops
    early (the kernels compare a per-launch epoch), so later calls are not affected by a stale word.
    """
    _words = {}

    @classmethod
    def word(cls, device: torch.device) -> torch.Tensor:
        idx = device.index if device.index is not None else torch.cuda.current_device()
        w = cls._words.get(idx)
        if w is None:
            w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
            cls._words[idx] = w
        return w


def check_status(device=None) -> None:
    """Raise ``RuntimeError`` if a kernel on ``device`` recorded a failure since the last check."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = DeviceStatus.word(device)
    v = int(w.item()) & 0xFFFFFFFF
    if v != 0:
        w.zero_()
        code, site, epoch, blk = v >> 24, (v >> 16) & 0xFF, (v >> 8) & 0xFF, v & 0xFF
        raise RuntimeError(f"fa4_nvfp4 kernel failure: code {code} (1 = bounded wait expired), "
                           f"wait site {site}, launch epoch {epoch}, block {blk} (mod 256)")


def flash_attn_fp4_func(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
    q_sf: torch.Tensor, k_sf: torch.Tensor, v_sf: torch.Tensor,
    q_scale, k_scale, v_scale,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
    return_lse: bool = False,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    sf_layout: str = "linear",
    variant: int = VARIANT_AUTO,
    num_splits: int = 1,
    window_size: Tuple[Optional[int], Optional[int]] = (None, None),
    learnable_sink: Optional[torch.Tensor] = None,
    softcap: float = 0.0,
    seqused_k: Optional[torch.Tensor] = None,
    page_table: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """NVFP4 attention forward.

    q (B,Sq,Hq,D/2), k (B,Sk,Hkv,D/2), v (B,Hkv,Dv,Skp/2): packed e2m1 bytes (V key-contiguous, its
    key axis padded with zeros to Skp = Sk rounded up to a multiple of 32; the quantisers do that).
    *_sf: e4m3 block scales, ``sf_layout="linear"``: (B,S,H,D/16) / (B,Hkv,Dv,Skp/16), converted
    to the tiled layout by a small kernel; ``"tiled"``: already (B,H,ceil(rows/128),column tiles,512), see ``sf_to_tiled``.
    *_scale: fp32 per-tensor scales.  Returns ``(out bf16 (B,Sq,Hq,Dv), lse fp32 (B,Hq,Sq) | None)``.

    ``num_splits``: 1 = one pass over K/V per query tile; k > 1 = split-KV with a combine kernel
    (the reference's ``num_splits``, interface.py:494-510), for short Sq against long Sk;
    0 = choose (split only when the query tiles alone leave most SMs idle).  Decode and append
    shapes (D = Dv = 128, Sq * Hq / Hkv <= 32, no window / sink / softcap) run the transposed
    decode kernel (``VARIANT_DECODE``: keys on the tile's lanes, grid = splits x Hkv x B); there
    ``num_splits=0`` is what a serving loop wants (about two CTAs per SM).

    ``window_size=(left, right)``: local attention, query row i sees keys
    ``i + Sk - Sq - left <= j <= i + Sk - Sq + right`` (``None`` = unlimited; ``causal`` is
    ``right = 0``), the reference's semantics (flash_attn/cute/interface.py:256-276).

    ``learnable_sink``: (Hq,) logits that join every row's softmax normalisation (and the LSE)
    without contributing a value, the reference's argument of the same name (testing.py:406-416).

    ``softcap`` > 0: the scaled scores become ``softcap * tanh(scores / softcap)`` before masking
    (the reference's ``softcap``, interface.py:528-530 / testing.py:373-374), with the hardware
    ``tanh.approx`` as in the reference's kernel; one more transcendental per score.

    KV cache, the reference's ``seqused_k`` / ``page_table`` (interface.py:296-300, paged_kv.py):
    ``seqused_k`` (B,) int32: batch entry b attends to its first ``seqused_k[b]`` keys only (any
    value in 0..Sk; causal and window limits align to it).  ``page_table`` (B, pages_per_seq)
    int32: k, v and their scales are then a POOL of pages, k (num_pages, page_size, Hkv, D/2),
    v (num_pages, Hkv, Dv, page_size/2), scales per page in either layout, page_size a multiple
    of 128; the logical key length is ``pages_per_seq * page_size``.  Scale bytes of unused
    cache slots must not be NaN encodings (a zero-filled cache is fine).

    Built so far: D = Dv = 128 or 64, or (D, Dv) = (192, 128) (every feature but split-KV and the
    decode kernel); any Sq and Sk, as in the reference (partial last tiles are handled by
    zero-filled loads, a key-length mask and unstored rows).  Anything else raises ``NotImplementedError``
    before a launch.
    """
    q, k, v = _as_u8(q, "q"), _as_u8(k, "k"), _as_u8(v, "v")
    q_sf, k_sf, v_sf = _as_u8(q_sf, "q_sf"), _as_u8(k_sf, "k_sf"), _as_u8(v_sf, "v_sf")
    assert q.dim() == 4 and k.dim() == 4 and v.dim() == 4, "q, k, v must be 4-D"
    assert q.is_cuda and k.is_cuda and v.is_cuda, "inputs must be on CUDA"
    q, k, v = (t if t.stride(-1) == 1 else t.contiguous() for t in (q, k, v))
    B, Sq, Hq, Dh = q.shape
    Bk, Sk, Hkv, Dhk = k.shape
    Bv, Hv, Dv, Skh = v.shape
    D = 2 * Dh
    paged = page_table is not None
    if paged:
        # k / v are a pool of Bk pages of Sk (= page_size) keys
        assert page_table.dim() == 2 and page_table.shape[0] == B and page_table.dtype == torch.int32 \
            and page_table.is_cuda, "page_table must be a (B, pages_per_seq) int32 CUDA tensor"
        assert Bv == Bk, "k and v pools differ in their number of pages"
        if Sk % 128 != 0:
            raise NotImplementedError("page_size must be a multiple of 128 (whole K/V blocks per page)")
        page_table = page_table.contiguous()
        num_pages, page_size, pages_per_seq = Bk, Sk, page_table.shape[1]
        B_kv, Sk_kv = num_pages, page_size           # shapes of the K / V operands
        Sk = pages_per_seq * page_size               # logical key length
    else:
        assert Bk == B and Bv == B, "batch size mismatch"
        B_kv, Sk_kv = B, Sk
    if seqused_k is not None:
        assert seqused_k.shape == (B,) and seqused_k.dtype == torch.int32 and seqused_k.is_cuda, \
            "seqused_k must be a (B,) int32 CUDA tensor"
        seqused_k = seqused_k.contiguous()
    assert Dhk == Dh, "q and k head dims differ"
    Sk_pad = (Sk_kv + 31) // 32 * 32           # V's key axis is padded to whole 32-key groups (zeros)
    assert Hv == Hkv and Skh * 2 == Sk_pad, \
        f"v must be (B, Hkv, Dv, Skp/2) with Skp = seqlen_k rounded up to a multiple of 32, got {tuple(v.shape)}"
    assert Hq % Hkv == 0, "num_head must be divisible by num_head_kv"
    if not ((D == Dv and D in (64, 128)) or (D == 192 and Dv == 128)):
        raise NotImplementedError(f"head dims (D={D}, Dv={Dv}) not built; supported: (128, 128), (64, 64) "
                                  "and (192, 128)")
    device = q.device
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(D)
    if sf_layout == "linear":
        _validate_tensor(q_sf, "q_sf", (B, Sq, Hq, D // 16), torch.uint8, device)
        _validate_tensor(k_sf, "k_sf", (B_kv, Sk_kv, Hkv, D // 16), torch.uint8, device)
        _validate_tensor(v_sf, "v_sf", (B_kv, Hkv, Dv, Sk_pad // 16), torch.uint8, device)
        q_sf, k_sf, v_sf = (t if t.stride(-1) == 1 else t.contiguous() for t in (q_sf, k_sf, v_sf))
        q_sf, k_sf, v_sf = sf_to_tiled(q_sf, 1, 2), sf_to_tiled(k_sf, 1, 2), sf_to_tiled(v_sf, 2, 1, 2)
    elif sf_layout == "tiled":
        _validate_tensor(q_sf, "q_sf", (B, Hq, (Sq + 127) // 128, D // 64, 512), torch.uint8, device)
        _validate_tensor(k_sf, "k_sf", (B_kv, Hkv, (Sk_kv + 127) // 128, D // 64, 512), torch.uint8, device)
        _validate_tensor(v_sf, "v_sf", (B_kv, Hkv, (Dv + 127) // 128, 2 * ((Sk_kv + 127) // 128), 512), torch.uint8,
                         device)
        assert q_sf.is_contiguous() and k_sf.is_contiguous() and v_sf.is_contiguous()
    else:
        raise ValueError(f"sf_layout must be 'linear' or 'tiled', got {sf_layout!r}")

    if out is None:
        out = torch.empty(B, Sq, Hq, Dv, dtype=torch.bfloat16, device=device)
    else:
        _validate_tensor(out, "out", (B, Sq, Hq, Dv), torch.bfloat16, device)
        assert out.stride(-1) == 1
    if lse is None:
        lse = torch.empty(B, Hq, Sq, dtype=torch.float32, device=device) if return_lse else None
    else:
        _validate_tensor(lse, "lse", (B, Hq, Sq), torch.float32, device)
        assert lse.is_contiguous()

    p = _lib.Params()
    p.struct_size = ctypes.sizeof(_lib.Params)
    p.variant = int(variant)
    p.q, p.k, p.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    p.q_sf, p.k_sf, p.v_sf = q_sf.data_ptr(), k_sf.data_ptr(), v_sf.data_ptr()
    p.out = out.data_ptr()
    p.lse = lse.data_ptr() if lse is not None else None
    p.status = DeviceStatus.word(device).data_ptr()
    p.q_stride_b, p.q_stride_s, p.q_stride_h = q.stride(0), q.stride(1), q.stride(2)
    p.k_stride_b, p.k_stride_s, p.k_stride_h = k.stride(0), k.stride(1), k.stride(2)
    p.v_stride_b, p.v_stride_h, p.v_stride_d = v.stride(0), v.stride(1), v.stride(2)
    p.o_stride_b, p.o_stride_s, p.o_stride_h = out.stride(0), out.stride(1), out.stride(2)
    p.B, p.Sq, p.Sk, p.Hq, p.Hkv, p.D, p.Dv = B, Sq, Sk, Hq, Hkv, D, Dv
    p.causal = 1 if causal else 0
    p.q_scale, p.k_scale, p.v_scale = (_scalar(q_scale, "q_scale"), _scalar(k_scale, "k_scale"),
                                       _scalar(v_scale, "v_scale"))
    p.softmax_scale = float(softmax_scale)
    p.wait_budget_ns = 0
    if num_splits < 0 or num_splits > 128:
        raise ValueError("num_splits must be in 0..128")
    auto_splits = num_splits == 0
    if auto_splits:
        num_splits = choose_num_splits(B, Sq, Sk, Hq, causal, device)
    causal, win_left, win_right = resolve_window(causal, window_size)
    p.causal = 1 if causal else 0
    # A handful of query rows per kv head (decode, append): the transposed kernel, which always
    # splits the keys over CTAs and merges with the combine kernel.
    decode_ok = (D == 128 and Dv == 128 and Sq * (Hq // Hkv) <= 32 and win_left is None
                 and (win_right is None or win_right == 0) and learnable_sink is None and not softcap)
    if variant == VARIANT_DECODE and not decode_ok:
        raise NotImplementedError("the decode kernel takes D = Dv = 128, Sq * (Hq / Hkv) <= 32, no window / "
                                  "sink / softcap")
    if variant == VARIANT_AUTO and decode_ok:
        variant = VARIANT_DECODE
    if variant == VARIANT_DECODE:
        p.variant = VARIANT_DECODE
        if auto_splits:
            num_splits = choose_decode_splits(B, Hkv, Sk, device)
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        sink = None
        if learnable_sink is not None:
            assert learnable_sink.shape == (Hq,), "learnable_sink must have one entry per query head"
            sink = learnable_sink.to(device=device, dtype=torch.float32).contiguous()
        softcap = 0.0 if softcap is None else float(softcap)
        if softcap < 0.0 or not math.isfinite(softcap):
            raise ValueError("softcap must be a finite number >= 0")
        if (num_splits == 1 and sink is None and win_left is None and (win_right is None or win_right == 0)
                and softcap == 0.0 and seqused_k is None and not paged and variant != VARIANT_DECODE):
            rc = _lib.lib().fa4_nvfp4_fwd(ctypes.byref(p), stream)
            what = "fa4_nvfp4_fwd"
        else:
            x = _lib.Ext()
            x.struct_size = ctypes.sizeof(_lib.Ext)
            x.num_splits = num_splits
            x.window_left = -1 if win_left is None else int(win_left)
            x.window_right = -1 if win_right is None else int(win_right)
            x.sink = sink.data_ptr() if sink is not None else None
            x.softcap, x.reserved = softcap, 0
            x.seqused_k = seqused_k.data_ptr() if seqused_k is not None else None
            x.page_table = page_table.data_ptr() if paged else None
            if paged:
                x.page_size, x.pages_per_seq, x.num_pages = page_size, pages_per_seq, num_pages
            workspace = None
            if num_splits > 1 or variant == VARIANT_DECODE:
                nbytes = _lib.lib().fa4_nvfp4_splitkv_workspace_bytes(ctypes.byref(p), max(2, num_splits))
                if nbytes < 0:
                    _lib.check(int(nbytes), "fa4_nvfp4_splitkv_workspace_bytes")
                workspace = torch.empty(nbytes, dtype=torch.uint8, device=device)   # stream-ordered scratch
                x.workspace, x.workspace_bytes = workspace.data_ptr(), nbytes
            rc = _lib.lib().fa4_nvfp4_fwd_ex(ctypes.byref(p), ctypes.byref(x), stream)
            what = "fa4_nvfp4_fwd_ex"
    _lib.check(rc, what)
    return out, lse


def choose_decode_splits(B: int, Hkv: int, Sk: int, device=None) -> int:
    """Key splits of the decode kernel (grid = splits x Hkv x B; three CTAs fit an SM).

    The kernel streams K and V at the pace of HBM once about two CTAs per SM pull on it, so the
    count aims at 2 x SMs CTAs (more splits only add partials for the combine kernel), with at
    least two 128-key blocks per split.  When B x Hkv alone exceeds the 3 x SMs resident CTAs the
    grid runs in waves anyway: then the count (up to 4) that minimises waves x (blocks per split + 4
    blocks of fixed cost per CTA) evens out the last wave.  Measured on B200 (Hq 32, Hkv 8, us per
    call): B=4, Sk=32768: 9 or 13 splits 46, 18 splits 54; B=1, Sk=131072: 37 splits 50, 55 splits
    54; B=64, Sk=4096: 1 split 89, 2 splits 79."""
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    blocks = (Sk + 127) // 128
    units = max(1, B * Hkv)
    if units > 3 * sms:
        cost = lambda ns: -(-ns * units // (3 * sms)) * (-(-blocks // ns) + 4)
        return min((ns for ns in range(1, 5) if ns <= max(1, blocks // 2)), key=lambda ns: (cost(ns), ns))
    want = max(1, (2 * sms + units // 2) // units)
    return max(1, min(128, want, max(1, blocks // 2)))


def resolve_window(causal: bool, window_size) -> Tuple[bool, Optional[int], Optional[int]]:
    """(causal, left, right) after the reference's rules (flash_attn/cute/interface.py:256-276):
    causal sets right = 0; a window whose two limits sum to less than zero means no window;
    (None, 0) is plain causal.  One difference: the reference keeps a negative limit whose partner
    outweighs it (a band shifted off the diagonal, e.g. (-2, 5)); the C ABI encodes "no limit" as
    -1, so such windows raise ``NotImplementedError`` here instead."""
    left, right = window_size
    if causal:
        right = 0
    if left is not None and right is not None and left + right < 0:
        left, right = None, None
    if (left is not None and left < 0) or (right is not None and right < 0):
        raise NotImplementedError("negative window limits (a band shifted off the diagonal) are not built")
    return right == 0 and left is None, left, right


def choose_num_splits(B: int, Sq: int, Sk: int, Hq: int, causal: bool, device) -> int:
    """Split count for ``num_splits=0``.

    1 unless the query tiles alone would leave more than half of the SMs idle.  Otherwise the
    count that minimises (waves of work items over the SMs) x (K/V blocks per item + 2 blocks of
    fixed cost per item), at least four blocks per split -- the efficiency search of the
    reference's heuristic (flash_attn/cute/interface.py:494-510) on this kernel's cost model.
    """
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    tiles = B * Hq * ((Sq + 127) // 128)
    blocks = (Sk + 127) // 128          # the last query rows see every key, causal or not
    if tiles * 2 > sms or blocks < 8:
        return 1
    best, best_cost = 1, None
    for n in range(1, min(blocks // 4, 128) + 1):
        per = (blocks + n - 1) // n
        if n > 1 and per * (n - 1) >= blocks:
            continue                      # the last split would be empty
        cost = ((tiles * n + sms - 1) // sms) * (per + 2)
        if best_cost is None or cost < best_cost:
            best, best_cost = n, cost
    return best


def flash_attn_func(
    q, k, v,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
    window_size: Tuple[Optional[int], Optional[int]] = (None, None),
    learnable_sink: Optional[torch.Tensor] = None,
    softcap: float = 0.0,
    num_splits: int = 1,
    pack_gqa: Optional[bool] = None,
    deterministic: bool = False,
    mask_mod: Optional[Callable] = None,
    full_block_cnt: Optional[torch.Tensor] = None,
    full_block_idx: Optional[torch.Tensor] = None,
    mask_block_cnt: Optional[torch.Tensor] = None,
    mask_block_idx: Optional[torch.Tensor] = None,
    block_size: Optional[Tuple[int, int]] = None,
    return_lse: bool = False,
):
    """Same signature as the reference's ``flash_attn_func`` (interface.py:1753-1772); q, k, v are
    :class:`NVFP4Tensor`.  Keyword arguments of features that are not built raise
    ``NotImplementedError``; ``pack_gqa`` and ``deterministic`` are accepted and ignored (the
    forward is deterministic, and query heads of a kv head share K/V through L2 instead of being
    packed into one tile)."""
    if not all(isinstance(t, NVFP4Tensor) for t in (q, k, v)):
        raise TypeError("flash_attn_func of this package takes NVFP4Tensor operands; "
                        "see quantize_qkv()")
    if mask_mod is not None or any(t is not None for t in (full_block_cnt, full_block_idx,
                                                           mask_block_cnt, mask_block_idx)):
        raise NotImplementedError("mask_mod / block sparsity is not built")
    layouts = {t.tiled for t in (q, k, v)}
    if len(layouts) != 1 or any(t.sf_tiled is not None for t in (q, k, v)):
        q, k, v = (NVFP4Tensor(t.data, t.tiled_sf(), t.scale, True, t.is_v) for t in (q, k, v))
    return flash_attn_fp4_func(
        q.data, k.data, v.data, q.sf, k.sf, v.sf, q.scale, k.scale, v.scale,
        softmax_scale=softmax_scale, causal=causal, return_lse=return_lse,
        sf_layout="tiled" if q.tiled else "linear", num_splits=num_splits, window_size=tuple(window_size),
        learnable_sink=learnable_sink, softcap=0.0 if softcap is None else softcap)


def measure_fp4_mma_rate(iters: int = 1 << 16, device=None, repeats: int = 3) -> dict:
    """Dense block-scaled e2m1 tensor-pipe rate of this GPU, measured.

    Launches one CTA per SM that issues ``iters`` 128x128x64 MMAs back to back from shared memory
    (``fa4_nvfp4_debug_mma_rate``) and times the launch with CUDA events.  Returns the best of
    ``repeats``: ``{"tflops", "clk_per_mma" (median over CTAs, in-kernel clocks), "ms", "sms"}``.
    The benchmark reports it beside the nominal dense-FP4 figure.
    """
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    clocks = torch.zeros(sms, dtype=torch.int64, device=device)
    status = DeviceStatus.word(device)
    stream = torch.cuda.current_stream(device)
    best = None
    for _ in range(repeats + 1):          # the first launch is the warm-up
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        _lib.check(_lib.lib().fa4_nvfp4_debug_mma_rate(iters, sms, clocks.data_ptr(), status.data_ptr(),
                                                      stream.cuda_stream), "fa4_nvfp4_debug_mma_rate")
        e1.record(stream)
        e1.synchronize()
        ms = e0.elapsed_time(e1)
        if best is None or ms < best:
            best = ms
    check_status(device)
    flops = sms * iters * 2.0 * 128 * 128 * 64
    return {"tflops": flops / (best * 1e-3) / 1e12, "ms": best, "sms": sms,
            "clk_per_mma": float(clocks.double().median().item()) / iters}


def measure_ex2_rate(iters: int = 1 << 12, device=None) -> dict:
    """Rate of the exponential unit of this GPU, measured (``fa4_nvfp4_debug_ex2_rate``): one CTA of
    16 warps per SM, 16 independent ``ex2.approx`` per thread and round.  Returns
    ``{"per_clk_per_sm" (median over CTAs), "sms"}``; the benchmark's exponential roofline uses it."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    clocks = torch.zeros(sms, dtype=torch.int64, device=device)
    scratch = torch.zeros(1, dtype=torch.float32, device=device)
    stream = torch.cuda.current_stream(device)
    for _ in range(2):                    # the first launch is the warm-up
        _lib.check(_lib.lib().fa4_nvfp4_debug_ex2_rate(iters, sms, clocks.data_ptr(), scratch.data_ptr(),
                                                      stream.cuda_stream), "fa4_nvfp4_debug_ex2_rate")
    torch.cuda.synchronize(device)
    clk = float(clocks.double().median().item())
    return {"per_clk_per_sm": 512.0 * iters * 16 / clk, "sms": sms}
