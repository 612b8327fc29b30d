"""Variable-length (packed) batches: the call surface of the reference's ``flash_attn_varlen_func``
(flash_attn/cute/interface.py:1795-1840) for NVFP4 operands, in ONE kernel launch.

Sequences are packed along the token axis, ``cu_seqlens_*`` are the usual exclusive prefix sums
(int32, on the device):

    q     (total_q, Hq,  D/2)    packed e2m1        q_sf  (total_q, Hq,  D/16)
    k     (total_k, Hkv, D/2)                       k_sf  (total_k, Hkv, D/16)
    v     (Hkv, Dv, total_kp/2)  key-contiguous     v_sf  (Hkv, Dv, total_kp/16)
    out   (total_q, Hq, Dv) bf16                    lse   (Hq, total_q) fp32

(total_kp: V's own key axis, see below).  The reference walks all
sequences inside one persistent kernel (flash_attn/cute/tile_scheduler.py:755-1087); so does this:
the kernel's work list is (sequence, 128-row block of the LONGEST sequence, head), every CTA reads
the bounds of its sequence from ``cu_seqlens`` on the device, a tile past the end of a short
sequence is skipped, the last tile of a sequence stores only its own rows.  Nothing is read back
to the host when ``max_seqlen_q`` / ``max_seqlen_k`` are given, as in the reference's call; without
them they are taken from ``cu_seqlens`` (one synchronising read).  Query and key boundaries are
free.  V alone has a layout rule: it is blocked by 16 keys and its rows must start on 16-byte
boundaries, so INSIDE V every sequence starts on a multiple of 32 keys.  ``cu_seqlens_v`` gives
those starts (slot i is ``cu_seqlens_v[i] .. cu_seqlens_v[i+1]``, its tail beyond the sequence's
keys zero, total_kp = ``cu_seqlens_v[-1]``); :func:`quantize_varlen_qkv` builds V that way from
packed bf16 tensors.  Without ``cu_seqlens_v`` V is taken to be packed like K (total_kp = total_k
rounded up to 32), which needs key-sequence starts that are multiples of 32 themselves.  The
results are bit-identical to dense calls on the single sequences.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Tuple

import torch

from . import _lib
from .interface import DeviceStatus, _as_u8, _scalar, resolve_window
from .quant import NVFP4Tensor, quantize_qkv_fused


def padded_key_offsets(cu_seqlens_k: torch.Tensor) -> torch.Tensor:
    """``cu_seqlens_v`` for a packed batch: the starts of the sequences inside V, every sequence
    padded to a multiple of 32 keys (device int32, no synchronisation)."""
    cu = cu_seqlens_k.to(torch.int64)
    slots = (cu[1:] - cu[:-1] + 31) // 32 * 32
    return torch.cat([cu.new_zeros(1), slots.cumsum(0)]).to(torch.int32)


def quantize_varlen_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_k, total_v: Optional[int] = None):
    """Packed bf16 ``q (total_q, Hq, D)``, ``k (total_k, Hkv, D)``, ``v (total_k, Hkv, Dv)`` ->
    ``(Q, K, V, cu_seqlens_v)`` for :func:`flash_attn_varlen_fp4_func`: three :class:`NVFP4Tensor`
    with a leading batch axis of 1 (pass ``X.data[0]``, ``X.sf[0]``) and the starts of the sequences
    inside V.  Q and K are quantised as packed; V's keys are first moved to slots of whole 32-key
    groups per sequence (zeros between), so that no 16-key scale block mixes two sequences and every
    sequence's rows start on a 16-byte boundary.  ``total_v`` (= sum of the padded lengths) avoids
    the one synchronising read that sizes V."""
    dev = q.device
    cu_k = _device_i32(cu_seqlens_k, "cu_seqlens_k", dev)
    cu_v = padded_key_offsets(cu_k)
    if total_v is None:
        total_v = int(cu_v[-1])
    total_k = k.shape[0]
    # destination slot of every key: its index plus the padding inserted before its sequence
    lens = (cu_k[1:] - cu_k[:-1]).to(torch.int64)
    shift = (cu_v[:-1] - cu_k[:-1]).to(torch.int64)
    dst = torch.arange(total_k, device=dev) + torch.repeat_interleave(shift, lens, output_size=total_k)
    v_slots = v.new_zeros(total_v, v.shape[1], v.shape[2])
    v_slots[dst] = v
    Q, K, V = quantize_qkv_fused(q[None], k[None], v_slots[None])
    return Q, K, V, cu_v


def _device_i32(x, name: str, device) -> torch.Tensor:
    if not isinstance(x, torch.Tensor):
        x = torch.tensor(list(x), dtype=torch.int32)
    assert x.dim() == 1, f"{name} must be one-dimensional"
    return x.to(device=device, dtype=torch.int32).contiguous()


def _tiled_packed(sf, cu, num_seqs, n_inner, max_rows, max_cols, stride_inner, stride_row, mult, packed_rows):
    ct = ((max_cols + 3) // 4 + mult - 1) // mult * mult
    out = torch.empty(num_seqs, n_inner, (max_rows + 127) // 128, ct, 512, dtype=torch.uint8, device=sf.device)
    stream = torch.cuda.current_stream(sf.device).cuda_stream
    rc = _lib.lib().fa4_nvfp4_sf_linear_to_tiled_packed(sf.data_ptr(), out.data_ptr(), cu.data_ptr(), num_seqs,
                                                       n_inner, max_rows, max_cols, stride_inner, stride_row,
                                                       mult, 1 if packed_rows else 0, stream)
    _lib.check(rc, "fa4_nvfp4_sf_linear_to_tiled_packed")
    return out


def flash_attn_varlen_fp4_func(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
    q_sf: torch.Tensor, k_sf: torch.Tensor, v_sf: torch.Tensor,
    q_scale, k_scale, v_scale,
    cu_seqlens_q, cu_seqlens_k,
    seqused_k=None,
    cu_seqlens_v=None,
    max_seqlen_q: Optional[int] = None,
    max_seqlen_k: Optional[int] = None,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
    window_size: Tuple[Optional[int], Optional[int]] = (None, None),
    learnable_sink: Optional[torch.Tensor] = None,
    softcap: float = 0.0,
    return_lse: bool = False,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """NVFP4 attention over a packed batch in one launch; see the module docstring for the layouts.

    ``cu_seqlens_v`` (optional): the starts of the sequences inside ``v`` / ``v_sf`` when V pads
    every sequence to whole 32-key groups (what :func:`quantize_varlen_qkv` returns); without it
    the key-sequence starts of ``cu_seqlens_k`` must be multiples of 32.
    ``seqused_k[i]`` (optional, any value up to the slot) is the number of valid keys of sequence i
    when its slot ``cu_seqlens_k[i+1] - cu_seqlens_k[i]`` is padded; causal alignment is then taken
    against the valid length.  A sequence without keys gives zero rows and LSE = -inf (LSE = sink
    with a learnable sink), as the dense call does.
    """
    q, k, v = _as_u8(q, "q"), _as_u8(k, "k"), _as_u8(v, "v")
    q_sf, k_sf, v_sf = _as_u8(q_sf, "q_sf"), _as_u8(k_sf, "k_sf"), _as_u8(v_sf, "v_sf")
    assert q.dim() == 3 and k.dim() == 3 and v.dim() == 3, "packed operands are 3-D"
    # offsets that arrive as host sequences are checked here, before any launch; device tensors are
    # taken as they are (reading them back would synchronise)
    for name, cu, total in (("cu_seqlens_q", cu_seqlens_q, q.shape[0]), ("cu_seqlens_k", cu_seqlens_k, k.shape[0])):
        if not isinstance(cu, torch.Tensor):
            c = [int(x_) for x_ in cu]
            assert len(c) >= 2 and c[0] == 0 and all(b_ >= a_ for a_, b_ in zip(c, c[1:])), \
                f"{name} must be non-decreasing and start at 0"
            assert c[-1] == total, f"{name} does not cover the packed tensor"
            if name == "cu_seqlens_k" and cu_seqlens_v is None and any(x_ % 32 for x_ in c[:-1]):
                raise NotImplementedError("key-sequence starts that are not multiples of 32 need V in padded slots: "
                                          "pass cu_seqlens_v (see quantize_varlen_qkv)")
    if not isinstance(cu_seqlens_q, torch.Tensor) and not isinstance(cu_seqlens_k, torch.Tensor):
        assert len(list(cu_seqlens_q)) == len(list(cu_seqlens_k)), \
            "cu_seqlens_q and cu_seqlens_k describe different batch sizes"
    assert q.is_cuda and k.is_cuda and v.is_cuda, "inputs must be on CUDA"
    q, k, v = (t if t.stride(-1) == 1 else t.contiguous() for t in (q, k, v))
    q_sf, k_sf, v_sf = (t.contiguous() for t in (q_sf, k_sf, v_sf))
    device = q.device
    total_q, Hq, Dh = q.shape
    total_k, Hkv, Dhk = k.shape
    Hv, Dv, Tkh = v.shape
    D = 2 * Dh
    total_kp = 2 * Tkh if cu_seqlens_v is not None else (total_k + 31) // 32 * 32
    assert Dhk == Dh and Hv == Hkv and Hq % Hkv == 0, "head counts / head dims of q, k, v do not fit"
    assert Tkh * 2 == total_kp and total_kp % 32 == 0 and total_kp >= total_k, \
        f"v must be (Hkv, Dv, total_kp/2) with total_kp = {total_kp}, got {tuple(v.shape)}"
    assert q_sf.shape == (total_q, Hq, D // 16) and k_sf.shape == (total_k, Hkv, D // 16) and \
        v_sf.shape == (Hkv, Dv, total_kp // 16), "scale factors must be the packed linear layouts"
    if not ((D == Dv and D in (64, 128)) or (D == 192 and Dv == 128)):
        raise NotImplementedError(f"head dims (D={D}, Dv={Dv}) not built")
    cu_q = _device_i32(cu_seqlens_q, "cu_seqlens_q", device)
    cu_k = _device_i32(cu_seqlens_k, "cu_seqlens_k", device)
    assert cu_q.numel() == cu_k.numel() and cu_q.numel() >= 2, "cu_seqlens_q / cu_seqlens_k describe different batches"
    num_seqs = cu_q.numel() - 1
    cu_v = None
    if cu_seqlens_v is not None:
        if not isinstance(cu_seqlens_v, torch.Tensor):
            cv = [int(x_) for x_ in cu_seqlens_v]
            assert len(cv) == num_seqs + 1 and cv[0] == 0 and all(x_ % 32 == 0 for x_ in cv) and cv[-1] == total_kp, \
                "cu_seqlens_v must start at 0, hold multiples of 32 and end at the length of v's key axis"
        cu_v = _device_i32(cu_seqlens_v, "cu_seqlens_v", device)
        assert cu_v.numel() == num_seqs + 1
    used = None
    if seqused_k is not None:
        used = _device_i32(seqused_k, "seqused_k", device)
        assert used.numel() == num_seqs
    if max_seqlen_q is None or max_seqlen_k is None:
        # one synchronising read; pass both to stay asynchronous, as the reference's callers do
        max_seqlen_q = int((cu_q[1:] - cu_q[:-1]).max())
        max_seqlen_k = int((cu_k[1:] - cu_k[:-1]).max())
    max_seqlen_q = min(max(1, int(max_seqlen_q)), total_q)
    max_seqlen_k = min(max(1, int(max_seqlen_k)), total_k)
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(D)
    causal, win_left, win_right = resolve_window(causal, window_size)

    # per-sequence tiled scale factors, padded to the longest sequence (a conversion kernel each)
    q_t = _tiled_packed(q_sf, cu_q, num_seqs, Hq, max_seqlen_q, D // 16, D // 16, Hq * (D // 16), 1, True)
    k_t = _tiled_packed(k_sf, cu_k, num_seqs, Hkv, max_seqlen_k, D // 16, D // 16, Hkv * (D // 16), 1, True)
    v_t = _tiled_packed(v_sf, cu_v if cu_v is not None else cu_k, num_seqs, Hkv, Dv, (max_seqlen_k + 15) // 16,
                        Dv * (total_kp // 16), total_kp // 16, 2, False)

    out = torch.empty(total_q, Hq, Dv, dtype=torch.bfloat16, device=device)
    lse = torch.empty(Hq, total_q, dtype=torch.float32, device=device) if return_lse else None

    p = _lib.Params()
    p.struct_size = ctypes.sizeof(_lib.Params)
    p.variant = 0
    p.q, p.k, p.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    p.q_sf, p.k_sf, p.v_sf = q_t.data_ptr(), k_t.data_ptr(), v_t.data_ptr()
    p.out = out.data_ptr()
    p.lse = lse.data_ptr() if lse is not None else None
    p.status = DeviceStatus.word(device).data_ptr()
    p.q_stride_s, p.q_stride_h, p.q_stride_b = q.stride(0), q.stride(1), q.stride(0) * max(1, total_q)
    p.k_stride_s, p.k_stride_h, p.k_stride_b = k.stride(0), k.stride(1), k.stride(0) * max(1, total_k)
    p.v_stride_h, p.v_stride_d, p.v_stride_b = v.stride(0), v.stride(1), v.stride(0) * Hkv
    p.o_stride_s, p.o_stride_h, p.o_stride_b = out.stride(0), out.stride(1), out.stride(0) * max(1, total_q)
    p.B, p.Sq, p.Sk, p.Hq, p.Hkv, p.D, p.Dv = num_seqs, max_seqlen_q, max_seqlen_k, Hq, Hkv, D, Dv
    p.causal = 1 if causal else 0
    p.q_scale, p.k_scale, p.v_scale = _scalar(q_scale, "q_scale"), _scalar(k_scale, "k_scale"), _scalar(v_scale, "v_scale")
    p.softmax_scale = float(softmax_scale)
    p.wait_budget_ns = 0

    x = _lib.Varlen()
    x.struct_size = ctypes.sizeof(_lib.Varlen)
    x.num_seqs = num_seqs
    x.cu_seqlens_q, x.cu_seqlens_k = cu_q.data_ptr(), cu_k.data_ptr()
    x.seqused_k = used.data_ptr() if used is not None else None
    x.total_q, x.total_k = total_q, total_k
    x.max_seqlen_q, x.max_seqlen_k = max_seqlen_q, max_seqlen_k
    x.window_left = -1 if win_left is None else int(win_left)
    x.window_right = -1 if win_right is None else int(win_right)
    sink = None
    if learnable_sink is not None:
        assert learnable_sink.shape == (Hq,), "learnable_sink must have one entry per query head"
        sink = learnable_sink.to(device=device, dtype=torch.float32).contiguous()
    x.sink = sink.data_ptr() if sink is not None else None
    x.softcap = float(softcap or 0.0)
    x.reserved = 0
    x.cu_seqlens_v = cu_v.data_ptr() if cu_v is not None else None
    x.total_v = total_kp if cu_v is not None else 0
    x.reserved2 = 0
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        rc = _lib.lib().fa4_nvfp4_fwd_varlen(ctypes.byref(p), ctypes.byref(x), stream)
    _lib.check(rc, "fa4_nvfp4_fwd_varlen")
    return out, lse
