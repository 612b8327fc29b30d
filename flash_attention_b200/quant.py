"""NVFP4 quantisation of attention operands (torch ops; runs on whatever device the input is on).

Format: e2m1 elements (two per byte, even index in the low nibble), one e4m3 scale per 16
consecutive elements, one fp32 scale per tensor:
    per-tensor scale = amax / (6 * 448)
    block scale      = e4m3(block_amax / 6 / per-tensor scale)
    element          = e2m1 round-to-nearest-even of x / (block scale * per-tensor scale)
Q and K are blocked along the head dimension, V along the key axis (V is stored transposed,
(B, Hkv, Dv, Sk), because 4-bit tensor-core operands must be contiguous along the contraction).

The reference has no quantiser for this path (flash_attn/cute/interface.py:370 rejects anything
but fp16/bf16); the nearest precedent is the FP8 path of the Hopper generation, which takes
per-(batch, kv-head) descale factors (hopper/flash_attn_interface.py:81-83).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib

_MID = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
_TIE_UP = (False, True, False, True, False, True, False)


def _e2m1_codes(x: torch.Tensor) -> torch.Tensor:
    mag = x.abs()
    code = torch.zeros_like(x, dtype=torch.uint8)
    for mid, up in zip(_MID, _TIE_UP):
        code += (mag >= mid).to(torch.uint8) if up else (mag > mid).to(torch.uint8)
    sign = ((x < 0) & (code > 0)).to(torch.uint8)
    return code | (sign << 3)


def quantize_lastdim(x: torch.Tensor, scale: Optional[float] = None):
    """x (..., n) float -> (packed uint8 (..., n/2), sf uint8-viewed e4m3 (..., n/16), scale)."""
    assert x.shape[-1] % 16 == 0, "NVFP4 blocks are 16 elements"
    xf = x.float()
    if scale is None:
        amax = float(xf.abs().max())
        scale = amax / (6.0 * 448.0) if amax > 0 else 1.0
    scale = float(torch.tensor(scale, dtype=torch.float32))  # round to fp32 once
    xb = xf.reshape(*xf.shape[:-1], xf.shape[-1] // 16, 16)
    bmax = xb.abs().amax(dim=-1)
    sf8 = (bmax / 6.0 / scale).clamp(max=448.0).to(torch.float8_e4m3fn)
    denom = (sf8.float() * scale).unsqueeze(-1)
    scaled = torch.where(denom > 0, xb / denom, torch.zeros_like(xb))
    codes = _e2m1_codes(scaled).reshape(xf.shape)
    packed = codes[..., 0::2] | (codes[..., 1::2] << 4)
    return packed.contiguous(), sf8.view(torch.uint8).contiguous(), scale


_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def dequantize_lastdim(packed: torch.Tensor, sf: torch.Tensor, scale: float) -> torch.Tensor:
    """Inverse of quantize_lastdim, fp32."""
    lut = torch.tensor(_E2M1 + tuple(-v for v in _E2M1), dtype=torch.float32, device=packed.device)
    codes = torch.stack([packed & 0xF, packed >> 4], dim=-1).reshape(*packed.shape[:-1], -1)
    vals = lut[codes.long()]
    sff = sf.view(torch.float8_e4m3fn).float() * scale
    vb = vals.reshape(*vals.shape[:-1], vals.shape[-1] // 16, 16) * sff.unsqueeze(-1)
    return vb.reshape(vals.shape)


def sf_to_tiled(sf: torch.Tensor, rows_dim: int, head_dim: Optional[int],
                col_tile_multiple: int = 1) -> torch.Tensor:
    """Linear block scales -> the tiled layout the kernel reads (see include/fa4_nvfp4.h).

    ``sf`` is (B, S, H, C) with ``rows_dim=1, head_dim=2`` (Q, K) or (B, H, R, C) with
    ``rows_dim=2, head_dim=1`` (V, which also needs ``col_tile_multiple=2``: a 128-key block is two
    64-key column tiles).  Returns uint8 (B, H, ceil(rows/128), CT, 512) with CT = ceil(C/4)
    rounded up to a multiple of ``col_tile_multiple``.
    Runs the library's conversion kernel on CUDA tensors; the result is scratch the attention
    call reads.
    """
    assert sf.dim() == 4 and sf.dtype == torch.uint8 and sf.stride(-1) == 1
    B = sf.shape[0]
    H, R, C = sf.shape[head_dim], sf.shape[rows_dim], sf.shape[3]
    ct = ((C + 3) // 4 + col_tile_multiple - 1) // col_tile_multiple * col_tile_multiple
    out = torch.empty(B, H, (R + 127) // 128, ct, 512, dtype=torch.uint8, device=sf.device)
    if not sf.is_cuda:
        raise RuntimeError("sf_to_tiled needs CUDA tensors (the conversion is a CUDA kernel)")
    stream = torch.cuda.current_stream(sf.device).cuda_stream
    rc = _lib.lib().fa4_nvfp4_sf_linear_to_tiled(
        sf.data_ptr(), out.data_ptr(), B, H, R, C, sf.stride(0), sf.stride(head_dim),
        sf.stride(rows_dim), col_tile_multiple, stream)
    _lib.check(rc, "fa4_nvfp4_sf_linear_to_tiled")
    return out


@dataclass
class NVFP4Tensor:
    """One quantised attention operand.

    data   uint8, packed e2m1: (B, S, H, D/2) for q/k, (B, Hkv, Dv, Sk/2) for v
    sf     uint8 (e4m3 bits): linear (B, S, H, D/16) / (B, Hkv, Dv, Sk/16), or tiled
    scale  fp32 per-tensor scale
    tiled  whether ``sf`` is already in the tiled layout
    """
    data: torch.Tensor
    sf: torch.Tensor
    scale: float
    tiled: bool = False
    is_v: bool = False
    sf_tiled: Optional[torch.Tensor] = None   # tiled copy of a linear ``sf`` when one exists already

    def tiled_sf(self) -> torch.Tensor:
        if self.tiled:
            return self.sf
        if self.sf_tiled is not None:
            return self.sf_tiled
        return sf_to_tiled(self.sf, 2, 1, 2) if self.is_v else sf_to_tiled(self.sf, 1, 2)

    def dequantize(self) -> torch.Tensor:
        """fp32 values in the reference layout (B, S, H, D) (linear scale factors only; for V the
        key axis still carries its zero padding to a multiple of 32)."""
        assert not self.tiled
        x = dequantize_lastdim(self.data, self.sf, self.scale)
        return x.permute(0, 3, 1, 2).contiguous() if self.is_v else x


def _pad_keys(v: torch.Tensor) -> torch.Tensor:
    """V (B, Sk, H, D) with its key axis padded with zeros to a multiple of 32: V is quantised and
    stored key-contiguous in blocks of 16 keys, and a row of the packed tensor must be a multiple
    of 16 bytes for the tiled loads.  The kernels mask keys >= Sk (the length of K)."""
    pad = (-v.shape[1]) % 32
    if pad == 0:
        return v
    return torch.cat([v, v.new_zeros(v.shape[0], pad, v.shape[2], v.shape[3])], dim=1)


def quantize_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
    """bf16/fp32 (B,S,H,D) tensors in the reference layout -> three NVFP4Tensor (linear scales)."""
    qd, qs, qg = quantize_lastdim(q)
    kd, ks, kg = quantize_lastdim(k)
    v = _pad_keys(v)
    vt = v.permute(0, 2, 3, 1)  # (B, Hkv, Dv, Skp): blocks along the key axis
    vd, vs, vg = quantize_lastdim(vt)
    return (NVFP4Tensor(qd, qs, qg), NVFP4Tensor(kd, ks, kg), NVFP4Tensor(vd, vs, vg, is_v=True))


def quantize_qkv_fused(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, linear_sf: bool = True):
    """CUDA quantiser: bf16 (B,S,H,D) tensors in the reference layout -> three NVFP4Tensor.

    Same results as :func:`quantize_qkv` computed with correctly rounded fp32 divisions (the CPU
    oracle's arithmetic), in two passes per tensor over HBM (amax, then quantise) instead of a few
    dozen torch kernels: ``fa4_nvfp4_amax_bf16`` + ``fa4_nvfp4_quantize_qk_bf16`` /
    ``fa4_nvfp4_quantize_v_bf16``.  V is transposed to key-contiguous on the way.  The tiled scale
    factors the attention kernel reads are always produced; ``linear_sf=False`` skips the linear
    copies (then ``NVFP4Tensor.dequantize`` is unavailable).  One host synchronisation at the end
    fetches the three per-tensor scales.
    """
    L = _lib.lib()
    outs = []
    dev = q.device
    amax = torch.zeros(3, dtype=torch.float32, device=dev)
    scales = torch.empty(3, dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    v = _pad_keys(v)
    for i, (x, is_v) in enumerate(((q, False), (k, False), (v, True))):
        if not (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 4 and x.stride(-1) == 1):
            raise AssertionError("quantize_qkv_fused takes CUDA bf16 (B, S, H, D) tensors, last dim contiguous")
        B, S, H, D = x.shape
        a_ptr = amax.data_ptr() + 4 * i
        s_ptr = scales.data_ptr() + 4 * i
        _lib.check(L.fa4_nvfp4_amax_bf16(x.data_ptr(), B, S, H, D, x.stride(0), x.stride(1), x.stride(2),
                                         a_ptr, stream), "fa4_nvfp4_amax_bf16")
        if is_v:
            packed = torch.empty(B, H, D, S // 2, dtype=torch.uint8, device=dev)
            lin = torch.empty(B, H, D, S // 16, dtype=torch.uint8, device=dev) if linear_sf else None
            tiled = torch.empty(B, H, (D + 127) // 128, 2 * ((S + 127) // 128), 512, dtype=torch.uint8,
                                device=dev)
            fn, what = L.fa4_nvfp4_quantize_v_bf16, "fa4_nvfp4_quantize_v_bf16"
        else:
            packed = torch.empty(B, S, H, D // 2, dtype=torch.uint8, device=dev)
            lin = torch.empty(B, S, H, D // 16, dtype=torch.uint8, device=dev) if linear_sf else None
            tiled = torch.empty(B, H, (S + 127) // 128, D // 64, 512, dtype=torch.uint8, device=dev)
            fn, what = L.fa4_nvfp4_quantize_qk_bf16, "fa4_nvfp4_quantize_qk_bf16"
        _lib.check(fn(x.data_ptr(), B, S, H, D, x.stride(0), x.stride(1), x.stride(2), a_ptr,
                      packed.data_ptr(), lin.data_ptr() if lin is not None else None,
                      tiled.data_ptr(), s_ptr, stream), what)
        outs.append((packed, lin, tiled, is_v))
    host_scales = scales.tolist()
    res = []
    for (packed, lin, tiled, is_v), sc in zip(outs, host_scales):
        if lin is not None:
            res.append(NVFP4Tensor(packed, lin, float(sc), False, is_v, tiled))
        else:
            res.append(NVFP4Tensor(packed, tiled, float(sc), True, is_v))
    return tuple(res)
