"""Variable-length (packed) batches: the call surface of the reference's ``flash_attn_varlen_func``
(flash_attn/cute/interface.py:1795-1840) for NVFP4 operands.

Sequences are packed along the token axis, ``cu_seqlens_*`` are the usual exclusive prefix sums:

    q     (total_q, Hq,  D/2)    packed e2m1        q_sf  (total_q, Hq,  D/16)
    k     (total_k, Hkv, D/2)                       k_sf  (total_k, Hkv, D/16)
    v     (Hkv, Dv, total_k/2)   key-contiguous     v_sf  (Hkv, Dv, total_k/16)
    out   (total_q, Hq, Dv) bf16                    lse   (Hq, total_q) fp32

This first version runs the dense kernel once per sequence on views of the packed tensors (pointer
offsets and strides only, no copies): every sequence is an independent problem, so the results
are those of the dense call.  The reference instead walks all sequences inside one persistent
kernel (tile_scheduler.py:755-1087); with launches of a few microseconds each this wrapper is
the same thing for prefill-sized sequences and launch-bound for many tiny ones.  Because V is
blocked by 16 keys and its rows must start on 16-byte boundaries, every key-sequence boundary
must be a multiple of 32 (pad the keys of a sequence up to it; padded keys are masked when
``seqused_k`` gives the true lengths).  Query boundaries are free.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from .interface import flash_attn_fp4_func


def _host_offsets(cu, name: str) -> Sequence[int]:
    if isinstance(cu, torch.Tensor):
        cu = cu.tolist()          # device tensors are read back once (a synchronisation)
    cu = [int(x) for x in cu]
    assert len(cu) >= 2 and cu[0] == 0 and all(b >= a for a, b in zip(cu, cu[1:])), \
        f"{name} must be non-decreasing and start at 0"
    return cu


def flash_attn_varlen_fp4_func(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
    q_sf: torch.Tensor, k_sf: torch.Tensor, v_sf: torch.Tensor,
    q_scale, k_scale, v_scale,
    cu_seqlens_q, cu_seqlens_k,
    seqused_k: Optional[Sequence[int]] = None,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
    window_size: Tuple[Optional[int], Optional[int]] = (None, None),
    learnable_sink: Optional[torch.Tensor] = None,
    return_lse: bool = False,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """NVFP4 attention over a packed batch; see the module docstring for the layouts.

    ``seqused_k[i]`` (optional) is the number of valid keys of sequence i when its slot
    ``cu_seqlens_k[i+1] - cu_seqlens_k[i]`` is padded; it must be a multiple of 32 too (the key
    granule of the kernel), and causal alignment is then taken against the valid length.
    """
    assert q.dim() == 3 and k.dim() == 3 and v.dim() == 3, "packed operands are 3-D"
    total_q, Hq, Dh = q.shape
    total_k, Hkv, _ = k.shape
    Dv = v.shape[1]
    cq, ck = _host_offsets(cu_seqlens_q, "cu_seqlens_q"), _host_offsets(cu_seqlens_k, "cu_seqlens_k")
    assert len(cq) == len(ck), "cu_seqlens_q and cu_seqlens_k describe different batch sizes"
    assert cq[-1] == total_q and ck[-1] == total_k, "cu_seqlens do not cover the packed tensors"
    if any(x % 32 for x in ck):
        raise NotImplementedError("key-sequence boundaries must be multiples of 32 (16-key scale blocks, "
                                  "16-byte rows of V); pad each sequence's keys")
    out = torch.empty(total_q, Hq, Dv, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(Hq, total_q, dtype=torch.float32, device=q.device) if return_lse else None
    for i in range(len(cq) - 1):
        q0, q1, k0, k1 = cq[i], cq[i + 1], ck[i], ck[i + 1]
        if q1 == q0:
            continue
        sk = k1 - k0 if seqused_k is None else int(seqused_k[i])
        assert 0 <= sk <= k1 - k0
        if sk == 0:
            out[q0:q1].zero_()
            if lse is not None:
                lse[:, q0:q1] = float("-inf")
            continue
        if sk % 32:
            raise NotImplementedError("seqused_k must be a multiple of 32")
        o_i, l_i = flash_attn_fp4_func(
            q[q0:q1].unsqueeze(0), k[k0:k0 + sk].unsqueeze(0), v[:, :, k0 // 2:(k0 + sk) // 2].unsqueeze(0),
            q_sf[q0:q1].unsqueeze(0), k_sf[k0:k0 + sk].unsqueeze(0),
            v_sf[:, :, k0 // 16:(k0 + sk) // 16].unsqueeze(0),
            q_scale, k_scale, v_scale, softmax_scale=softmax_scale, causal=causal, return_lse=return_lse,
            out=out[q0:q1].unsqueeze(0), window_size=window_size, learnable_sink=learnable_sink)
        if lse is not None:
            lse[:, q0:q1] = l_i[0]
    return out, lse
