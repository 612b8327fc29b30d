"""Sharding of one attention problem over the GPUs of a node.

Every (batch, kv-head) pair -- with the Hq/Hkv query heads that read it -- is independent of every
other (a work tile of the reference touches one batch and one kv head,
flash_attn/cute/flash_fwd_sm100.py:1290-1299), so the B*Hkv units are dealt out contiguously
to the ranks and nothing is exchanged on the data path.  Per-tensor scales are computed on the
whole tensor before sharding, which makes a sharded run bit-identical to the single-GPU run.
``gather_output`` (NCCL all-gather of O / LSE) exists for verification only.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .quant import NVFP4Tensor


@dataclass(frozen=True)
class Shard:
    """Rank ``rank`` of ``world`` owns batches [b0, b1) and, inside them, kv heads [h0, h1)."""
    rank: int
    world: int
    b0: int
    b1: int
    h0: int
    h1: int

    @property
    def units(self) -> int:
        return (self.b1 - self.b0) * (self.h1 - self.h0)


def plan_shard(B: int, Hkv: int, world: int, rank: int) -> Shard:
    """Contiguous split of the B*Hkv units.  Either whole batches per rank, or a head range inside
    one batch; anything else (a rank straddling a batch boundary) is rejected."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    units = B * Hkv
    if units % world != 0:
        raise ValueError(f"{units} (batch x kv-head) units do not divide over {world} ranks")
    per = units // world
    if per % Hkv == 0:
        nb = per // Hkv
        return Shard(rank, world, rank * nb, (rank + 1) * nb, 0, Hkv)
    if Hkv % per == 0:
        ranks_per_batch = Hkv // per
        b = rank // ranks_per_batch
        h0 = (rank % ranks_per_batch) * per
        return Shard(rank, world, b, b + 1, h0, h0 + per)
    raise ValueError(f"{per} units per rank neither whole batches nor a divisor of Hkv={Hkv}")


def shard_operands(q: NVFP4Tensor, k: NVFP4Tensor, v: NVFP4Tensor, s: Shard):
    """Views of this rank's slice of linear-layout NVFP4 operands (no copy; scales unchanged)."""
    assert not (q.tiled or k.tiled or v.tiled), "shard before converting scale factors to tiles"
    Hq, Hkv = q.data.shape[2], k.data.shape[2]
    g = Hq // Hkv
    qs = NVFP4Tensor(q.data[s.b0:s.b1, :, s.h0 * g:s.h1 * g], q.sf[s.b0:s.b1, :, s.h0 * g:s.h1 * g], q.scale)
    ks = NVFP4Tensor(k.data[s.b0:s.b1, :, s.h0:s.h1], k.sf[s.b0:s.b1, :, s.h0:s.h1], k.scale)
    vs = NVFP4Tensor(v.data[s.b0:s.b1, s.h0:s.h1], v.sf[s.b0:s.b1, s.h0:s.h1], v.scale, is_v=True)
    return qs, ks, vs


def gather_output(out: torch.Tensor, lse: Optional[torch.Tensor], s: Shard, B: int, Hq: int,
                  Hkv: int, group=None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """All-gather the shards of O (B_s, Sq, Hq_s, Dv) and LSE (B_s, Hq_s, Sq) into full tensors on
    every rank.  Verification helper: never inside a timed region."""
    import torch.distributed as dist
    g = Hq // Hkv

    def gather(t):
        parts = [torch.empty_like(t) for _ in range(s.world)]
        dist.all_gather(parts, t.contiguous(), group=group)
        return parts

    o_parts = gather(out)
    full_o = torch.empty(B, out.shape[1], Hq, out.shape[3], dtype=out.dtype, device=out.device)
    full_l = None
    l_parts = gather(lse) if lse is not None else None
    if lse is not None:
        full_l = torch.empty(B, Hq, lse.shape[2], dtype=lse.dtype, device=lse.device)
    for r in range(s.world):
        sr = plan_shard(B, Hkv, s.world, r)
        full_o[sr.b0:sr.b1, :, sr.h0 * g:sr.h1 * g] = o_parts[r]
        if full_l is not None:
            full_l[sr.b0:sr.b1, sr.h0 * g:sr.h1 * g] = l_parts[r]
    return full_o, full_l
