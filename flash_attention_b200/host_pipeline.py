"""Attention forward for operands that live in HOST memory.

``flash_attn_fp4_func`` takes device tensors, like the reference's ``flash_attn_func``
(flash_attn/cute/interface.py:384-398 asserts CUDA inputs).  A caller whose quantised operands
sit in pinned host memory (a KV store, a data loader) would otherwise pay
copy-in -> compute -> copy-out one after the other, and at NVFP4 sizes the copies dominate: the
headline workload moves 113 MB in and 273 MB out for 2 ms of kernel time.  :class:`HostPipeline`
splits the call into independent pieces -- a batch entry's K/V, then ranges of its query rows --
and runs three CUDA streams (copy-in, compute, copy-out) so that both PCIe directions and the
kernel overlap.  A range of query rows [s0, s1) of a causal problem is itself a causal problem
with Sq = s1 - s0 and Sk = s1 (bottom-right aligned), so every piece goes through the same
entry point; rows are split at multiples of 128 (the kernel's tile), which keeps each row's
summation order, hence the result, bit-identical to the single call.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .interface import flash_attn_fp4_func, check_status


class HostPipeline:
    """Reusable device staging buffers and streams for one problem shape on one GPU.

    ``run`` only enqueues work (it never synchronises); ``out_host`` / ``lse_host`` are valid once
    ``done`` (a CUDA event) has completed, e.g. after :meth:`wait`.  Successive ``run`` calls on the
    same object overlap: the next copy-in starts while the previous copy-out drains.
    """

    def __init__(self, B: int, Sq: int, Sk: int, Hq: int, Hkv: int, D: int = 128, Dv: int = 128,
                 device=None, row_chunks: Optional[int] = None):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.shape = (B, Sq, Sk, Hq, Hkv, D, Dv)
        dev = self.device
        u8 = torch.uint8
        self.q = torch.empty(B, Sq, Hq, D // 2, dtype=u8, device=dev)
        self.k = torch.empty(B, Sk, Hkv, D // 2, dtype=u8, device=dev)
        skp = (Sk + 31) // 32 * 32          # V's key axis is padded to whole 32-key groups
        self.v = torch.empty(B, Hkv, Dv, skp // 2, dtype=u8, device=dev)
        self.q_sf = torch.empty(B, Sq, Hq, D // 16, dtype=u8, device=dev)
        self.k_sf = torch.empty(B, Sk, Hkv, D // 16, dtype=u8, device=dev)
        self.v_sf = torch.empty(B, Hkv, Dv, skp // 16, dtype=u8, device=dev)
        self.out = torch.empty(B, Sq, Hq, Dv, dtype=torch.bfloat16, device=dev)
        self.lse = torch.empty(B, Hq, Sq, dtype=torch.float32, device=dev)
        self.s_in = torch.cuda.Stream(dev)
        self.s_compute = torch.cuda.Stream(dev)
        self.s_out = torch.cuda.Stream(dev)
        self.inputs_free = None      # event: the previous run's kernels have read the staging inputs
        self.outputs_free = None     # event: the previous run's copy-out has drained the staging outputs
        self.done = None
        # query-row ranges: equal numbers of 128-row tiles, the last range takes the remainder.
        # Every piece costs about ten stream operations on the host; the default keeps a piece's
        # output at 8 MiB or more (up to four ranges per batch entry) so that small problems --
        # one GPU's shard of a sharded call -- are not bound by the host's launch rate, and at
        # least four pieces per call so that the three streams have something to overlap.
        tiles = (Sq + 127) // 128
        if row_chunks is None:
            row_chunks = max(1, min(4, (Sq * Hq * Dv * 2) // (8 << 20)))
            if B * row_chunks < 4:
                row_chunks = -(-4 // B)
        n = max(1, min(row_chunks, tiles))
        per = (tiles + n - 1) // n
        self.ranges = [(t * 128, min(Sq, (t + per) * 128)) for t in range(0, tiles, per)]

    def run(self, q, k, v, q_sf, k_sf, v_sf, q_scale, k_scale, v_scale, out_host, lse_host=None,
            causal: bool = False, softmax_scale: Optional[float] = None):
        B, Sq, Sk, Hq, Hkv, D, Dv = self.shape
        for t, ref in ((q, self.q), (k, self.k), (v, self.v), (q_sf, self.q_sf), (k_sf, self.k_sf),
                       (v_sf, self.v_sf)):
            assert not t.is_cuda and tuple(t.shape) == tuple(ref.shape) and t.is_contiguous(), \
                "host operands must be contiguous CPU tensors of the pipeline's shape"
        assert tuple(out_host.shape) == tuple(self.out.shape) and out_host.dtype == torch.bfloat16
        if causal and Sq != Sk:
            raise NotImplementedError("HostPipeline splits causal problems only for Sq == Sk")
        caller = torch.cuda.current_stream(self.device)
        first = torch.cuda.Event()
        first.record(caller)
        self.s_in.wait_event(first)
        if self.inputs_free is not None:
            self.s_in.wait_event(self.inputs_free)
        if self.outputs_free is not None:
            self.s_compute.wait_event(self.outputs_free)
        last_compute = None
        for b in range(B):
            with torch.cuda.stream(self.s_in):
                for dst, src in ((self.k, k), (self.v, v), (self.k_sf, k_sf), (self.v_sf, v_sf)):
                    dst[b].copy_(src[b], non_blocking=True)
            for (s0, s1) in self.ranges:
                with torch.cuda.stream(self.s_in):
                    self.q[b, s0:s1].copy_(q[b, s0:s1], non_blocking=True)
                    self.q_sf[b, s0:s1].copy_(q_sf[b, s0:s1], non_blocking=True)
                    ev_in = torch.cuda.Event()
                    ev_in.record(self.s_in)
                sk = s1 if causal else Sk        # s1 is a multiple of 128, or Sq == Sk for the last range
                with torch.cuda.stream(self.s_compute):
                    self.s_compute.wait_event(ev_in)
                    self._piece(b, s0, s1, sk, q_scale, k_scale, v_scale, causal, softmax_scale)
                    ev_c = torch.cuda.Event()
                    ev_c.record(self.s_compute)
                    last_compute = ev_c
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(ev_c)
                    out_host[b, s0:s1].copy_(self.out[b, s0:s1], non_blocking=True)
            if lse_host is not None:
                with torch.cuda.stream(self.s_out):
                    lse_host[b].copy_(self.lse[b], non_blocking=True)
        self.inputs_free = last_compute
        self.outputs_free = torch.cuda.Event()
        self.outputs_free.record(self.s_out)
        self.done = self.outputs_free
        return self.done

    def _piece(self, b, s0, s1, sk, q_scale, k_scale, v_scale, causal, softmax_scale):
        """One range of query rows of batch entry b against its first ``sk`` keys.  The LSE rows of
        a partial range are a strided slice of (Hq, Sq): the kernel writes a small contiguous
        buffer that is copied into place on the same stream."""
        Sq = self.shape[1]
        whole = (s1 - s0 == Sq)
        _, lse_piece = flash_attn_fp4_func(
            self.q[b:b + 1, s0:s1], self.k[b:b + 1, :sk], self.v[b:b + 1, :, :, :(sk + 31) // 32 * 16],
            self.q_sf[b:b + 1, s0:s1], self.k_sf[b:b + 1, :sk], self.v_sf[b:b + 1, :, :, :(sk + 31) // 32 * 2],
            q_scale, k_scale, v_scale, softmax_scale=softmax_scale, causal=causal, return_lse=True,
            out=self.out[b:b + 1, s0:s1], lse=self.lse[b:b + 1] if whole else None, sf_layout="linear")
        if not whole:
            self.lse[b:b + 1, :, s0:s1].copy_(lse_piece)

    def wait(self):
        if self.done is not None:
            self.done.synchronize()
        check_status(self.device)


def flash_attn_fp4_host(q, k, v, q_sf, k_sf, v_sf, q_scale, k_scale, v_scale, causal: bool = False,
                        softmax_scale: Optional[float] = None, device=None, row_chunks: Optional[int] = None,
                        pipeline: Optional[HostPipeline] = None
                        ) -> Tuple[torch.Tensor, torch.Tensor]:
    """One-shot convenience wrapper: host operands in, pinned host ``(out, lse)`` back (synchronises)."""
    B, Sq, Hq, Dh = q.shape
    _, Sk, Hkv, _ = k.shape
    Dv = v.shape[2]
    pipe = pipeline or HostPipeline(B, Sq, Sk, Hq, Hkv, 2 * Dh, Dv, device=device, row_chunks=row_chunks)
    out_host = torch.empty(B, Sq, Hq, Dv, dtype=torch.bfloat16).pin_memory()
    lse_host = torch.empty(B, Hq, Sq, dtype=torch.float32).pin_memory()
    pipe.run(q, k, v, q_sf, k_sf, v_sf, q_scale, k_scale, v_scale, out_host, lse_host, causal=causal,
             softmax_scale=softmax_scale)
    pipe.wait()
    return out_host, lse_host
