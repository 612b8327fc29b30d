"""Generate the golden fixtures in this directory from the REFERENCE's own code.

Run once, in a container that has the reference checkout (it is not needed to run the tests):

    python tests/golden/make_golden.py /path/to/reference

What it pins: the CPU oracle's ``attention_oracle_a`` (oracle/nvfp4_oracle.py) against the
reference's ``attention_ref`` (flash_attn/cute/testing.py:323-434, imported by file path so
that ``flash_attn/__init__`` and its compiled extensions are not needed), on NVFP4-dequantised
inputs: MHA / GQA / MQA head mapping, bottom-right aligned causal masks with Sq < Sk and
Sq > Sk (fully masked rows), ragged lengths.  The LSE fixture is computed the way the
reference's tests compute it (tests/cute/test_flash_attn.py:1534-1539: logsumexp of the masked,
scaled scores, mask = triu(diagonal = Sk - Sq + 1)).

Each fixture stores the quantised operands (packed e2m1 bytes, e4m3 block scales, fp32 tensor
scale) and the reference's fp32 output; inputs are N(0,1) bf16 draws from the stated seed,
quantised by oracle.nvfp4_oracle.quantize_nvfp4.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import nvfp4_oracle as orc  # noqa: E402

CASES = [
    # name, B, Sq, Sk, Hq, Hkv, D, causal, seed, window (left, right)
    ("mha_noncausal", 1, 128, 128, 2, 2, 128, False, 0, (None, None)),
    ("gqa_causal_sq_lt_sk", 2, 64, 192, 4, 2, 128, True, 1, (None, None)),
    ("mqa_causal_sq_gt_sk", 1, 160, 96, 2, 1, 128, True, 2, (None, None)),
    ("mqa_noncausal_ragged", 1, 113, 208, 3, 1, 64, False, 3, (None, None)),
    # local attention (the reference's construct_local_mask, testing.py:249-288)
    ("gqa_sliding_window_causal", 1, 320, 320, 4, 2, 128, True, 4, (100, 0)),
    ("mha_window_both_sides_sq_lt_sk", 1, 96, 352, 2, 2, 128, False, 5, (40, 70)),
    # learnable sink (testing.py:406-416): seeded N(0, 1) logits, one per query head
    ("gqa_causal_learnable_sink", 1, 192, 192, 4, 2, 128, True, 6, (None, None)),
    # soft cap (testing.py:373-374): scores = softcap * tanh(scores / softcap), value in SOFTCAP
    ("gqa_causal_softcap", 1, 256, 256, 4, 2, 128, True, 7, (None, None)),
]
SOFTCAP = {"gqa_causal_softcap": 2.0}


def load_reference_testing(ref_root):
    path = os.path.join(ref_root, "flash_attn", "cute", "testing.py")
    spec = importlib.util.spec_from_file_location("ref_cute_testing", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference [fixture name ...]")
    ref_root = sys.argv[1]
    only = set(sys.argv[2:])        # regenerate these only (an .npz is a zip: rewriting changes its bytes)
    ref = load_reference_testing(ref_root)
    torch.set_num_threads(4)
    for name, B, Sq, Sk, Hq, Hkv, D, causal, seed, window in CASES:
        if only and name not in only:
            continue
        softcap = SOFTCAP.get(name, 0.0)
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(B, Sq, Hq, D, generator=g).bfloat16().float().numpy()
        k = torch.randn(B, Sk, Hkv, D, generator=g).bfloat16().float().numpy()
        v = torch.randn(B, Sk, Hkv, D, generator=g).bfloat16().float().numpy()
        Q, K = orc.quantize_nvfp4(q), orc.quantize_nvfp4(k)
        V = orc.quantize_nvfp4(np.ascontiguousarray(np.transpose(v, (0, 2, 3, 1))))  # (B,Hkv,Dv,Sk)
        qd = torch.from_numpy(orc.dequantize_nvfp4(Q))
        kd = torch.from_numpy(orc.dequantize_nvfp4(K))
        vd = torch.from_numpy(np.ascontiguousarray(np.transpose(orc.dequantize_nvfp4(V), (0, 3, 1, 2))))
        sink = torch.randn(Hq, generator=g) * 2.0 if "sink" in name else None
        out_ref, _ = ref.attention_ref(qd, kd, vd, causal=causal, window_size=window, upcast=True,
                                       learnable_sink=sink, softcap=softcap)
        kk = kd.repeat_interleave(Hq // Hkv, dim=2)
        qk = torch.einsum("bshd,bthd->bhst", qd, kk) / (D ** 0.5)
        if softcap > 0:
            qk = torch.tanh(qk / softcap) * softcap
        if window != (None, None):
            w = (window[0], 0) if causal else window
            mask = ref.construct_local_mask(Sq, Sk, w)
            qk = qk.masked_fill(mask, float("-inf"))
        elif causal:
            mask = torch.triu(torch.ones(Sq, Sk, dtype=torch.bool), diagonal=Sk - Sq + 1)
            qk = qk.masked_fill(mask, float("-inf"))
        if sink is not None:
            qk = torch.cat([qk, sink.reshape(1, Hq, 1, 1).expand(B, Hq, Sq, 1)], dim=-1)
        lse_ref = torch.logsumexp(qk, dim=-1)
        np.savez_compressed(
            os.path.join(HERE, f"{name}.npz"),
            q_data=Q.data, q_sf=Q.sf, q_scale=np.float32(Q.scale),
            k_data=K.data, k_sf=K.sf, k_scale=np.float32(K.scale),
            v_data=V.data, v_sf=V.sf, v_scale=np.float32(V.scale),
            out_ref=out_ref.numpy().astype(np.float32), lse_ref=lse_ref.numpy().astype(np.float32),
            causal=np.bool_(causal), seed=np.int64(seed),
            window=np.array([-1 if x is None else x for x in window], dtype=np.int64),
            sink=(sink.numpy().astype(np.float32) if sink is not None else np.zeros(0, dtype=np.float32)),
            softcap=np.float32(softcap))
        print(name, out_ref.shape, float(out_ref.abs().max()))


if __name__ == "__main__":
    main()
