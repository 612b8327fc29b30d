"""Shared helpers of the test-suite: seeded inputs of the benchmark configurations' kind and the
tolerance recipe.

Tolerances (stated here, used by every parity test):

* kernel vs oracle B (the kernel's arithmetic model: same NVFP4 rounding of P) -- the reference's
  own recipe (tests/cute/test_flash_attn.py:265-310): the error may be at most twice the error of
  a same-precision implementation plus a small absolute term.  Here "same precision" is oracle B
  rounded to bf16, so  max|out - B| <= 2 * max|bf16(B) - B| + atol_b  with atol_b = 2^-7 * max|B|
  (a handful of P values sit on an e2m1 rounding boundary and flip with the last bit of the
  hardware exp2), and rel-RMS(out, B) <= 0.01.
* kernel vs oracle A (fp32 attention on the dequantised inputs): rel-RMS(out, A) <=
  1.25 * rel-RMS(B, A) + 0.01 -- the 4-bit P dominates this figure (about 0.11-0.14 on N(0,1)
  inputs) -- and max|out - A| <= 1.25 * max|B - A| + 0.02 * max|A|.
* LSE does not see the P rounding: max|lse - lse_A| <= 1e-3 * max(1, max|lse_A|).
"""
import math

import torch

from oracle import nvfp4_oracle as orc

LOG2E = 1.4426950408889634


def make_qkv(B, Sq, Sk, Hq, Hkv, D, seed, v_std=1.0, outlier_frac=0.0, device="cpu"):
    """bf16 N(0,1) operands in the reference layout (B,S,H,D), as the benchmark configs draw them;
    ``outlier_frac`` of the channels of q and k are multiplied by 20 (long-context config)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Sq, Hq, D, generator=g)
    k = torch.randn(B, Sk, Hkv, D, generator=g)
    v = torch.randn(B, Sk, Hkv, D, generator=g) * v_std
    if outlier_frac > 0:
        n = max(1, int(round(outlier_frac * D)))
        for t in (q, k):
            idx = torch.randperm(D, generator=g)[:n]
            t[..., idx] *= 20.0
    return tuple(t.bfloat16().to(device) for t in (q, k, v))


def p_scale_rule_of_the_64_key_kernel() -> str:
    """The P block-scale rule the loaded library's 64-key kernel was built with (a compile-time
    choice the library reports: fa4_nvfp4_query(102))."""
    import flash_attention_b200 as fa
    return "e4m3" if fa.lib().fa4_nvfp4_query(102) == 1 else "pow2"


def kernel_model(D, num_splits=1, window=(None, None), sink=None, variant=0, softcap=0.0, rows=None):
    """Which kernel the library's automatic choice runs, as oracle B keywords: the decode kernel
    for a handful of query rows, the 64-key kernel for every other call that does not split the
    keys (windows, sinks, the soft cap and KV-cache views included), the 128-key kernel for split
    calls (mirrors validate_fwd in csrc/api.cu).  ``variant`` 1 / 2 force the 128-key model, 3 the
    64-key one, 4 the decode kernel's."""
    plain = num_splits == 1
    # decode / append shapes: the transposed kernel, 128-key steps upwards, any number of splits
    decode_ok = (D == 128 and rows is not None and rows <= 32 and window in ((None, None), (None, 0))
                 and sink is None and not softcap)
    if variant == 4 or (variant == 0 and decode_ok):
        return {"step_keys": 128, "ascending": True}
    if variant == 3 or (variant == 0 and plain):
        return {"step_keys": 64, "ascending": True, "p_scale": p_scale_rule_of_the_64_key_kernel()}
    return {"step_keys": 128, "ascending": False}


def oracles(Q, K, V, causal, softmax_scale=None, num_splits=1, window=(None, None), sink=None, variant=0,
            softcap=0.0):
    """Q, K, V: NVFP4Tensor with linear scales.  Returns (out_a, lse_a, out_b, lse_b) on CPU;
    oracle B models the kernel that ``variant`` (0 = automatic) selects for this problem."""
    qd, kd, vd = Q.dequantize().cpu(), K.dequantize().cpu(), V.dequantize().cpu()
    vd = vd[:, :kd.shape[1]]            # V's key axis carries zero padding to a multiple of 32
    D = qd.shape[-1]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    oa, la = orc.attention_oracle_a(qd, kd, vd, causal=causal, softmax_scale=scale, window=window, sink=sink,
                                    softcap=softcap)
    sl2 = float(torch.tensor(scale, dtype=torch.float32) * torch.tensor(Q.scale, dtype=torch.float32)
                * torch.tensor(K.scale, dtype=torch.float32) * torch.tensor(LOG2E, dtype=torch.float32))
    c1 = 0.0
    if softcap:
        # the kernel caps the raw products: tanh(raw * c1), then works in units of softcap * log2(e)
        c1 = float(torch.tensor(scale, dtype=torch.float32) * torch.tensor(Q.scale, dtype=torch.float32)
                   * torch.tensor(K.scale, dtype=torch.float32) / torch.tensor(softcap, dtype=torch.float32))
        sl2 = float(torch.tensor(softcap, dtype=torch.float32) * torch.tensor(LOG2E, dtype=torch.float32))
    ob, lb = orc.attention_oracle_b(qd / Q.scale, kd / K.scale, vd / V.scale, sl2, V.scale, causal=causal,
                                    num_splits=num_splits, window=window, sink=sink,
                                    softcap_c1=c1,
                                    **kernel_model(D, num_splits, window, sink, variant, softcap,
                                                   rows=qd.shape[1] * (qd.shape[2] // kd.shape[2])
                                                   if vd.shape[-1] == D else None))
    return oa, la, ob, lb


def assert_parity(out, lse, oa, la, ob, lb):
    out, lse = out.float().cpu(), lse.float().cpu()
    assert not torch.isnan(out).any() and not torch.isnan(lse).any()
    # vs oracle B
    bf16_err = (ob.bfloat16().float() - ob).abs().max().item()
    atol_b = 2.0 ** -7 * ob.abs().max().item()
    eb = orc.error_metrics(out, ob)
    assert eb["max_abs"] <= 2 * bf16_err + atol_b, (eb, bf16_err, atol_b)
    assert eb["rel_rms"] <= 0.01, eb
    # vs oracle A
    ea, eba = orc.error_metrics(out, oa), orc.error_metrics(ob, oa)
    assert ea["rel_rms"] <= 1.25 * eba["rel_rms"] + 0.01, (ea, eba)
    assert ea["max_abs"] <= 1.25 * eba["max_abs"] + 0.02 * oa.abs().max().item(), (ea, eba)
    # LSE, including the -inf pattern of rows that see no key
    assert torch.equal(torch.isinf(lse), torch.isinf(la))
    el = orc.error_metrics(lse, la)
    fin = la[torch.isfinite(la)]
    assert el["max_abs"] <= 1e-3 * max(1.0, fin.abs().max().item() if fin.numel() else 1.0), el
    return {"vs_b": eb, "vs_a": ea, "b_vs_a": eba, "lse": el}
