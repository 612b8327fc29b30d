"""CPU tests of the oracle: number formats against known answers, the attention restatement
against golden vectors produced by the reference's attention_ref (tests/golden/make_golden.py)."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_e2m1_known_answers():
    # every representable value round-trips; ties go to the even code; saturation at 6
    vals = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], dtype=np.float32)
    for sgn in (1, -1):
        assert np.array_equal(orc.e2m1_decode(orc.e2m1_encode(sgn * vals)), sgn * vals)
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    assert np.array_equal(orc.e2m1_decode(orc.e2m1_encode(ties)), [0, 1, 1, 2, 2, 4, 4])
    assert np.array_equal(orc.e2m1_decode(orc.e2m1_encode(np.array([7.0, 100.0, -9.0], dtype=np.float32))),
                          [6, 6, -6])
    # bit patterns: sign is bit 3, magnitude codes in value order
    assert np.array_equal(orc.e2m1_encode(np.array([0.5, 6.0, -1.0], dtype=np.float32)), [1, 7, 0b1010])
    # matches torch's own float4 table if this torch exposes it through float8 rounding of exact values
    assert np.array_equal(orc.pack_nibbles(np.array([[1, 2, 3, 4]], dtype=np.uint8)), [[0x21, 0x43]])
    assert np.array_equal(orc.unpack_nibbles(np.array([[0x21, 0x43]], dtype=np.uint8)), [[1, 2, 3, 4]])


def test_e4m3_known_answers():
    x = np.array([0.0, 2.0 ** -9, 2.0 ** -6, 1.0, 1.125, 448.0, 1000.0], dtype=np.float32)
    b = orc.e4m3_encode(x)
    assert np.array_equal(b, [0x00, 0x01, 0x08, 0x38, 0x39, 0x7E, 0x7E])
    assert np.array_equal(orc.e4m3_decode(b)[:6], x[:6])


def test_quantize_roundtrip_and_format():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 40, 128)).astype(np.float32)
    q = orc.quantize_nvfp4(x)
    assert q.data.shape == (3, 40, 64) and q.sf.shape == (3, 40, 8)
    assert abs(q.scale - np.abs(x).max() / (6 * 448)) < 1e-9
    xd = orc.dequantize_nvfp4(q)
    # idempotence: quantising the dequantised tensor with the same scales changes nothing
    q2 = orc.quantize_nvfp4(xd)
    assert np.array_equal(orc.dequantize_nvfp4(q2), xd) or np.allclose(orc.dequantize_nvfp4(q2), xd, rtol=0, atol=0)
    rel = np.linalg.norm(xd - x) / np.linalg.norm(x)
    assert 0.05 < rel < 0.12            # 4-bit rounding: about 0.09 on N(0,1)
    # all-zero block and all-zero tensor
    z = np.zeros((2, 32), dtype=np.float32)
    qz = orc.quantize_nvfp4(z)
    assert not np.any(orc.dequantize_nvfp4(qz)) and qz.scale == 1.0


def test_sf_tiled_layout():
    rows, cols = 200, 6
    sf = np.arange(rows * cols, dtype=np.uint32).reshape(rows, cols)
    sf8 = (sf % 251).astype(np.uint8)
    t = orc.sf_linear_to_tiled(sf8)
    assert t.shape == (2, 2, 512)
    for r, c in [(0, 0), (31, 3), (32, 0), (127, 3), (128, 4), (199, 5)]:
        tile = t[r // 128, c // 4]
        rr, cc = r % 128, c % 4
        assert tile[(rr % 32) * 16 + (rr // 32) * 4 + cc] == sf8[r, c]
    assert t[1, 0][(100 % 32) * 16 + (100 // 32) * 4] == 0      # row 228 is padding


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "*.npz"))))
def test_oracle_a_matches_reference_golden(path):
    z = np.load(path)
    Q = orc.NVFP4(z["q_data"], z["q_sf"], float(z["q_scale"]))
    K = orc.NVFP4(z["k_data"], z["k_sf"], float(z["k_scale"]))
    V = orc.NVFP4(z["v_data"], z["v_sf"], float(z["v_scale"]))
    qd = torch.from_numpy(orc.dequantize_nvfp4(Q))
    kd = torch.from_numpy(orc.dequantize_nvfp4(K))
    vd = torch.from_numpy(np.ascontiguousarray(np.transpose(orc.dequantize_nvfp4(V), (0, 3, 1, 2))))
    window = tuple(None if int(x) < 0 else int(x) for x in z["window"]) if "window" in z else (None, None)
    sink = z["sink"] if "sink" in z and z["sink"].size else None
    softcap = float(z["softcap"]) if "softcap" in z.files else 0.0
    out, lse = orc.attention_oracle_a(qd, kd, vd, causal=bool(z["causal"]), window=window, sink=sink,
                                      softcap=softcap)
    ref_out, ref_lse = torch.from_numpy(z["out_ref"]), torch.from_numpy(z["lse_ref"])
    assert out.shape == ref_out.shape and lse.shape == ref_lse.shape
    assert torch.allclose(out, ref_out, rtol=1e-5, atol=1e-6)
    assert torch.equal(torch.isinf(lse), torch.isinf(ref_lse))
    fin = torch.isfinite(ref_lse)
    assert torch.allclose(lse[fin], ref_lse[fin], rtol=1e-5, atol=1e-5)


def test_golden_fixtures_present():
    assert len(glob.glob(os.path.join(GOLDEN, "*.npz"))) >= 8


def test_oracle_b_close_to_a():
    """The kernel model differs from exact attention only by the 4-bit P: bounded, and the LSE
    (which never sees P's rounding) agrees to fp32 accuracy."""
    from tests.helpers import make_qkv
    q, k, v = make_qkv(1, 256, 256, 2, 1, 128, seed=0)
    Q, K = orc.quantize_nvfp4(q.float().numpy()), orc.quantize_nvfp4(k.float().numpy())
    V = orc.quantize_nvfp4(np.ascontiguousarray(v.float().permute(0, 2, 3, 1).numpy()))
    qd, kd = torch.from_numpy(orc.dequantize_nvfp4(Q)), torch.from_numpy(orc.dequantize_nvfp4(K))
    vd = torch.from_numpy(orc.dequantize_nvfp4(V)).permute(0, 3, 1, 2).contiguous()
    for causal in (False, True):
        oa, la = orc.attention_oracle_a(qd, kd, vd, causal=causal)
        sl2 = (128 ** -0.5) * Q.scale * K.scale * 1.4426950408889634
        ob, lb = orc.attention_oracle_b(qd / Q.scale, kd / K.scale, vd / V.scale, sl2, V.scale, causal=causal)
        e = orc.error_metrics(ob, oa)
        assert e["rel_rms"] < 0.2, e
        assert orc.error_metrics(lb, la)["max_abs"] < 1e-4
        # the model of the 64-key kernel (steps of 64 keys, ascending): another rounding of P under
        # other reference maxima, the same distance from exact attention and the same LSE
        o64, l64 = orc.attention_oracle_b(qd / Q.scale, kd / K.scale, vd / V.scale, sl2, V.scale, causal=causal,
                                          step_keys=64, ascending=True)
        e64 = orc.error_metrics(o64, oa)
        assert abs(e64["rel_rms"] - e["rel_rms"]) < 0.03, (e64, e)
        assert orc.error_metrics(l64, la)["max_abs"] < 1e-4
        assert not torch.equal(o64, ob)


def test_flops_formula():
    # the benchmark configurations' FLOP counts
    assert orc.attention_flops(1, 256, 256, 4, 128, 128, False) == pytest.approx(1.342e8, rel=1e-3)
    assert orc.attention_flops(4, 4096, 4096, 32, 128, 128, False) == pytest.approx(1.0995e12, rel=1e-4)
    assert orc.attention_flops(4, 8192, 8192, 32, 128, 128, True) == pytest.approx(2.1990e12, rel=1e-4)
