"""GPU parity tests: every call goes through the C ABI (ctypes) of libfa4_nvfp4.so.

Small cases are checked against the CPU oracle (model B tightly, exact attention A within the
stated tolerance, tests/helpers.py); full-size cases through properties that need no oracle."""
import ctypes

import numpy as np
import pytest
import torch

import flash_attention_b200 as fa
from oracle import nvfp4_oracle as orc
from tests.helpers import assert_parity, make_qkv, oracles, p_scale_rule_of_the_64_key_kernel

pytestmark = pytest.mark.gpu

VARIANTS = [fa.VARIANT_WS, fa.VARIANT_WS64]


def run(Q, K, V, causal, variant=fa.VARIANT_AUTO, **kw):
    out, lse = fa.flash_attn_fp4_func(Q.data, K.data, V.data, Q.sf, K.sf, V.sf, Q.scale, K.scale,
                                      V.scale, causal=causal, return_lse=True, variant=variant,
                                      sf_layout="tiled" if Q.tiled else "linear", **kw)
    torch.cuda.synchronize()
    fa.check_status(out.device)
    return out, lse


def test_library_is_the_cuda_path(cuda_device):
    assert fa.lib().fa4_nvfp4_query(0) == 1


def test_qk_tile_probe_pins_descriptor_and_scale_layout(cuda_device):
    """One block-scaled 128x128x128 tile against the CPU product of the dequantised operands:
    pins the shared-memory swizzle, the matrix / instruction descriptors and the scale-factor
    chunk layout, for TMA-staged (mode 0) and store-staged (mode 1) operands."""
    rng = np.random.default_rng(0)
    Q = orc.quantize_nvfp4(rng.standard_normal((128, 128)).astype(np.float32))
    K = orc.quantize_nvfp4(rng.standard_normal((128, 128)).astype(np.float32))
    ref = (orc.dequantize_nvfp4(Q) / np.float32(Q.scale)).astype(np.float64) @ \
          (orc.dequantize_nvfp4(K) / np.float32(K.scale)).astype(np.float64).T
    dev = cuda_device
    tq, tk = torch.from_numpy(Q.data).to(dev), torch.from_numpy(K.data).to(dev)
    tqs = torch.from_numpy(orc.sf_linear_to_tiled(Q.sf).reshape(-1)).to(dev)
    tks = torch.from_numpy(orc.sf_linear_to_tiled(K.sf).reshape(-1)).to(dev)
    for mode in (0, 1):
        s = torch.full((128, 128), float("nan"), device=dev)
        st = torch.zeros(1, dtype=torch.int32, device=dev)
        rc = fa.lib().fa4_nvfp4_debug_qk_tile(tq.data_ptr(), tk.data_ptr(), tqs.data_ptr(), tks.data_ptr(),
                                              s.data_ptr(), 128, mode, st.data_ptr(), None)
        torch.cuda.synchronize()
        assert rc == 0 and int(st.item()) == 0
        got = s.cpu().numpy().astype(np.float64)
        assert np.abs(got - ref).max() <= 1e-5 * np.abs(ref).max()


def test_bounded_wait_gives_up_and_reports(cuda_device):
    """A wait on a barrier nothing arrives at returns after its limit with a status word; the
    context stays usable."""
    st = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    rc = fa.lib().fa4_nvfp4_debug_wait_expiry(st.data_ptr(), 5_000_000, None)
    torch.cuda.synchronize()
    assert rc == 0
    v = int(st.item()) & 0xFFFFFFFF
    assert v >> 24 == 1 and (v >> 16) & 0xFF == 99
    assert float(torch.ones(4, device=cuda_device).sum()) == 4.0


def test_mma_rate_probe_runs_and_is_plausible(cuda_device):
    # 148 SMs x 32768 FLOP/clk at ~1.9 GHz is ~9 PFLOP/s; anything from a quarter of that up to a
    # little above it is a sane reading, and 128x128x64 cannot retire faster than 64 clk.
    r = fa.measure_fp4_mma_rate(iters=1 << 14, device=cuda_device)
    assert r["sms"] >= 1 and r["clk_per_mma"] >= 60.0
    assert 2000.0 < r["tflops"] * 148 / r["sms"] < 11000.0
    assert lib_rc_rejects_bad_iters()


def lib_rc_rejects_bad_iters():
    return fa.lib().fa4_nvfp4_debug_mma_rate(3, 1, 1, None, None) < 0


def test_sf_linear_to_tiled_bit_exact(cuda_device):
    rng = np.random.default_rng(3)
    for shape, rows_dim, head_dim, mult in [((2, 300, 3, 8), 1, 2, 1), ((1, 2, 128, 40), 2, 1, 1),
                                            ((1, 5, 1, 3), 1, 2, 1), ((1, 2, 128, 10), 2, 1, 2)]:
        sf = rng.integers(0, 255, size=shape, dtype=np.uint8)
        got = fa.sf_to_tiled(torch.from_numpy(sf).to(cuda_device), rows_dim, head_dim, mult).cpu().numpy()
        lin = sf if rows_dim == 2 else np.transpose(sf, (0, 2, 1, 3))
        assert np.array_equal(got, orc.sf_linear_to_tiled(lin, mult))
    # strided (non-contiguous) source
    big = torch.from_numpy(rng.integers(0, 255, size=(2, 256, 6, 8), dtype=np.uint8)).to(cuda_device)
    view = big[:, :, 2:4]
    assert torch.equal(fa.sf_to_tiled(view, 1, 2), fa.sf_to_tiled(view.contiguous(), 1, 2))


CASES = [
    # name, B, Sq, Sk, Hq, Hkv, causal, v_std, outliers
    ("cfg0_cpu_reference_case", 1, 256, 256, 4, 4, False, 1.0, 0.0),
    ("causal_gqa", 1, 384, 384, 4, 2, True, 0.5, 0.0),
    ("causal_sq_lt_sk", 1, 128, 384, 2, 1, True, 1.0, 0.0),
    ("causal_sq_gt_sk_masked_rows", 1, 384, 128, 2, 2, True, 1.0, 0.0),
    ("noncausal_sq_ne_sk_batch", 2, 128, 512, 2, 2, False, 1.0, 0.0),
    ("mqa_outlier_channels", 1, 256, 256, 8, 1, True, 1.0, 0.01),
    # partial last tiles: Sq free, Sk a multiple of 32 (the reference's ragged shapes,
    # tests/cute/test_flash_attn.py:91-119, restricted to what 16-key scale blocks allow)
    ("ragged_noncausal", 2, 113, 224, 3, 1, False, 1.0, 0.0),
    ("ragged_causal_sq_lt_sk", 1, 200, 352, 4, 2, True, 1.0, 0.0),
    ("ragged_causal_sq_gt_sk", 1, 300, 160, 2, 2, True, 1.0, 0.0),
    ("single_query_row", 1, 1, 160, 2, 1, True, 1.0, 0.0),
    # any Sk, as in the reference (tests/cute/test_flash_attn.py:91-119): keys that do not fill a
    # 16-key scale block, Sq and Sk odd
    ("ragged_sk_203_noncausal", 1, 113, 203, 3, 1, False, 1.0, 0.0),
    ("ragged_sk_799_causal", 1, 800, 799, 2, 2, True, 1.0, 0.0),
    ("ragged_sk_1_causal", 2, 1, 1, 2, 1, True, 1.0, 0.0),
]


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_parity_with_oracle(cuda_device, case, variant):
    _, B, Sq, Sk, Hq, Hkv, causal, v_std, outl = case
    q, k, v = make_qkv(B, Sq, Sk, Hq, Hkv, 128, seed=0, v_std=v_std, outlier_frac=outl, device=cuda_device)
    Q, K, V = fa.quantize_qkv(q, k, v)
    out, lse = run(Q, K, V, causal, variant)
    assert out.dtype == torch.bfloat16 and out.shape == (B, Sq, Hq, 128)
    assert lse.dtype == torch.float32 and lse.shape == (B, Hq, Sq)
    assert_parity(out, lse, *oracles(Q, K, V, causal, variant=variant))


@pytest.mark.parametrize("name", ["mha_noncausal", "gqa_causal_sq_lt_sk", "mqa_causal_sq_gt_sk",
                                  "mqa_noncausal_ragged",
                                  "gqa_sliding_window_causal",
                                  "mha_window_both_sides_sq_lt_sk", "gqa_causal_learnable_sink",
                                  "gqa_causal_softcap"])
def test_golden_fixture_through_the_kernel(cuda_device, name):
    """The fixtures generated by the reference's attention_ref, through the kernel."""
    import os
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", name + ".npz"))
    dev = cuda_device
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    window = tuple(None if int(x) < 0 else int(x) for x in z["window"])
    # the fixtures hold V with exactly Sk keys; the call takes its key axis padded with zeros to a
    # multiple of 32 (the ragged fixture has Sk = 208 -> 224)
    v_data, v_sf = z["v_data"], z["v_sf"]
    pad = (-2 * v_data.shape[-1]) % 32
    if pad:
        v_data = np.concatenate([v_data, np.zeros(v_data.shape[:-1] + (pad // 2,), np.uint8)], axis=-1)
        v_sf = np.concatenate([v_sf, np.zeros(v_sf.shape[:-1] + (pad // 16,), np.uint8)], axis=-1)
    out, lse = fa.flash_attn_fp4_func(t(z["q_data"]), t(z["k_data"]), t(v_data), t(z["q_sf"]),
                                      t(z["k_sf"]), t(v_sf), float(z["q_scale"]), float(z["k_scale"]),
                                      float(z["v_scale"]), causal=bool(z["causal"]), return_lse=True,
                                      window_size=window,
                                      learnable_sink=torch.from_numpy(z["sink"]) if z["sink"].size else None,
                                      softcap=float(z["softcap"]) if "softcap" in z.files else 0.0)
    torch.cuda.synchronize()
    fa.check_status(dev)
    ref_out, ref_lse = torch.from_numpy(z["out_ref"]), torch.from_numpy(z["lse_ref"])
    e = orc.error_metrics(out.float().cpu(), ref_out)
    assert e["rel_rms"] < 0.2, e                       # 4-bit P: about 0.13 on N(0,1) inputs
    assert torch.equal(torch.isinf(lse.cpu()), torch.isinf(ref_lse))
    assert orc.error_metrics(lse.cpu(), ref_lse)["max_abs"] < 1e-3


def test_softmax_scale_and_preallocated_outputs(cuda_device):
    q, k, v = make_qkv(1, 128, 256, 2, 2, 128, seed=7, device=cuda_device)
    Q, K, V = fa.quantize_qkv(q, k, v)
    out = torch.empty(1, 128, 2, 128, dtype=torch.bfloat16, device=cuda_device)
    lse = torch.empty(1, 2, 128, dtype=torch.float32, device=cuda_device)
    o2, l2 = run(Q, K, V, False, softmax_scale=0.05, out=out, lse=lse)
    assert o2.data_ptr() == out.data_ptr() and l2.data_ptr() == lse.data_ptr()
    assert_parity(out, lse, *oracles(Q, K, V, False, softmax_scale=0.05))
    o3, l3 = fa.flash_attn_func(Q, K, V, softmax_scale=0.05)
    assert l3 is None and torch.equal(o3, out)
    with pytest.raises(AssertionError):
        fa.flash_attn_fp4_func(Q.data, K.data, V.data, Q.sf, K.sf, V.sf, 1.0, 1.0, 1.0,
                               out=torch.empty(1, 128, 2, 64, dtype=torch.bfloat16, device=cuda_device))
    with pytest.raises(AssertionError):        # Sk = 144: V must come with its key axis padded to 160
        fa.flash_attn_fp4_func(Q.data, K.data[:, :144], V.data[..., :72].contiguous(), Q.sf, K.sf[:, :144],
                               V.sf[..., :9].contiguous(), 1.0, 1.0, 1.0)


def test_strided_views_and_tiled_scales(cuda_device):
    """Operands that are views into larger buffers (strides a multiple of 16 bytes) and scale
    factors passed already tiled give the same bits as the contiguous / linear call."""
    q, k, v = make_qkv(2, 256, 256, 4, 2, 128, seed=11, device=cuda_device)
    Q, K, V = fa.quantize_qkv(q, k, v)
    base, _ = run(Q, K, V, True)
    pad = torch.zeros(2, 256, 6, 64, dtype=torch.uint8, device=cuda_device)
    pad[:, :, 1:5] = Q.data
    Qv = fa.NVFP4Tensor(pad[:, :, 1:5], Q.sf, Q.scale)
    assert torch.equal(run(Qv, K, V, True)[0], base)
    Qt, Kt, Vt = (fa.NVFP4Tensor(t.data, t.tiled_sf(), t.scale, True, t.is_v) for t in (Q, K, V))
    assert torch.equal(run(Qt, Kt, Vt, True)[0], base)


# ---------------------------------------------------------------------------------------------
# full-size properties (no oracle needed)
# ---------------------------------------------------------------------------------------------
def _cfg(name, device):
    cfgs = {"cfg1": (4, 4096, 32, 32, False, 1.0), "cfg2": (4, 8192, 32, 8, True, 0.5)}
    B, S, Hq, Hkv, causal, v_std = cfgs[name]
    g = torch.Generator(device=device).manual_seed(0)
    q = torch.randn(B, S, Hq, 128, generator=g, device=device, dtype=torch.bfloat16)
    k = torch.randn(B, S, Hkv, 128, generator=g, device=device, dtype=torch.bfloat16)
    v = (torch.randn(B, S, Hkv, 128, generator=g, device=device) * v_std).bfloat16()
    Q, K, V = fa.quantize_qkv(q, k, v)
    del q, k, v
    Q, K, V = (fa.NVFP4Tensor(t.data, t.tiled_sf(), t.scale, True, t.is_v) for t in (Q, K, V))
    return Q, K, V, causal


@pytest.mark.parametrize("kernel", [fa.VARIANT_WS, fa.VARIANT_WS64], ids=["ws128", "ws64"])
@pytest.mark.parametrize("name", ["cfg1", "cfg2"])
def test_full_size_properties(cuda_device, name, kernel):
    Q, K, V, causal = _cfg(name, cuda_device)
    out, lse = run(Q, K, V, causal, kernel)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    # determinism: a second run gives the same bits
    out2, lse2 = run(Q, K, V, causal, kernel)
    assert torch.equal(out, out2) and torch.equal(lse, lse2)
    # the other production kernel walks the keys in other steps and the other direction and rounds
    # P under other references: two independent 4-bit roundings of the same attention (each about
    # 0.13 from the exact result), the same LSE up to fp32 summation order
    outs, lses = run(Q, K, V, causal, fa.VARIANT_WS64 if kernel == fa.VARIANT_WS else fa.VARIANT_WS)
    e = orc.error_metrics(out.float(), outs.float())
    assert e["rel_rms"] < 0.25, e
    assert (lse - lses).abs().max().item() < 1e-4
    del outs, lses, out2, lse2
    # linearity in V: doubling V's tensor scale doubles O exactly (power of two), LSE unchanged
    V2 = fa.NVFP4Tensor(V.data, V.sf, 2.0 * V.scale, True, True)
    out_v2, lse_v2 = run(Q, K, V2, causal, kernel)
    assert torch.equal(out_v2.float(), 2.0 * out.float()) and torch.equal(lse_v2, lse)
    # every output row is a convex combination of V rows: bounded by max |V|
    vmax = 6.0 * 448.0 * V.scale
    assert out.float().abs().max().item() <= vmax
    # a slice of the batch computed alone gives the same bits (what sharding relies on)
    Qs = fa.NVFP4Tensor(Q.data[1:2], Q.sf[1:2], Q.scale, True)
    Ks = fa.NVFP4Tensor(K.data[1:2], K.sf[1:2], K.scale, True)
    Vs = fa.NVFP4Tensor(V.data[1:2], V.sf[1:2], V.scale, True, True)
    o1, l1 = run(Qs, Ks, Vs, causal, kernel)
    assert torch.equal(o1, out[1:2]) and torch.equal(l1, lse[1:2])


def test_sampled_heads_of_cfg2_against_oracle(cuda_device):
    """cfg2-shaped problem (S = 8192 causal GQA), two (batch, head) pairs checked against exact
    attention on a window of query rows (the full oracle would need 34 GB of scores)."""
    Q, K, V, causal = _cfg("cfg2", cuda_device)
    out, lse = run(Q, K, V, causal)          # the automatic choice, what the benchmark times
    g = torch.Generator(device=cuda_device).manual_seed(0)
    S = 8192
    q = torch.randn(4, S, 32, 128, generator=g, device=cuda_device, dtype=torch.bfloat16)
    k = torch.randn(4, S, 8, 128, generator=g, device=cuda_device, dtype=torch.bfloat16)
    v = (torch.randn(4, S, 8, 128, generator=g, device=cuda_device) * 0.5).bfloat16()
    Ql, Kl, Vl = fa.quantize_qkv(q, k, v)
    for (b, h, r0) in [(0, 0, 0), (3, 29, 8064), (1, 13, 4000)]:
        hk = h // 4
        qd = fa.dequantize_lastdim(Ql.data[b, r0:r0 + 128, h], Ql.sf[b, r0:r0 + 128, h], Ql.scale).double()
        kd = fa.dequantize_lastdim(Kl.data[b, :, hk], Kl.sf[b, :, hk], Kl.scale).double()
        vd = fa.dequantize_lastdim(Vl.data[b, hk], Vl.sf[b, hk], Vl.scale).double().T     # (Sk, Dv)
        s = (qd @ kd.T) / 128 ** 0.5
        rows = torch.arange(r0, r0 + 128, device=cuda_device)[:, None]
        s = s.masked_fill(torch.arange(S, device=cuda_device)[None, :] > rows, float("-inf"))
        ref_l = torch.logsumexp(s, dim=-1)
        ref_o = torch.softmax(s, dim=-1) @ vd
        got_o, got_l = out[b, r0:r0 + 128, h].double(), lse[b, h, r0:r0 + 128].double()
        assert (got_l - ref_l).abs().max().item() < 1e-3
        rel = ((got_o - ref_o).norm() / ref_o.norm()).item()
        assert rel < 0.2, rel


def _check_windows(Ql, Kl, Vl, out, lse, samples, causal, softmax_scale, group):
    """Sampled (batch, head, first row) windows of 128 query rows of a full-size run against
    (A) exact attention on the dequantised operands, in fp64 on the GPU, and (B) the oracle's
    model of the 64-key kernel on the CPU.  A window of a causal Sq = Sk problem that starts at a
    multiple of 128 is itself a causal problem (128 queries, bottom-right aligned against keys
    0 .. r0 + 127) whose tile walks the same steps in the same order, so model B applies to it
    unchanged.  Tolerances: tests/helpers.py (B: two bf16 roundings + 2^-7 max, rel-RMS 0.01;
    A: 1.25 x the B-vs-A gap + 0.01; LSE 1e-3)."""
    dev = out.device
    S = Kl.data.shape[1]
    D = Ql.data.shape[-1] * 2
    for (b, h, r0) in samples:
        hk = h // group
        sk = r0 + 128 if causal else S
        qd = fa.dequantize_lastdim(Ql.data[b, r0:r0 + 128, h], Ql.sf[b, r0:r0 + 128, h], Ql.scale)
        kd = fa.dequantize_lastdim(Kl.data[b, :sk, hk], Kl.sf[b, :sk, hk], Kl.scale)
        vd = fa.dequantize_lastdim(Vl.data[b, hk, :, :sk // 2], Vl.sf[b, hk, :, :sk // 16], Vl.scale).T   # (sk, Dv)
        s = (qd.double() @ kd.double().T) * softmax_scale
        if causal:
            rows = torch.arange(r0, r0 + 128, device=dev)[:, None]
            s = s.masked_fill(torch.arange(sk, device=dev)[None, :] > rows, float("-inf"))
        la = torch.logsumexp(s, dim=-1).float().cpu()[None, None]                      # (1, 1, 128)
        oa = (torch.softmax(s, dim=-1) @ vd.double()).float().cpu()[None, :, None]     # (1, 128, 1, Dv)
        sl2 = float(torch.tensor(softmax_scale, dtype=torch.float32) * torch.tensor(Ql.scale, dtype=torch.float32)
                    * torch.tensor(Kl.scale, dtype=torch.float32) * torch.tensor(1.4426950408889634, dtype=torch.float32))
        ob, lb = orc.attention_oracle_b((qd / Ql.scale).cpu()[None, :, None], (kd / Kl.scale).cpu()[None, :, None],
                                        (vd / Vl.scale).cpu()[None, :, None], sl2, Vl.scale, causal=causal,
                                        step_keys=64, ascending=True,
                                        p_scale=p_scale_rule_of_the_64_key_kernel())
        got_o = out[b, r0:r0 + 128, h][None, :, None]
        got_l = lse[b, h, r0:r0 + 128][None, None]
        assert_parity(got_o, got_l, oa, la, ob, lb)


def test_sampled_windows_of_cfg1_against_both_oracles(cuda_device):
    """The non-causal benchmark configuration (B=4, H=32/32, S=4096, D=128) at full size: three
    (batch, head, window) samples against exact attention and against the kernel model."""
    B, S, H = 4, 4096, 32
    q, k, v = make_qkv(B, S, S, H, H, 128, seed=0, device=cuda_device)
    Ql, Kl, Vl = fa.quantize_qkv_fused(q, k, v)
    del q, k, v
    out, lse = fa.flash_attn_func(Ql, Kl, Vl, causal=False, return_lse=True)
    torch.cuda.synchronize()
    fa.check_status(cuda_device)
    _check_windows(Ql, Kl, Vl, out, lse, [(0, 0, 0), (2, 17, 2048), (3, 31, S - 128)], False, 128 ** -0.5, 1)


def test_sampled_windows_of_cfg2_against_the_kernel_model(cuda_device):
    """The causal GQA benchmark configuration (B=4, Hq=32, Hkv=8, S=8192) at full size, held to
    the tight bound against the kernel model too (first, a middle and the last tile)."""
    B, S, Hq, Hkv = 4, 8192, 32, 8
    q, k, v = make_qkv(B, S, S, Hq, Hkv, 128, seed=0, v_std=0.5, device=cuda_device)
    Ql, Kl, Vl = fa.quantize_qkv_fused(q, k, v)
    del q, k, v
    out, lse = fa.flash_attn_func(Ql, Kl, Vl, causal=True, return_lse=True)
    torch.cuda.synchronize()
    fa.check_status(cuda_device)
    _check_windows(Ql, Kl, Vl, out, lse, [(0, 0, 0), (1, 13, 3968), (3, 29, S - 128)], True, 128 ** -0.5, Hq // Hkv)


@pytest.mark.parametrize("causal", [False, True], ids=["noncausal", "causal"])
@pytest.mark.parametrize("S", [4096, 16384])
@pytest.mark.parametrize("D,Dv", [(64, 64), (128, 128), (192, 128)], ids=["d64", "d128", "d192"])
def test_sweep_shapes_at_size_against_both_oracles(cuda_device, D, Dv, S, causal):
    """The head-dim / shape sweep at its real size (B = 8, H = 16, i.e. B * H = 128): thousands of
    tiles per launch, several per CTA, the snake order over CTAs and the 32-byte-swizzled
    sub-tiles of head dims 64 and 192.  First, a middle and the last tile of sampled (batch,
    head) pairs against exact attention and the kernel model."""
    B, H = 8, 16
    g = torch.Generator(device=cuda_device).manual_seed(5)
    q, k = (torch.randn(B, S, H, D, generator=g, device=cuda_device, dtype=torch.bfloat16) for _ in range(2))
    v = torch.randn(B, S, H, Dv, generator=g, device=cuda_device, dtype=torch.bfloat16)
    Ql, Kl, Vl = fa.quantize_qkv_fused(q, k, v)
    del q, k, v
    out, lse = fa.flash_attn_func(Ql, Kl, Vl, causal=causal, return_lse=True)
    torch.cuda.synchronize()
    fa.check_status(cuda_device)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    _check_windows(Ql, Kl, Vl, out, lse, [(0, 0, 0), (5, 9, S // 2), (7, 15, S - 128)], causal, D ** -0.5, 1)


@pytest.mark.parametrize("shape", [(1, 256, 256, 4, 2, True), (2, 2048, 2048, 16, 4, True),
                                   (4, 1024, 1024, 32, 32, False)],
                         ids=["small", "causal_several_tiles_per_cta", "noncausal_several_tiles_per_cta"])
def test_a_thousand_runs_give_the_same_bits(cuda_device, shape):
    """The reference's race / determinism loop (tests/cute/test_flash_attn_race_condition.py:310-344:
    re-run 1000 times, torch.equal against the first result), on one small problem and on problems
    with several tiles per CTA, where a missed barrier phase or a slot reused too early would show
    as a changed bit sooner or later.  Differences are accumulated on the device and read once."""
    B, Sq, Sk, Hq, Hkv, causal = shape
    q, k, v = make_qkv(B, Sq, Sk, Hq, Hkv, 128, seed=31, device=cuda_device)
    Q, K, V = fa.quantize_qkv_fused(q, k, v, linear_sf=False)
    out0, lse0 = run(Q, K, V, causal)
    out = torch.empty_like(out0)
    lse = torch.empty_like(lse0)
    bad = torch.zeros((), dtype=torch.int64, device=cuda_device)
    for _ in range(1000):
        fa.flash_attn_fp4_func(Q.data, K.data, V.data, Q.sf, K.sf, V.sf, Q.scale, K.scale, V.scale,
                               causal=causal, return_lse=True, sf_layout="tiled", out=out, lse=lse)
        bad += (out.view(torch.int16) != out0.view(torch.int16)).sum() + \
               (lse.view(torch.int32) != lse0.view(torch.int32)).sum()
        out.zero_()
    torch.cuda.synchronize()
    fa.check_status(cuda_device)
    assert int(bad.item()) == 0


@pytest.mark.parametrize("causal", [False, True])
def test_host_pipeline_matches_the_single_call_bit_for_bit(cuda_device, causal):
    B, S, Hq, Hkv = 2, 640, 4, 2
    q, k, v = make_qkv(B, S, S, Hq, Hkv, 128, seed=21, device=cuda_device)
    Q, K, V = fa.quantize_qkv(q, k, v)
    dev_ops = [t.to(cuda_device) for t in (Q.data, K.data, V.data, Q.sf, K.sf, V.sf)]
    want_o, want_l = fa.flash_attn_fp4_func(*dev_ops, Q.scale, K.scale, V.scale, causal=causal, return_lse=True)
    host_ops = [t.cpu().pin_memory() for t in (Q.data, K.data, V.data, Q.sf, K.sf, V.sf)]
    pipe = fa.HostPipeline(B, S, S, Hq, Hkv, device=cuda_device, row_chunks=3)
    assert len(pipe.ranges) == 3 and pipe.ranges[-1][1] == S
    out_h = torch.zeros(B, S, Hq, 128, dtype=torch.bfloat16).pin_memory()
    lse_h = torch.zeros(B, Hq, S, dtype=torch.float32).pin_memory()
    for _ in range(2):                      # the second run reuses the staging buffers
        pipe.run(*host_ops, Q.scale, K.scale, V.scale, out_h, lse_h, causal=causal)
    pipe.wait()
    assert torch.equal(out_h, want_o.cpu()) and torch.equal(lse_h, want_l.cpu())
    o2, l2 = fa.flash_attn_fp4_host(*host_ops, Q.scale, K.scale, V.scale, causal=causal, device=cuda_device)
    assert torch.equal(o2, want_o.cpu()) and torch.equal(l2, want_l.cpu())


def test_long_context_outlier_config_sampled_rows_and_head_split(cuda_device):
    """cfg3-shaped problem: B=1, Hq=64, Hkv=8, S=32768 causal, 1 % of the q/k channels x20.
    Sampled query rows against exact attention on the dequantised operands; one kv head (with its
    8 query heads) computed alone gives the same bits as inside the full call (the 8-way head
    split of the multi-GPU run)."""
    S, Hq, Hkv = 32768, 64, 8
    q, k, v = make_qkv(1, S, S, Hq, Hkv, 128, seed=3, outlier_frac=0.01, device=cuda_device)
    Ql, Kl, Vl = fa.quantize_qkv_fused(q, k, v)
    del q, k, v
    out, lse = fa.flash_attn_func(Ql, Kl, Vl, causal=True, return_lse=True)
    fa.check_status(cuda_device)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    for (h, r0) in [(0, 0), (37, 16384), (63, S - 128)]:
        hk = h // (Hq // Hkv)
        qd = fa.dequantize_lastdim(Ql.data[0, r0:r0 + 128, h], Ql.sf[0, r0:r0 + 128, h], Ql.scale).double()
        kd = fa.dequantize_lastdim(Kl.data[0, :, hk], Kl.sf[0, :, hk], Kl.scale).double()
        vd = fa.dequantize_lastdim(Vl.data[0, hk], Vl.sf[0, hk], Vl.scale).double().T
        s = (qd @ kd.T) / 128 ** 0.5
        rows = torch.arange(r0, r0 + 128, device=cuda_device)[:, None]
        s = s.masked_fill(torch.arange(S, device=cuda_device)[None, :] > rows, float("-inf"))
        ref_l = torch.logsumexp(s, dim=-1)
        ref_o = torch.softmax(s, dim=-1) @ vd
        got_o, got_l = out[0, r0:r0 + 128, h].double(), lse[0, h, r0:r0 + 128].double()
        assert ((got_l - ref_l).abs() / ref_l.abs().clamp(min=1.0)).max().item() < 1e-3
        rel = ((got_o - ref_o).norm() / ref_o.norm()).item()
        assert rel < 0.25, rel          # the 4-bit P: 0.11 - 0.14 on the other configurations
    # kv head 5 with its query heads 40..47, alone
    g0, g1 = 5 * (Hq // Hkv), 6 * (Hq // Hkv)
    Qs = fa.NVFP4Tensor(Ql.data[:, :, g0:g1], Ql.sf[:, :, g0:g1], Ql.scale)
    Ks = fa.NVFP4Tensor(Kl.data[:, :, 5:6], Kl.sf[:, :, 5:6], Kl.scale)
    Vs = fa.NVFP4Tensor(Vl.data[:, 5:6], Vl.sf[:, 5:6], Vl.scale, is_v=True)
    o1, l1 = fa.flash_attn_func(Qs, Ks, Vs, causal=True, return_lse=True)
    assert torch.equal(o1, out[:, :, g0:g1]) and torch.equal(l1, lse[:, g0:g1])


CASES_D64 = [
    # name, B, Sq, Sk, Hq, Hkv, causal
    ("d64_noncausal", 1, 256, 256, 4, 4, False),
    ("d64_causal_gqa", 2, 384, 384, 4, 2, True),
    ("d64_causal_sq_gt_sk_masked_rows", 1, 384, 128, 2, 2, True),
    ("d64_ragged_causal_sq_lt_sk", 1, 200, 352, 4, 1, True),
]


@pytest.mark.parametrize("case", CASES_D64, ids=[c[0] for c in CASES_D64])
def test_parity_with_oracle_head_dim_64(cuda_device, case):
    """Head dim 64 (the sweep configuration): one 64-element step of Q K^T on 32-byte-swizzled
    tiles, 64 output columns.  Both quantisers feed it."""
    _, B, Sq, Sk, Hq, Hkv, causal = case
    q, k, v = make_qkv(B, Sq, Sk, Hq, Hkv, 64, seed=5, device=cuda_device)
    Q, K, V = fa.quantize_qkv(q, k, v)
    for variant in (fa.VARIANT_AUTO, fa.VARIANT_WS, fa.VARIANT_WS64):   # both kernels build head dim 64
        out, lse = run(Q, K, V, causal, variant)
        assert out.dtype == torch.bfloat16 and out.shape == (B, Sq, Hq, 64)
        assert_parity(out, lse, *oracles(Q, K, V, causal, variant=variant))
    if Sk % 16 == 0:
        Qf, Kf, Vf = fa.quantize_qkv_fused(q, k, v)
        out_f, lse_f = fa.flash_attn_func(Qf, Kf, Vf, causal=causal, return_lse=True)
        assert_parity(out_f, lse_f, *oracles(Qf, Kf, Vf, causal))
    with pytest.raises(ValueError):                 # the retired bring-up variant's number
        run(Q, K, V, causal, 1)


@pytest.mark.parametrize("case", [
    # name, B, Sq, Sk, Hq, Hkv, causal
    ("d192_noncausal", 1, 256, 384, 2, 2, False),
    ("d192_causal_gqa", 2, 384, 384, 4, 2, True),
    ("d192_ragged_causal_sq_lt_sk", 1, 200, 352, 4, 1, True),
    ("d192_masked_rows", 1, 300, 160, 2, 2, True),
], ids=lambda c: c[0])
def test_parity_with_oracle_head_dim_192_128(cuda_device, case):
    """Q / K head dim 192 with V / O head dim 128 (the reference's only pair above 128,
    interface.py:84-99): three 64-element steps of Q K^T on 32-byte-wide sub-tiles, 64-key kernel
    only.  Both quantisers feed it; features of the 128-key kernel are refused for this shape."""
    _, B, Sq, Sk, Hq, Hkv, causal = case
    g = torch.Generator().manual_seed(17)
    q = torch.randn(B, Sq, Hq, 192, generator=g).bfloat16().to(cuda_device)
    k = torch.randn(B, Sk, Hkv, 192, generator=g).bfloat16().to(cuda_device)
    v = torch.randn(B, Sk, Hkv, 128, generator=g).bfloat16().to(cuda_device)
    Q, K, V = fa.quantize_qkv(q, k, v)
    out, lse = run(Q, K, V, causal)
    assert out.dtype == torch.bfloat16 and out.shape == (B, Sq, Hq, 128)
    assert_parity(out, lse, *oracles(Q, K, V, causal))
    if Sk % 16 == 0:
        Qf, Kf, Vf = fa.quantize_qkv_fused(q, k, v)
        out_f, lse_f = fa.flash_attn_func(Qf, Kf, Vf, causal=causal, return_lse=True)
        assert_parity(out_f, lse_f, *oracles(Qf, Kf, Vf, causal))
    for kw in ({"variant": fa.VARIANT_WS}, {"num_splits": 2}):
        with pytest.raises((ValueError, NotImplementedError)):
            run(Q, K, V, causal, **kw)
    # sinks, the soft cap and (when asked for explicitly) windows are features of the 64-key kernel
    sink = torch.linspace(-1.0, 1.0, Hq)
    out_s, lse_s = run(Q, K, V, causal, learnable_sink=sink)
    assert_parity(out_s, lse_s, *oracles(Q, K, V, causal, sink=sink.numpy()))
    out_w, lse_w = run(Q, K, V, causal, fa.VARIANT_WS64, window_size=(96, None if not causal else 0))
    assert_parity(out_w, lse_w, *oracles(Q, K, V, causal, window=(96, None), variant=fa.VARIANT_WS64))


CASES_SPLIT = [
    # name, B, Sq, Sk, Hq, Hkv, D, causal, splits
    ("decode_one_row", 2, 1, 2048, 8, 2, 128, True, 4),
    ("decode_17_rows_noncausal", 1, 17, 1536, 4, 4, 128, False, 3),
    ("short_prefill_causal", 1, 128, 2048, 4, 1, 128, True, 8),
    ("more_splits_than_blocks", 1, 64, 384, 2, 2, 128, False, 5),
    ("two_tiles_sq_gt_sk_masked_rows", 1, 384, 256, 2, 2, 128, True, 2),
    ("d64_decode", 2, 8, 1024, 4, 2, 64, True, 4),
]


@pytest.mark.parametrize("case", CASES_SPLIT, ids=[c[0] for c in CASES_SPLIT])
def test_split_kv_parity(cuda_device, case):
    _, B, Sq, Sk, Hq, Hkv, D, causal, splits = case
    q, k, v = make_qkv(B, Sq, Sk, Hq, Hkv, D, seed=9, device=cuda_device)
    Q, K, V = fa.quantize_qkv(q, k, v)
    out, lse = run(Q, K, V, causal, fa.VARIANT_WS, num_splits=splits)
    assert out.shape == (B, Sq, Hq, D) and lse.shape == (B, Hq, Sq)
    assert_parity(out, lse, *oracles(Q, K, V, causal, num_splits=splits, variant=fa.VARIANT_WS))
    # the un-split result agrees to within the 4-bit P noise of two different groupings
    out1, lse1 = run(Q, K, V, causal, fa.VARIANT_WS)
    fin = torch.isfinite(lse1)
    assert torch.equal(fin, torch.isfinite(lse))
    assert (lse[fin] - lse1[fin]).abs().max().item() < 1e-3
    e = orc.error_metrics(out.float(), out1.float())
    assert e["rel_rms"] < 0.2, e
    with pytest.raises((ValueError, NotImplementedError)):      # the 64-key kernel does not split
        run(Q, K, V, causal, fa.VARIANT_WS64, num_splits=splits)


def test_split_kv_heuristic_and_surface(cuda_device):
    assert fa.interface.choose_num_splits(4, 8192, 8192, 32, True, cuda_device) == 1
    n = fa.interface.choose_num_splits(1, 1, 32768, 8, True, cuda_device)
    assert 8 <= n <= 64
    q, k, v = make_qkv(1, 4, 4096, 8, 2, 128, seed=1, device=cuda_device)
    Q, K, V = fa.quantize_qkv(q, k, v)
    # 4 rows x 4 query heads per kv head = 16 rows: the automatic choice is the decode kernel
    o0, l0 = fa.flash_attn_func(Q, K, V, causal=True, return_lse=True, num_splits=0)
    n_dec = fa.interface.choose_decode_splits(1, 2, 4096, cuda_device)
    assert 2 <= n_dec <= 16
    assert_parity(o0, l0, *oracles(Q, K, V, True, num_splits=n_dec))
    # the prefill kernel's split heuristic, on the same problem
    o1, l1 = run(Q, K, V, True, fa.VARIANT_WS, num_splits=0)
    assert_parity(o1, l1, *oracles(Q, K, V, True, variant=fa.VARIANT_WS,
                                   num_splits=fa.interface.choose_num_splits(1, 4, 4096, 8, True, cuda_device)))


CASES_WINDOW = [
    # name, B, Sq, Sk, Hq, Hkv, D, causal, window, splits
    ("sliding_causal", 1, 640, 640, 4, 2, 128, True, (200, None), 1),
    ("sliding_causal_small_window", 2, 384, 384, 2, 2, 128, True, (17, None), 1),
    ("both_sides_noncausal", 1, 384, 512, 2, 1, 128, False, (150, 90), 1),
    ("right_only", 1, 256, 384, 2, 2, 128, False, (None, 64), 1),
    ("left_only_ragged", 1, 200, 352, 4, 2, 128, False, (130, None), 1),
    ("window_wider_than_sequence", 1, 256, 256, 2, 2, 128, True, (1000, None), 1),
    ("sliding_causal_sq_gt_sk_masked_rows", 1, 384, 128, 2, 2, 128, True, (64, None), 1),
    ("sliding_causal_d64", 1, 384, 384, 4, 2, 64, True, (128, None), 1),
    ("sliding_with_splits", 1, 128, 2048, 4, 1, 128, True, (900, None), 3),
]


@pytest.mark.parametrize("case", CASES_WINDOW, ids=[c[0] for c in CASES_WINDOW])
def test_local_attention_parity(cuda_device, case):
    """Sliding-window attention (window_size of the reference's flash_attn_func)."""
    _, B, Sq, Sk, Hq, Hkv, D, causal, window, splits = case
    q, k, v = make_qkv(B, Sq, Sk, Hq, Hkv, D, seed=13, device=cuda_device)
    Q, K, V = fa.quantize_qkv(q, k, v)
    out, lse = fa.flash_attn_func(Q, K, V, causal=causal, window_size=window, return_lse=True,
                                  num_splits=splits)
    torch.cuda.synchronize()
    fa.check_status(cuda_device)
    w = (window[0], 0) if causal else window
    assert_parity(out, lse, *oracles(Q, K, V, causal, num_splits=splits, window=w))


@pytest.mark.parametrize("splits", [1, 3])
def test_learnable_sink_parity(cuda_device, splits):
    """Sink logits join the normalisation and the LSE; rows without keys get LSE = sink, O = 0."""
    B, Sq, Sk, Hq, Hkv = 1, 384, 256, 4, 2            # causal with Sq > Sk: 128 rows see no key
    q, k, v = make_qkv(B, Sq, Sk, Hq, Hkv, 128, seed=17, device=cuda_device)
    Q, K, V = fa.quantize_qkv(q, k, v)
    sink = torch.tensor([0.5, -3.0, 4.0, 0.0])
    out, lse = fa.flash_attn_func(Q, K, V, causal=True, return_lse=True, learnable_sink=sink.to(cuda_device),
                                  num_splits=splits)
    torch.cuda.synchronize()
    fa.check_status(cuda_device)
    assert_parity(out, lse, *oracles(Q, K, V, True, num_splits=splits, sink=sink.numpy()))
    assert torch.equal(lse[0, :, :128].cpu(), sink[:, None].expand(4, 128))
    assert out[0, :128].abs().max().item() == 0.0


@pytest.mark.parametrize("case", [
    # name, B, Sq, Sk, Hq, Hkv, D, causal, softcap, splits, window
    ("softcap_causal_gqa", 1, 384, 384, 4, 2, 128, True, 3.0, 1, (None, None)),
    ("softcap_noncausal_ragged_strong_cap", 2, 113, 224, 3, 1, 128, False, 0.75, 1, (None, None)),
    ("softcap_masked_rows_d64", 1, 300, 160, 2, 2, 64, True, 2.0, 1, (None, None)),
    ("softcap_with_splits_and_window", 1, 96, 1024, 4, 2, 128, True, 5.0, 3, (300, None)),
], ids=lambda c: c[0])
def test_softcap_parity(cuda_device, case):
    """scores = softcap * tanh(scores / softcap) (the reference's softcap, testing.py:373-374).  The
    kernel uses the hardware tanh approximation (relative error about 2^-11, as the reference's
    kernel does), which moves a score by up to softcap * log2(e) * 2^-11 in the exponent: more P
    values than usual land on the other side of an e2m1 rounding boundary than in the model, so
    the bound against model B is looser here (rel-RMS 0.05); the bounds against exact attention
    and on the LSE are the usual ones."""
    _, B, Sq, Sk, Hq, Hkv, D, causal, cap, splits, window = case
    q, k, v = make_qkv(B, Sq, Sk, Hq, Hkv, D, seed=31, device=cuda_device)
    Q, K, V = fa.quantize_qkv(q * 2.0, k * 2.0, v)       # scores of std 4: the cap bites
    out, lse = run(Q, K, V, causal, softcap=cap, num_splits=splits, window_size=window)
    oa, la, ob, lb = oracles(Q, K, V, causal, softcap=cap, num_splits=splits, window=window)
    o = out.float().cpu()
    assert torch.isfinite(o).all()
    eb, ea, eba = orc.error_metrics(o, ob), orc.error_metrics(o, oa), orc.error_metrics(ob, oa)
    assert eb["rel_rms"] <= 0.05, eb
    assert ea["rel_rms"] <= 1.25 * eba["rel_rms"] + 0.01, (ea, eba)
    assert torch.equal(torch.isinf(lse.cpu()), torch.isinf(la))
    fin = torch.isfinite(la)
    assert (lse.cpu()[fin] - la[fin]).abs().max().item() <= 2e-3 * max(1.0, la[fin].abs().max().item())
    # the cap changes the result (the test would not notice a kernel that ignored it otherwise)
    out0, _ = run(Q, K, V, causal, num_splits=splits, window_size=window)
    assert orc.error_metrics(out0.float().cpu(), oa)["rel_rms"] > 0.3
    if splits > 1:
        with pytest.raises((ValueError, NotImplementedError)):      # the 64-key kernel does not split
            run(Q, K, V, causal, fa.VARIANT_WS64, softcap=cap, num_splits=splits, window_size=window)


@pytest.mark.parametrize("case", [
    # name, B, Sq, Sk, Hq, Hkv, causal, splits (0 = chosen)
    ("one_row_gqa4", 2, 1, 1024, 8, 2, True, 2),
    ("one_row_mqa_ragged_keys", 1, 1, 160, 2, 1, True, 1),
    ("four_rows_three_splits", 1, 4, 640, 4, 2, True, 3),
    ("two_rows_noncausal", 2, 2, 384, 8, 2, False, 1),
    ("sixteen_rows_mha", 1, 16, 512, 2, 2, True, 2),
    ("eight_rows_more_splits_than_blocks", 1, 2, 256, 8, 2, True, 5),
    ("one_row_chosen_splits", 3, 1, 4096, 8, 2, True, 0),
    # row counts that do not fill the kernel's 4 / 8 / 16-row forms (padding rows see nothing)
    ("three_rows_of_four", 1, 3, 416, 2, 2, True, 2),
    ("six_rows_of_eight_noncausal", 2, 3, 300, 4, 2, False, 1),
    ("twelve_rows_of_sixteen", 1, 3, 1000, 8, 2, True, 3),
    # more than sixteen rows: the 32-row form (N = 32), a thread owns a row with all 32 keys of its warp
    ("thirty_two_rows", 2, 8, 1200, 8, 2, True, 3),
    ("twenty_four_rows_of_thirty_two_noncausal", 1, 3, 700, 8, 1, False, 2),
    ("seventeen_rows_mha", 1, 17, 400, 2, 2, True, 1),
], ids=lambda c: c[0])
def test_decode_kernel_parity(cuda_device, case):
    """The transposed decode kernel (keys on the lanes, the Sq * Hq / Hkv <= 32 query rows of a kv
    head on the N side), which the automatic choice runs for these shapes: against the oracle's
    model of it (128-key steps upwards, contiguous shares of the blocks per split) at the usual
    tolerances, and deterministic."""
    _, B, Sq, Sk, Hq, Hkv, causal, splits = case
    q, k, v = make_qkv(B, Sq, Sk, Hq, Hkv, 128, seed=13, device=cuda_device)
    Q, K, V = fa.quantize_qkv(q, k, v)
    out, lse = run(Q, K, V, causal, num_splits=splits)
    n = splits if splits else fa.interface.choose_decode_splits(B, Hkv, Sk, cuda_device)
    assert_parity(out, lse, *oracles(Q, K, V, causal, num_splits=n))
    out2, lse2 = run(Q, K, V, causal, fa.VARIANT_DECODE, num_splits=splits)
    assert torch.equal(out, out2) and torch.equal(lse, lse2)
    # the prefill kernel on the same problem: another grouping of the same 4-bit P
    out_w, lse_w = run(Q, K, V, causal, fa.VARIANT_WS)
    assert (lse - lse_w).abs().max().item() < 1e-3
    assert orc.error_metrics(out.float(), out_w.float())["rel_rms"] < 0.25


def test_decode_kernel_refuses_other_shapes(cuda_device):
    q, k, v = make_qkv(1, 33, 256, 2, 2, 128, seed=1, device=cuda_device)
    Q, K, V = fa.quantize_qkv(q, k, v)
    with pytest.raises(NotImplementedError):
        run(Q, K, V, True, fa.VARIANT_DECODE)                      # 33 rows
    q, k, v = make_qkv(1, 2, 256, 2, 2, 128, seed=1, device=cuda_device)
    Q, K, V = fa.quantize_qkv(q, k, v)
    for kw in ({"window_size": (64, 0)}, {"softcap": 2.0}, {"learnable_sink": torch.zeros(2)}):
        with pytest.raises(NotImplementedError):
            run(Q, K, V, True, fa.VARIANT_DECODE, **kw)


@pytest.mark.parametrize("case", [
    # name, Sq, page_size, pages_per_seq, seqused, D, causal, splits
    ("decode_one_row", 1, 128, 5, [208, 640, 48], 128, True, 1),
    ("append_17_rows_split", 17, 256, 3, [768, 304, 17 + 15], 128, True, 2),
    ("prefill_tile_and_a_half_empty_entry", 192, 128, 4, [512, 0, 336], 128, True, 1),
    ("noncausal_d64", 40, 128, 3, [384, 16, 272], 64, False, 1),
], ids=lambda c: c[0])
def test_kv_cache_seqused_and_page_table(cuda_device, case):
    """The reference's seqused_k / page_table (interface.py:296-300, paged_kv.py): every batch entry
    attends to its first seqused_k[b] keys, with and without K / V living in a shuffled page pool.
    Each entry is checked against the oracle on its own truncated operands; the paged call must give
    the bits of the contiguous one (same arithmetic, other addresses)."""
    _, Sq, page_size, pps, used, D, causal, splits = case
    B, Hq, Hkv, Sk = len(used), 4, 2, page_size * pps
    q, k, v = make_qkv(B, Sq, Sk, Hq, Hkv, D, seed=41, device=cuda_device)
    Q, K, V = fa.quantize_qkv(q, k, v)
    su = torch.tensor(used, dtype=torch.int32, device=cuda_device)
    # what the automatic choice runs for this shape: the decode kernel for a handful of rows
    model = (fa.VARIANT_DECODE if (D == 128 and Sq * (Hq // Hkv) <= 32)
             else (fa.VARIANT_WS64 if splits == 1 else fa.VARIANT_WS))
    out, lse = run(Q, K, V, causal, seqused_k=su, num_splits=splits)
    for b, sk in enumerate(used):
        if sk == 0:
            assert torch.all(out[b] == 0) and torch.all(torch.isinf(lse[b]) & (lse[b] < 0))
            continue
        Qb = fa.NVFP4Tensor(Q.data[b:b + 1], Q.sf[b:b + 1], Q.scale)
        Kb = fa.NVFP4Tensor(K.data[b:b + 1, :sk], K.sf[b:b + 1, :sk], K.scale)
        Vb = fa.NVFP4Tensor(V.data[b:b + 1, :, :, :sk // 2], V.sf[b:b + 1, :, :, :sk // 16], V.scale, is_v=True)
        assert_parity(out[b:b + 1], lse[b:b + 1], *oracles(Qb, Kb, Vb, causal, num_splits=splits, variant=model))
    # the same through a page pool: pages of all entries shuffled among three spare pages whose
    # packed bytes are noise (their scale bytes stay zero: no NaN encodings)
    g = torch.Generator(device="cpu").manual_seed(7)
    n_pages = B * pps + 3
    perm = torch.randperm(n_pages, generator=g)[:B * pps].reshape(B, pps)
    kp = torch.randint(0, 256, (n_pages, page_size, Hkv, D // 2), dtype=torch.uint8, generator=g).to(cuda_device)
    vp = torch.randint(0, 256, (n_pages, Hkv, D, page_size // 2), dtype=torch.uint8, generator=g).to(cuda_device)
    ksp = torch.zeros(n_pages, page_size, Hkv, D // 16, dtype=torch.uint8, device=cuda_device)
    vsp = torch.zeros(n_pages, Hkv, D, page_size // 16, dtype=torch.uint8, device=cuda_device)
    for b in range(B):
        for j in range(pps):
            pg, k0 = int(perm[b, j]), j * page_size
            kp[pg] = K.data[b, k0:k0 + page_size]
            ksp[pg] = K.sf[b, k0:k0 + page_size]
            vp[pg] = V.data[b, :, :, k0 // 2:(k0 + page_size) // 2]
            vsp[pg] = V.sf[b, :, :, k0 // 16:(k0 + page_size) // 16]
    table = perm.to(torch.int32).to(cuda_device)
    out_p, lse_p = fa.flash_attn_fp4_func(Q.data, kp, vp, Q.sf, ksp, vsp, Q.scale, K.scale, V.scale, causal=causal,
                                          return_lse=True, seqused_k=su, page_table=table, num_splits=splits)
    torch.cuda.synchronize()
    fa.check_status(cuda_device)
    assert torch.equal(out_p, out) and torch.equal(lse_p, lse)
    # a table without seqused_k: every entry sees the whole logical length
    out_f, lse_f = fa.flash_attn_fp4_func(Q.data, kp, vp, Q.sf, ksp, vsp, Q.scale, K.scale, V.scale, causal=causal,
                                          return_lse=True, page_table=table)
    model1 = fa.VARIANT_DECODE if model == fa.VARIANT_DECODE else fa.VARIANT_WS64      # this call does not split
    want_f, want_l = run(Q, K, V, causal, model1)
    torch.cuda.synchronize()
    assert torch.equal(out_f, want_f) and torch.equal(lse_f, want_l)
    with pytest.raises(NotImplementedError):
        fa.flash_attn_fp4_func(Q.data, kp[:, :96], vp[..., :48], Q.sf, ksp[:, :96], vsp[..., :6], Q.scale, K.scale,
                               V.scale, page_table=table)


def test_varlen_packed_batch_matches_dense_calls(cuda_device):
    """flash_attn_varlen_func surface: three sequences packed along the token axis give the bits
    of three dense calls, and the oracle's tolerance per sequence; one slot is padded
    (seqused_k)."""
    Hq, Hkv, D = 4, 2, 128
    sq, slot_k, used_k = [70, 128, 1], [96, 256, 160], [96, 224, 160]
    cq = [0] + list(np.cumsum(sq))
    ck = [0] + list(np.cumsum(slot_k))
    g = torch.Generator().manual_seed(31)
    q = torch.randn(1, cq[-1], Hq, D, generator=g).bfloat16().to(cuda_device)
    k = torch.randn(1, ck[-1], Hkv, D, generator=g).bfloat16().to(cuda_device)
    v = torch.randn(1, ck[-1], Hkv, D, generator=g).bfloat16().to(cuda_device)
    Q, K, V = fa.quantize_qkv(q, k, v)                      # one tensor scale for the whole pack
    out, lse = fa.flash_attn_varlen_fp4_func(
        Q.data[0], K.data[0], V.data[0], Q.sf[0], K.sf[0], V.sf[0], Q.scale, K.scale, V.scale,
        torch.tensor(cq, dtype=torch.int32), ck, seqused_k=used_k, causal=True, return_lse=True)
    torch.cuda.synchronize()
    fa.check_status(cuda_device)
    assert out.shape == (cq[-1], Hq, D) and lse.shape == (Hq, cq[-1])
    for i in range(3):
        q0, q1, k0, k1 = cq[i], cq[i + 1], ck[i], ck[i] + used_k[i]
        Qi = fa.NVFP4Tensor(Q.data[:, q0:q1].contiguous(), Q.sf[:, q0:q1].contiguous(), Q.scale)
        Ki = fa.NVFP4Tensor(K.data[:, k0:k1].contiguous(), K.sf[:, k0:k1].contiguous(), K.scale)
        Vi = fa.NVFP4Tensor(V.data[..., k0 // 2:k1 // 2].contiguous(), V.sf[..., k0 // 16:k1 // 16].contiguous(),
                            V.scale, is_v=True)
        # (the packed call runs the 64-key kernel for every sequence; the dense call would pick the
        # decode kernel for the one-token sequence, so the kernel is named here)
        o_d, l_d = run(Qi, Ki, Vi, True, fa.VARIANT_WS64)
        assert torch.equal(out[q0:q1], o_d[0]) and torch.equal(lse[:, q0:q1], l_d[0])
        assert_parity(o_d, l_d, *oracles(Qi, Ki, Vi, True, variant=fa.VARIANT_WS64))


def test_varlen_one_launch_device_offsets_noncausal_window_and_sink(cuda_device):
    """Packed batch with odd query lengths, device cu_seqlens and max_seqlen given (nothing is read
    back): non-causal, a sliding window, and a learnable sink, each bit-identical to the dense
    call on the single sequences."""
    Hq, Hkv, D = 4, 2, 128
    sq, sk = [257, 3, 128, 60], [320, 64, 128, 96]
    cq = [0] + list(np.cumsum(sq))
    ck = [0] + list(np.cumsum(sk))
    g = torch.Generator().manual_seed(32)
    q = torch.randn(1, cq[-1], Hq, D, generator=g).bfloat16().to(cuda_device)
    k = torch.randn(1, ck[-1], Hkv, D, generator=g).bfloat16().to(cuda_device)
    v = torch.randn(1, ck[-1], Hkv, D, generator=g).bfloat16().to(cuda_device)
    Q, K, V = fa.quantize_qkv(q, k, v)
    cu_q = torch.tensor(cq, dtype=torch.int32, device=cuda_device)
    cu_k = torch.tensor(ck, dtype=torch.int32, device=cuda_device)
    sink = torch.tensor([0.3, -1.0, 2.0, 0.0])
    for kw in (dict(causal=False), dict(causal=True, window_size=(100, None)), dict(causal=True, learnable_sink=sink)):
        out, lse = fa.flash_attn_varlen_fp4_func(
            Q.data[0], K.data[0], V.data[0], Q.sf[0], K.sf[0], V.sf[0], Q.scale, K.scale, V.scale,
            cu_q, cu_k, max_seqlen_q=max(sq), max_seqlen_k=max(sk), return_lse=True, **kw)
        torch.cuda.synchronize()
        fa.check_status(cuda_device)
        for i in range(len(sq)):
            q0, q1, k0, k1 = cq[i], cq[i + 1], ck[i], ck[i + 1]
            Qi = fa.NVFP4Tensor(Q.data[:, q0:q1].contiguous(), Q.sf[:, q0:q1].contiguous(), Q.scale)
            Ki = fa.NVFP4Tensor(K.data[:, k0:k1].contiguous(), K.sf[:, k0:k1].contiguous(), K.scale)
            Vi = fa.NVFP4Tensor(V.data[..., k0 // 2:k1 // 2].contiguous(), V.sf[..., k0 // 16:k1 // 16].contiguous(),
                                V.scale, is_v=True)
            kw_d = dict(kw)
            causal_d = kw_d.pop("causal")
            o_d, l_d = run(Qi, Ki, Vi, causal_d, fa.VARIANT_WS64, **kw_d)     # the kernel the packed call runs
            assert torch.equal(out[q0:q1], o_d[0]) and torch.equal(lse[:, q0:q1], l_d[0]), (kw, i)


def test_varlen_many_short_sequences_cost_about_a_dense_call(cuda_device):
    """512 sequences of 128 tokens in one launch: bit-identical to, and within 1.5x of, the dense
    call on the same tokens shaped (512, 128) (measured 1.36x: the packed call runs the kernel's
    KV-cache flavour, which reads every sequence's bounds from the device; 512 per-sequence
    launches took more than ten times as long)."""
    Hq, Hkv, D, n, L = 8, 2, 128, 512, 128
    g = torch.Generator(device=cuda_device).manual_seed(5)
    q = torch.randn(n, L, Hq, D, generator=g, device=cuda_device, dtype=torch.bfloat16)
    k = torch.randn(n, L, Hkv, D, generator=g, device=cuda_device, dtype=torch.bfloat16)
    v = torch.randn(n, L, Hkv, D, generator=g, device=cuda_device, dtype=torch.bfloat16)
    Qd, Kd, Vd = fa.quantize_qkv_fused(q, k, v)
    # the same tokens packed: (n * L, H, D), V key-contiguous over the packed keys
    Qp, Kp, Vp = fa.quantize_qkv_fused(q.reshape(1, n * L, Hq, D), k.reshape(1, n * L, Hkv, D),
                                       v.reshape(1, n * L, Hkv, D))
    cu = torch.arange(0, (n + 1) * L, L, dtype=torch.int32, device=cuda_device)

    def dense():      # linear scale factors, converted per call like the packed call's
        return fa.flash_attn_fp4_func(Qd.data, Kd.data, Vd.data, Qd.sf, Kd.sf, Vd.sf, Qd.scale, Kd.scale, Vd.scale,
                                      causal=True, return_lse=True)

    def packed():
        return fa.flash_attn_varlen_fp4_func(Qp.data[0], Kp.data[0], Vp.data[0], Qp.sf[0], Kp.sf[0], Vp.sf[0],
                                             Qp.scale, Kp.scale, Vp.scale, cu, cu, max_seqlen_q=L, max_seqlen_k=L,
                                             causal=True, return_lse=True)
    o_d, l_d = dense()
    o_p, l_p = packed()
    torch.cuda.synchronize()
    fa.check_status(cuda_device)
    assert torch.equal(o_p.reshape(n, L, Hq, D), o_d)
    assert torch.equal(l_p.reshape(Hq, n, L).permute(1, 0, 2), l_d)

    def best_ms(fn):
        ts = []
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record(); e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        return min(ts)
    t_d, t_p = best_ms(dense), best_ms(packed)
    assert t_p <= 1.5 * t_d, (t_p, t_d)



@pytest.mark.parametrize("shape", [
    # name, B, Sq, Sk, Hq, Hkv, causal
    ("prefill", 2, 384, 384, 4, 2, True),
    ("decode", 2, 1, 2048, 8, 2, True),
], ids=lambda c: c[0])
def test_calls_replay_from_a_cuda_graph(cuda_device, shape):
    """A serving loop captures its steps in CUDA graphs: the prefill call and the decode call
    (decode kernel + combine kernel, a programmatic dependent launch) are captured once after a
    warm-up call and replayed on new operand CONTENTS in the same buffers; every replay gives the
    bits of an eager call on those operands."""
    _, B, Sq, Sk, Hq, Hkv, causal = shape
    ops = []
    for seed in (51, 52):
        q, k, v = make_qkv(B, Sq, Sk, Hq, Hkv, 128, seed=seed, device=cuda_device)
        Q, K, V = fa.quantize_qkv(q, k, v)
        ops.append([t.to(cuda_device) for t in (Q.data, K.data, V.data, Q.tiled_sf(), K.tiled_sf(), V.tiled_sf())]
                   + [Q.scale, K.scale, V.scale])
    static = [t.clone() for t in ops[0][:6]]
    out = torch.empty(B, Sq, Hq, 128, dtype=torch.bfloat16, device=cuda_device)
    lse = torch.empty(B, Hq, Sq, dtype=torch.float32, device=cuda_device)
    # per-tensor scales are host floats baked into the captured launch: both operand sets are
    # dequantised with the first set's scales here, in the eager calls too
    scales = ops[0][6:]

    def call(bufs, o, l):
        return fa.flash_attn_fp4_func(*bufs, *scales, causal=causal, return_lse=True, out=o, lse=l, sf_layout="tiled")

    side = torch.cuda.Stream(cuda_device)
    side.wait_stream(torch.cuda.current_stream(cuda_device))
    with torch.cuda.stream(side):
        call(static, out, lse)                      # warm-up outside the capture (kernel attributes are set here)
    torch.cuda.current_stream(cuda_device).wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        call(static, out, lse)
    for which in (1, 0, 1):
        for dst, src in zip(static, ops[which][:6]):
            dst.copy_(src)
        out.zero_()
        lse.zero_()
        graph.replay()
        torch.cuda.synchronize()
        fa.check_status(cuda_device)
        want_o, want_l = call(ops[which][:6], torch.empty_like(out), torch.empty_like(lse))
        torch.cuda.synchronize()
        assert torch.equal(out, want_o) and torch.equal(lse, want_l), which


def test_varlen_arbitrary_key_lengths_through_padded_v_slots(cuda_device):
    """A packed batch whose key sequences start anywhere (lengths 70, 129, 1, 333 -- the reference's
    varlen call has no alignment rule): K stays packed, V puts every sequence into a slot of whole
    32-key groups (quantize_varlen_qkv / cu_seqlens_v).  Each sequence gives the bits of the dense
    call on its own operands and meets the oracle's tolerance."""
    Hq, Hkv, D = 4, 2, 128
    sq, sk = [70, 5, 1, 200], [70, 129, 1, 333]
    cq = [0] + list(np.cumsum(sq))
    ck = [0] + list(np.cumsum(sk))
    g = torch.Generator().manual_seed(33)
    q = torch.randn(cq[-1], Hq, D, generator=g).bfloat16().to(cuda_device)
    k = torch.randn(ck[-1], Hkv, D, generator=g).bfloat16().to(cuda_device)
    v = torch.randn(ck[-1], Hkv, D, generator=g).bfloat16().to(cuda_device)
    cu_q = torch.tensor(cq, dtype=torch.int32, device=cuda_device)
    cu_k = torch.tensor(ck, dtype=torch.int32, device=cuda_device)
    Q, K, V, cu_v = fa.quantize_varlen_qkv(q, k, v, cu_k)
    cv = [int(x) for x in cu_v.cpu()]
    assert cv == [0, 96, 256, 288, 640] and V.data.shape == (1, Hkv, D, 320)
    for causal in (True, False):
        out, lse = fa.flash_attn_varlen_fp4_func(
            Q.data[0], K.data[0], V.data[0], Q.sf[0], K.sf[0], V.sf[0], Q.scale, K.scale, V.scale,
            cu_q, cu_k, cu_seqlens_v=cu_v, max_seqlen_q=max(sq), max_seqlen_k=max(sk), causal=causal, return_lse=True)
        torch.cuda.synchronize()
        fa.check_status(cuda_device)
        for i in range(len(sq)):
            q0, q1, k0, k1, v0 = cq[i], cq[i + 1], ck[i], ck[i + 1], cv[i]
            v1 = v0 + (sk[i] + 31) // 32 * 32
            Qi = fa.NVFP4Tensor(Q.data[:, q0:q1].contiguous(), Q.sf[:, q0:q1].contiguous(), Q.scale)
            Ki = fa.NVFP4Tensor(K.data[:, k0:k1].contiguous(), K.sf[:, k0:k1].contiguous(), K.scale)
            Vi = fa.NVFP4Tensor(V.data[..., v0 // 2:v1 // 2].contiguous(), V.sf[..., v0 // 16:v1 // 16].contiguous(),
                                V.scale, is_v=True)
            o_d, l_d = run(Qi, Ki, Vi, causal, fa.VARIANT_WS64)
            assert torch.equal(out[q0:q1], o_d[0]) and torch.equal(lse[:, q0:q1], l_d[0]), (causal, i)
            assert_parity(o_d, l_d, *oracles(Qi, Ki, Vi, causal, variant=fa.VARIANT_WS64))
    # without cu_seqlens_v the unaligned starts are refused on the host
    with pytest.raises(NotImplementedError):
        fa.flash_attn_varlen_fp4_func(Q.data[0], K.data[0], V.data[0], Q.sf[0], K.sf[0], V.sf[0], Q.scale, K.scale,
                                      V.scale, cq, ck, causal=True)
