"""GPU parity of the fused NVFP4 quantiser: bit-exact against the CPU oracle's quantiser."""
import numpy as np
import pytest
import torch

import flash_attention_b200 as fa
from oracle import nvfp4_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda_device():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    fa.lib()
    return torch.device("cuda", 0)


def _oracle_qk(x):
    return orc.quantize_nvfp4(x.float().cpu().numpy())


def _oracle_v(v):
    # V is quantised key-contiguous with its key axis padded with zeros to a multiple of 32
    pad = (-v.shape[1]) % 32
    if pad:
        v = torch.cat([v, v.new_zeros(v.shape[0], pad, v.shape[2], v.shape[3])], dim=1)
    return orc.quantize_nvfp4(v.float().permute(0, 2, 3, 1).contiguous().cpu().numpy())


def _tiled(sf_np, mult):
    return orc.sf_linear_to_tiled(sf_np, mult)


CASES = [
    # B, S, Hq, Hkv, D, std
    (1, 256, 4, 4, 128, 1.0),
    (2, 208, 4, 2, 128, 1.0),      # ragged rows: zero padding of the tiled scales
    (1, 96, 2, 1, 64, 3.0),        # D = 64, Dv = 64 (half a d tile)
    (1, 1024, 3, 3, 192, 0.5),     # D = 192: three column tiles, two d tiles for V
]


@pytest.mark.parametrize("case", CASES, ids=[f"B{c[0]}_S{c[1]}_H{c[2]}_{c[3]}_D{c[4]}" for c in CASES])
def test_fused_quantiser_is_bit_exact(cuda_device, case):
    B, S, Hq, Hkv, D, std = case
    g = torch.Generator().manual_seed(11)
    q = (torch.randn(B, S, Hq, D, generator=g) * std).bfloat16()
    k = (torch.randn(B, S, Hkv, D, generator=g) * std).bfloat16()
    v = (torch.randn(B, S, Hkv, D, generator=g) * std).bfloat16()
    # exact ties and exact zeros exercise round-to-even and the sign of zero
    q[0, 0, 0, :16] = torch.tensor([0.25, -0.25, 0.75, -0.75, 1.25, 1.75, 2.5, -2.5, 3.5, 5.0, -5.0, 6.0,
                                    0.0, -0.0, 1e-3, -1e-3]).bfloat16() * 0.5
    k[0, 1, 0, 16:32] = 0.0
    Q, K, V = fa.quantize_qkv_fused(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device))
    for got, want, mult in ((Q, _oracle_qk(q), 1), (K, _oracle_qk(k), 1), (V, _oracle_v(v), 2)):
        assert got.scale == pytest.approx(want.scale, rel=0, abs=0)
        assert np.array_equal(got.sf.cpu().numpy(), want.sf)
        assert np.array_equal(got.data.cpu().numpy(), want.data)
        lin = want.sf if got.is_v else np.transpose(want.sf, (0, 2, 1, 3))
        assert np.array_equal(got.sf_tiled.cpu().numpy(), _tiled(lin, mult))


def test_tiny_magnitudes_take_the_exact_path(cuda_device):
    # tensor scale ~1e-36: the block denominators have no finite fp32 reciprocal
    g = torch.Generator().manual_seed(4)
    x = (torch.randn(1, 128, 2, 128, generator=g) * 1e-33).bfloat16()
    Q, _, V = fa.quantize_qkv_fused(x.to(cuda_device), x.to(cuda_device), x.to(cuda_device))
    for got, want in ((Q, _oracle_qk(x)), (V, _oracle_v(x))):
        assert got.scale == want.scale
        assert np.array_equal(got.sf.cpu().numpy(), want.sf)
        assert np.array_equal(got.data.cpu().numpy(), want.data)


def test_all_zero_tensor_and_strided_input(cuda_device):
    z = torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16, device=cuda_device)
    Q, K, V = fa.quantize_qkv_fused(z, z, z)
    assert Q.scale == 1.0 and int(Q.data.max()) == 0 and int(Q.sf.max()) == 0
    g = torch.Generator(device=cuda_device).manual_seed(5)
    big = torch.randn(2, 256, 6, 128, generator=g, device=cuda_device, dtype=torch.bfloat16)
    view = big[:, 64:192, 1:5]                      # strided batch / seq / head view
    Qa, _, Va = fa.quantize_qkv_fused(view, view, view)
    Qb, _, Vb = fa.quantize_qkv_fused(view.contiguous(), view.contiguous(), view.contiguous())
    for a, b in ((Qa, Qb), (Va, Vb)):
        assert a.scale == b.scale and torch.equal(a.data, b.data) and torch.equal(a.sf, b.sf)
        assert torch.equal(a.sf_tiled, b.sf_tiled)


def test_fused_quantiser_feeds_the_attention_kernel(cuda_device):
    g = torch.Generator(device=cuda_device).manual_seed(2)
    q = torch.randn(1, 384, 4, 128, generator=g, device=cuda_device, dtype=torch.bfloat16)
    k = torch.randn(1, 384, 2, 128, generator=g, device=cuda_device, dtype=torch.bfloat16)
    v = torch.randn(1, 384, 2, 128, generator=g, device=cuda_device, dtype=torch.bfloat16)
    Q, K, V = fa.quantize_qkv_fused(q, k, v)
    o1, l1 = fa.flash_attn_func(Q, K, V, causal=True, return_lse=True)
    # same operands with the scales tiled by the separate conversion kernel
    Q2, K2, V2 = (fa.NVFP4Tensor(t.data, t.sf, t.scale, False, t.is_v) for t in (Q, K, V))
    o2, l2 = fa.flash_attn_func(Q2, K2, V2, causal=True, return_lse=True)
    fa.check_status(cuda_device)
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    # tiled-only output
    Q3, K3, V3 = fa.quantize_qkv_fused(q, k, v, linear_sf=False)
    o3, _ = fa.flash_attn_func(Q3, K3, V3, causal=True, return_lse=True)
    assert torch.equal(o1, o3)
