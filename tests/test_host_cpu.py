"""CPU tests of the host side: the C ABI library loads and exports what include/fa4_nvfp4.h
declares, rejects bad arguments before touching a GPU, the Python surface mirrors the reference's
error behaviour, the product quantiser is bit-identical to the oracle's, and the sharding plan."""
import ctypes
import os
import re
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

import flash_attention_b200 as fa
from flash_attention_b200 import _lib, shard
from oracle import nvfp4_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fa4_nvfp4.h")


def test_library_exports_every_declared_symbol():
    L = fa.lib()
    text = open(HEADER).read()
    declared = set(re.findall(r"^(?:int|int64_t)\s+(fa4_nvfp4_\w+)\s*\(", text, flags=re.M))
    assert declared, "no declarations found in the header"
    assert declared == set(_lib.EXPORTS) or declared >= set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(L, name), f"{name} is declared but not exported"


def test_params_struct_matches_header():
    """sizeof / offsets of the ctypes mirror equal the C compiler's view of the header."""
    src = r'''
#include <stdio.h>
#include <stddef.h>
#include "fa4_nvfp4.h"
int main(void) {
  printf("%zu %zu %zu %zu %zu %zu\n", sizeof(fa4_nvfp4_params), offsetof(fa4_nvfp4_params, q),
         offsetof(fa4_nvfp4_params, q_stride_b), offsetof(fa4_nvfp4_params, B),
         offsetof(fa4_nvfp4_params, q_scale), offsetof(fa4_nvfp4_params, wait_budget_ns));
  return 0;
}'''
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "t.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "t")
        subprocess.run(["gcc", "-std=c99", "-I", os.path.join(ROOT, "include"), c, "-o", exe], check=True)
        got = [int(x) for x in subprocess.run([exe], capture_output=True, text=True, check=True).stdout.split()]
    P = _lib.Params
    assert got == [ctypes.sizeof(P), P.q.offset, P.q_stride_b.offset, P.B.offset, P.q_scale.offset,
                   P.wait_budget_ns.offset]


def test_query():
    L = fa.lib()
    assert L.fa4_nvfp4_query(0) == 1
    n = L.fa4_nvfp4_query(1)
    assert n >= 1 and 128 in [L.fa4_nvfp4_query(2 + i) for i in range(n)]
    assert L.fa4_nvfp4_query(100) <= 227 * 1024


def _good_params():
    p = _lib.Params()
    p.struct_size = ctypes.sizeof(_lib.Params)
    for f in ("q", "k", "v", "q_sf", "k_sf", "v_sf", "out"):
        setattr(p, f, 0x1000)
    p.B, p.Sq, p.Sk, p.Hq, p.Hkv, p.D, p.Dv = 1, 128, 128, 2, 1, 128, 128
    p.q_stride_b, p.q_stride_s, p.q_stride_h = 128 * 2 * 64, 2 * 64, 64
    p.k_stride_b, p.k_stride_s, p.k_stride_h = 128 * 64, 64, 64
    p.v_stride_b, p.v_stride_h, p.v_stride_d = 128 * 64, 128 * 64, 64
    p.o_stride_b, p.o_stride_s, p.o_stride_h = 128 * 2 * 128, 2 * 128, 128
    p.q_scale = p.k_scale = p.v_scale = 1.0
    p.softmax_scale = 0.088
    return p


@pytest.mark.parametrize("mutate,code", [
    (lambda p: setattr(p, "struct_size", 8), 7),
    (lambda p: setattr(p, "q", None), 1),
    (lambda p: setattr(p, "out", None), 1),
    (lambda p: (setattr(p, "Hq", 3), setattr(p, "Hkv", 2)), 2),   # Hq not a multiple of Hkv
    (lambda p: setattr(p, "D", 96), 2),
    (lambda p: setattr(p, "v_stride_d", 72), 3),   # V rows (the padded key axis) must be 16-byte multiples
    (lambda p: setattr(p, "Sk", 0), 2),
    (lambda p: setattr(p, "softmax_scale", 0.0), 2),
    (lambda p: setattr(p, "k", 0x1008), 4),
    (lambda p: setattr(p, "q_stride_s", 72), 3),
    (lambda p: setattr(p, "o_stride_h", 4), 3),
    (lambda p: setattr(p, "variant", 9), 5),
])
def test_fwd_rejects_bad_arguments_on_host(mutate, code):
    """Every rejection happens before any CUDA call, so this runs without a GPU."""
    p = _good_params()
    mutate(p)
    assert fa.lib().fa4_nvfp4_fwd(ctypes.byref(p), None) == -code
    assert fa.lib().fa4_nvfp4_fwd(None, None) == -1


def test_aux_entry_points_reject_bad_arguments():
    L = fa.lib()
    assert L.fa4_nvfp4_sf_linear_to_tiled(None, 0x1000, 1, 1, 1, 1, 1, 1, 1, 1, None) == -1
    assert L.fa4_nvfp4_sf_linear_to_tiled(0x1000, 0x1000, 1, 1, 0, 1, 1, 1, 1, 1, None) == -2
    assert L.fa4_nvfp4_sf_linear_to_tiled(0x1000, 0x1000, 1, 1, 1, 1, 1, 1, 1, 0, None) == -2
    assert L.fa4_nvfp4_sf_linear_to_tiled(0x1000, 0x1004, 1, 1, 1, 1, 1, 1, 1, 1, None) == -4
    assert L.fa4_nvfp4_debug_qk_tile(0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 64, 0, None, None) == -2
    assert L.fa4_nvfp4_debug_wait_expiry(None, 1000, None) == -1
    assert L.fa4_nvfp4_debug_wait_expiry(0x1000, 0, None) == -2


def test_python_surface_errors_before_launch():
    q = torch.zeros(1, 128, 2, 64, dtype=torch.uint8)
    sf = torch.zeros(1, 128, 2, 8, dtype=torch.uint8)
    v = torch.zeros(1, 2, 128, 64, dtype=torch.uint8)
    vsf = torch.zeros(1, 2, 128, 8, dtype=torch.uint8)
    with pytest.raises(AssertionError, match="CUDA"):
        fa.flash_attn_fp4_func(q, q, v, sf, sf, vsf, 1.0, 1.0, 1.0)
    with pytest.raises(AssertionError):
        fa.flash_attn_fp4_func(q.float(), q, v, sf, sf, vsf, 1.0, 1.0, 1.0)
    with pytest.raises(TypeError):
        fa.flash_attn_func(q, q, v)
    Q = fa.NVFP4Tensor(q, sf, 1.0)
    V = fa.NVFP4Tensor(v, vsf, 1.0, is_v=True)
    with pytest.raises(NotImplementedError):
        fa.flash_attn_func(Q, Q, V, mask_mod=lambda *a: True)


def test_product_quantiser_is_bit_identical_to_oracle():
    rng = np.random.default_rng(1)
    x = (rng.standard_normal((2, 48, 3, 128)) * rng.choice([0.1, 1.0, 30.0], size=(2, 48, 3, 1))).astype(np.float32)
    x[0, 0, 0, :16] = 0.0
    a = orc.quantize_nvfp4(x)
    d, s, g = fa.quantize_lastdim(torch.from_numpy(x))
    assert np.array_equal(a.data, d.numpy()) and np.array_equal(a.sf, s.numpy()) and a.scale == g
    assert np.array_equal(orc.dequantize_nvfp4(a), fa.dequantize_lastdim(d, s, g).numpy())
    q, k, v = (torch.from_numpy(x), torch.from_numpy(x[:, :, :1]), torch.from_numpy(x[:, :, :1] * 0.5))
    Q, K, V = fa.quantize_qkv(q, k, v)
    # V's key axis is padded with zeros to a multiple of 32 (48 -> 64 keys)
    assert V.data.shape == (2, 1, 128, 32) and V.sf.shape == (2, 1, 128, 4) and V.is_v
    assert V.dequantize().shape == (2, 64, 1, 128) and not V.dequantize()[:, 48:].any()


def test_shard_plan_covers_every_unit_once():
    for B, Hkv, world in [(4, 8, 1), (4, 8, 2), (4, 8, 4), (4, 8, 8), (1, 8, 8), (8, 16, 8), (4, 8, 16)]:
        seen = np.zeros((B, Hkv), dtype=int)
        for r in range(world):
            s = shard.plan_shard(B, Hkv, world, r)
            seen[s.b0:s.b1, s.h0:s.h1] += 1
            assert s.units == B * Hkv // world
        assert (seen == 1).all()
    with pytest.raises(ValueError):
        shard.plan_shard(3, 8, 5, 0)
    with pytest.raises(ValueError):
        shard.plan_shard(2, 6, 3, 0)     # 4 units per rank straddles a batch boundary


def _gloo_worker(rank, world, port, tmp):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from tests.helpers import make_qkv
    B, Sq, Sk, Hq, Hkv, D = 2, 128, 128, 4, 2, 128
    q, k, v = make_qkv(B, Sq, Sk, Hq, Hkv, D, seed=5)
    Q, K, V = fa.quantize_qkv(q, k, v)                      # scales from the WHOLE tensors
    s = shard.plan_shard(B, Hkv, world, rank)
    Qs, Ks, Vs = shard.shard_operands(Q, K, V, s)
    # stand-in for the kernel on CPU ranks: the oracle on this rank's slice
    o, l = orc.attention_oracle_a(Qs.dequantize(), Ks.dequantize(), Vs.dequantize(), causal=True)
    full_o, full_l = shard.gather_output(o, l, s, B, Hq, Hkv)
    ref_o, ref_l = orc.attention_oracle_a(Q.dequantize(), K.dequantize(), V.dequantize(), causal=True)
    ok = torch.equal(full_o, ref_o) and torch.equal(full_l, ref_l)
    open(os.path.join(tmp, f"ok{rank}"), "w").write(str(ok))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_run_equals_unsharded_gloo_world2():
    """World size 2 on CPU (gloo): shard -> per-rank attention -> all-gather reproduces the
    single-rank result bit for bit (per-tensor scales are global)."""
    import torch.multiprocessing as mp
    with tempfile.TemporaryDirectory() as tmp:
        port = 29500 + (os.getpid() % 2000)
        mp.spawn(_gloo_worker, args=(2, port, tmp), nprocs=2, join=True)
        assert [open(os.path.join(tmp, f"ok{r}")).read() for r in range(2)] == ["True", "True"]


def test_split_heuristic_cost_model():
    """choose_num_splits: no split when the query tiles fill the GPU, a wave-aware count otherwise."""
    from unittest import mock
    import flash_attention_b200.interface as I

    class Props:
        multi_processor_count = 148
    with mock.patch.object(torch.cuda, "get_device_properties", lambda d: Props):
        assert I.choose_num_splits(4, 8192, 8192, 32, True, None) == 1      # prefill: 8192 tiles
        assert I.choose_num_splits(4, 1, 32768, 32, True, None) == 1        # 128 tiles: nearly a wave
        n = I.choose_num_splits(1, 1, 131072, 32, True, None)               # 32 tiles, 1024 blocks
        assert 4 <= n <= 9 and (32 * n + 147) // 148 == 2
        assert I.choose_num_splits(1, 128, 512, 8, False, None) == 1        # too few blocks to split


def test_decode_split_choice_and_oracle_model_selection():
    """Host logic around the decode kernel: key splits aim at about two CTAs per SM (the kernel is HBM-bound from there)
    with at least two blocks per split, and the test helper picks the oracle model of the kernel
    the library would run."""
    from unittest import mock
    import flash_attention_b200.interface as I
    from tests.helpers import kernel_model

    class Props:
        multi_processor_count = 148
    with mock.patch.object(torch.cuda, "get_device_properties", lambda d: Props):
        assert I.choose_decode_splits(4, 8, 32768, None) == 9           # 288 CTAs: about two per SM
        assert I.choose_decode_splits(64, 8, 4096, None) == 2           # 512 units run in waves: 3 x 20 < 2 x 36
        assert I.choose_decode_splits(1, 1, 512, None) == 2             # at least two blocks per split
        assert I.choose_decode_splits(1, 8, 1 << 20, None) == 37
    assert kernel_model(128, rows=4) == {"step_keys": 128, "ascending": True}          # decode kernel
    assert kernel_model(128, rows=4, num_splits=5) == {"step_keys": 128, "ascending": True}
    def is64(m):       # the 64-key kernel's model (its P block-scale rule is whatever the library was built with)
        return (m["step_keys"], m["ascending"]) == (64, True) and m["p_scale"] in ("pow2", "e4m3")
    assert is64(kernel_model(128, rows=256))                           # 64-key prefill kernel
    assert is64(kernel_model(64, rows=4))                              # head dim 64: no decode kernel
    assert is64(kernel_model(128, rows=4, softcap=2.0))                # general 64-key kernel
    assert is64(kernel_model(128, rows=256, window=(64, None)))
    assert is64(kernel_model(128, rows=256, sink=[0.0]))
    assert kernel_model(128, rows=256, num_splits=2) == {"step_keys": 128, "ascending": False}
    assert kernel_model(128, rows=4, variant=2) == {"step_keys": 128, "ascending": False}


def test_oracle_split_model_matches_unsplit_statistics():
    from oracle import nvfp4_oracle as orc
    from tests.helpers import make_qkv, oracles
    q, k, v = make_qkv(1, 17, 1536, 2, 1, 128, seed=9)
    Q, K, V = fa.quantize_qkv(q, k, v)
    oa, la, ob1, lb1 = oracles(Q, K, V, False)
    _, _, ob3, lb3 = oracles(Q, K, V, False, num_splits=3)
    assert (lb1 - lb3).abs().max().item() < 1e-5
    e1, e3 = orc.error_metrics(ob1, oa), orc.error_metrics(ob3, oa)
    assert abs(e1["rel_rms"] - e3["rel_rms"]) < 0.03


def test_window_resolution_follows_the_reference_rules():
    """flash_attn/cute/interface.py:256-276: causal sets right = 0; (None, 0) is plain causal;
    limits that sum below zero mean no window."""
    from flash_attention_b200.interface import resolve_window
    assert resolve_window(False, (None, None)) == (False, None, None)
    assert resolve_window(True, (None, None)) == (True, None, 0)
    assert resolve_window(False, (None, 0)) == (True, None, 0)
    assert resolve_window(True, (128, None)) == (False, 128, 0)
    assert resolve_window(False, (64, 32)) == (False, 64, 32)
    assert resolve_window(False, (-1, -1)) == (False, None, None)
    assert resolve_window(True, (5, 99)) == (False, 5, 0)          # causal overrides the right limit


def test_oracle_window_masks_match_reference_formula():
    """_visibility_mask against the closed form of construct_local_mask (testing.py:249-288)."""
    for (sq, sk, causal, win) in [(5, 9, True, (None, None)), (7, 7, False, (2, 1)), (4, 10, True, (3, None)),
                                  (9, 4, False, (None, 2)), (6, 6, False, (0, 0))]:
        m = orc._visibility_mask(sq, sk, causal, win)
        left, right = win
        if causal:
            right = 0
        for i in range(sq):
            for j in range(sk):
                masked = (right is not None and j > i + sk - sq + right) or \
                         (left is not None and j < i + sk - sq - left)
                assert bool(m[i, j]) == masked


def test_varlen_surface_rejects_bad_offsets_before_any_launch():
    z = lambda *s: torch.zeros(*s, dtype=torch.uint8)
    args = (z(48, 2, 64), z(80, 1, 64), z(1, 128, 48), z(48, 2, 8), z(80, 1, 8), z(1, 128, 6), 1.0, 1.0, 1.0)
    with pytest.raises(NotImplementedError):          # a key sequence that starts at 48: not a multiple of 32
        fa.flash_attn_varlen_fp4_func(*args, [0, 16, 32, 48], [0, 32, 48, 80])
    with pytest.raises(AssertionError):               # offsets do not cover the packed tensor
        fa.flash_attn_varlen_fp4_func(*args, [0, 16, 40], [0, 32, 80])
    with pytest.raises(AssertionError):               # different batch sizes
        fa.flash_attn_varlen_fp4_func(*args, [0, 48], [0, 32, 80])


def test_varlen_entry_point_checks_its_arguments_on_the_host():
    """fa4_nvfp4_fwd_varlen without a GPU: every malformed description of the packed batch comes
    back with a negative argument code before anything could be launched."""
    import ctypes
    from flash_attention_b200 import _lib
    L = fa.lib()
    p = _lib.Params()
    p.struct_size = ctypes.sizeof(_lib.Params)
    for f in ("q", "k", "v", "q_sf", "k_sf", "v_sf", "out"):
        setattr(p, f, 0x1000)
    p.B, p.Sq, p.Sk, p.Hq, p.Hkv, p.D, p.Dv = 1, 128, 128, 2, 1, 128, 128
    p.q_scale = p.k_scale = p.v_scale = 1.0
    p.softmax_scale = 0.088

    def varlen(**kw):
        x = _lib.Varlen()
        x.struct_size = ctypes.sizeof(_lib.Varlen)
        x.num_seqs, x.total_q, x.total_k, x.max_seqlen_q, x.max_seqlen_k = 2, 200, 200, 128, 128
        x.cu_seqlens_q = x.cu_seqlens_k = 0x2000
        x.window_left = x.window_right = -1
        for k_, v_ in kw.items():
            setattr(x, k_, v_)
        return x

    call = lambda x: L.fa4_nvfp4_fwd_varlen(ctypes.byref(p), ctypes.byref(x), None)
    assert call(varlen(cu_seqlens_k=None)) == -1                       # NULL offsets
    assert call(varlen(struct_size=8)) == -7
    assert call(varlen(max_seqlen_k=300)) == -2                        # longer than the pack
    assert call(varlen(reserved=1)) == -2 and call(varlen(reserved2=1)) == -2
    assert call(varlen(total_v=224)) == -2                             # a V length without V offsets
    assert call(varlen(cu_seqlens_v=0x3000, total_v=100)) == -2        # V shorter than the keys
    assert call(varlen(cu_seqlens_v=0x3000, total_v=230)) == -2        # not a multiple of 32
    assert call(varlen(window_left=-2)) == -2
    p.variant = 2                                                      # the 128-key kernel has no packed form
    assert call(varlen()) == -5


def test_padded_key_offsets_of_a_packed_batch():
    cu = torch.tensor([0, 70, 199, 200, 533, 533], dtype=torch.int32)
    assert fa.padded_key_offsets(cu).tolist() == [0, 96, 256, 288, 640, 640]
    assert fa.padded_key_offsets(torch.tensor([0, 64, 128], dtype=torch.int32)).tolist() == [0, 64, 128]
