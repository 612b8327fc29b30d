"""The allocation-free entry point, fa4_nvfp4_fwd_linear_sf_noalloc, against the regular one.

Some hosts of this library may not allocate device memory while they run (their own arena owns
all of it, or their steady-state loop forbids the allocator because cudaMalloc synchronises the
device).  For them the scratch that the linear-scale-factor route needs sits in a fixed array
inside the library.  This file checks, through the C ABI, that the entry point gives exactly the
bits of the regular route, twice in a row with different problems (the array keeps the previous
call's contents, so a later call would show stale data if anything were left unwritten), that a
call the forward would reject is rejected before any kernel runs, and that it refuses a problem
whose scale factors exceed the array.

Named test_zz_* so that pytest collects it last."""
import ctypes

import pytest
import torch

import flash_attention_b200 as fa
from flash_attention_b200 import _lib
from flash_attention_b200.interface import DeviceStatus
from tests.helpers import make_qkv


def _params(Q, K, V, out, lse, causal, status, D=128, Dv=128):
    B, Sq, Hq, _ = Q.data.shape
    _, Sk, Hkv, _ = K.data.shape
    p = _lib.Params()
    p.struct_size = ctypes.sizeof(_lib.Params)
    p.variant = 0
    p.q, p.k, p.v = Q.data.data_ptr(), K.data.data_ptr(), V.data.data_ptr()
    p.q_sf, p.k_sf, p.v_sf = Q.sf.data_ptr(), K.sf.data_ptr(), V.sf.data_ptr()
    p.out, p.lse, p.status = out.data_ptr(), lse.data_ptr(), status.data_ptr()
    p.q_stride_b, p.q_stride_s, p.q_stride_h = Q.data.stride(0), Q.data.stride(1), Q.data.stride(2)
    p.k_stride_b, p.k_stride_s, p.k_stride_h = K.data.stride(0), K.data.stride(1), K.data.stride(2)
    p.v_stride_b, p.v_stride_h, p.v_stride_d = V.data.stride(0), V.data.stride(1), V.data.stride(2)
    p.o_stride_b, p.o_stride_s, p.o_stride_h = out.stride(0), out.stride(1), out.stride(2)
    p.B, p.Sq, p.Sk, p.Hq, p.Hkv, p.D, p.Dv = B, Sq, Sk, Hq, Hkv, D, Dv
    p.causal = 1 if causal else 0
    p.q_scale, p.k_scale, p.v_scale = Q.scale, K.scale, V.scale
    p.softmax_scale = D ** -0.5
    return p


def _free_bytes(dev):
    # free device memory as the driver sees it: an allocation made inside the library (which
    # torch's own counters cannot see) would show here
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info(dev)[0]


@pytest.mark.gpu
def test_noalloc_entry_matches_regular_entry_twice_in_a_row(cuda_device):
    dev = cuda_device
    L = fa.lib()
    stream = torch.cuda.current_stream(dev).cuda_stream
    # The larger problem first, so that later calls find the array full of other data.  The
    # ragged cases (rows and keys that do not fill their last tile, head dims 64 and (192, 128))
    # read zero padding that each call has to rewrite over whatever the previous call left.
    cases = [(2, 512, 384, 4, 2, 128, 128, True, 21), (1, 128, 256, 2, 1, 128, 128, False, 22),
             (1, 200, 160, 4, 2, 64, 64, True, 23), (2, 72, 96, 2, 2, 192, 128, False, 24),
             (1, 130, 32, 2, 1, 128, 128, False, 25)]
    for (B, Sq, Sk, Hq, Hkv, D, Dv, causal, seed) in cases:
        q, k, _ = make_qkv(B, Sq, Sk, Hq, Hkv, D, seed=seed, device=dev)
        _, _, v = make_qkv(B, Sq, Sk, Hq, Hkv, Dv, seed=seed + 100, device=dev)
        Q, K, V = fa.quantize_qkv(q, k, v)
        assert Q.sf.is_contiguous() and K.sf.is_contiguous() and V.sf.is_contiguous()
        want_o, want_l = fa.flash_attn_fp4_func(Q.data, K.data, V.data, Q.sf, K.sf, V.sf, Q.scale,
                                                K.scale, V.scale, causal=causal, return_lse=True)
        out = torch.full((B, Sq, Hq, Dv), float("nan"), dtype=torch.bfloat16, device=dev)
        lse = torch.full((B, Hq, Sq), float("nan"), dtype=torch.float32, device=dev)
        status = DeviceStatus.word(dev)
        p = _params(Q, K, V, out, lse, causal, status, D, Dv)
        # warm the entry point once so that loading the library image on this device (a one-off
        # cost of the first call) is not mistaken for a per-call allocation
        assert L.fa4_nvfp4_fwd_linear_sf_noalloc(ctypes.byref(p), stream) == 0
        before_torch, before_free = torch.cuda.memory_allocated(dev), _free_bytes(dev)
        rc = L.fa4_nvfp4_fwd_linear_sf_noalloc(ctypes.byref(p), stream)
        assert rc == 0
        assert torch.cuda.memory_allocated(dev) == before_torch   # nothing from torch's allocator
        assert _free_bytes(dev) >= before_free                    # nothing from cudaMalloc either
        fa.check_status(dev)
        # same kernels on the same bytes: tolerance zero
        assert torch.equal(out, want_o) and torch.equal(lse, want_l), (B, Sq, Sk, D)


def _dummy_params():
    """A call that fits the array and is well formed, on pointers that are never dereferenced by
    the host-side checks."""
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


@pytest.mark.parametrize("field,value,code", [
    ("q", 0, -1),                 # NULL operand
    ("out", 0x1008, -4),          # misaligned output
    ("D", 96, -2),                # head dim that is not built
    ("v_stride_d", 24, -3),       # V rows not padded to whole 32-key groups
    ("Hkv", 3, -2),               # Hq not a multiple of Hkv
    ("k_stride_s", 8, -3),        # 8-byte stride
    ("softmax_scale", 0.0, -2),
    ("variant", 9, -5),
    ("variant", 4, -2),           # decode variant on a prefill shape (and it would need a workspace)
])
def test_noalloc_entry_validates_the_forward_before_anything_runs(field, value, code):
    """Runs without a GPU: the calls fit the array but are bad for the forward.  Every one must come back with its negative argument code.
    Had the entry point started its layout kernels first, the result on a machine without a GPU
    would be a positive CUDA error instead, and on a GPU the shared array would already have
    been overwritten under a concurrent caller."""
    L = fa.lib()
    p = _dummy_params()
    setattr(p, field, value)
    assert L.fa4_nvfp4_fwd_linear_sf_noalloc(ctypes.byref(p), None) == code


def test_noalloc_entry_rejects_what_does_not_fit():
    """Host-side checks only: no GPU work is started for a rejected call."""
    L = fa.lib()
    p = _dummy_params()
    p.B, p.Sq, p.Sk, p.Hq, p.Hkv, p.D, p.Dv = 8, 8192, 8192, 32, 8, 128, 128   # 24 MiB of scales
    assert L.fa4_nvfp4_fwd_linear_sf_noalloc(ctypes.byref(p), None) == -8
    p.struct_size = 4
    assert L.fa4_nvfp4_fwd_linear_sf_noalloc(ctypes.byref(p), None) == -7
    assert L.fa4_nvfp4_fwd_linear_sf_noalloc(None, None) == -1
