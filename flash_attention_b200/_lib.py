"""ctypes binding of libfa4_nvfp4.so (the C ABI declared in include/fa4_nvfp4.h).

The library is built in-tree by ``build()`` with a plain ``nvcc`` command (no JIT cache, no
torch extension machinery) and loaded lazily.  There is no fallback: if the library is missing
or cannot be loaded, every operator of this package raises.
"""
from __future__ import annotations

import ctypes
import fcntl
import glob
import os
import shutil
import subprocess
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfa4_nvfp4.so")
CSRC = os.path.join(_HERE, "csrc")
LOCK_PATH = os.path.join(_HERE, ".build.lock")
SOURCES = ["api.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--shared", "-Xcompiler", "-fPIC"]

ERROR_NAMES = {1: "null pointer", 2: "unsupported shape", 3: "bad stride", 4: "misaligned pointer",
               5: "unknown variant", 6: "tensor map rejected", 7: "struct size mismatch",
               8: "problem too large for this entry point",
               9: "library built with a register count its kernels cannot run with"}


class Params(ctypes.Structure):
    """Mirror of ``fa4_nvfp4_params``."""
    _fields_ = [
        ("struct_size", ctypes.c_uint32), ("variant", ctypes.c_int32),
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p),
        ("q_sf", ctypes.c_void_p), ("k_sf", ctypes.c_void_p), ("v_sf", ctypes.c_void_p),
        ("out", ctypes.c_void_p), ("lse", ctypes.c_void_p), ("status", ctypes.c_void_p),
        ("q_stride_b", ctypes.c_int64), ("q_stride_s", ctypes.c_int64), ("q_stride_h", ctypes.c_int64),
        ("k_stride_b", ctypes.c_int64), ("k_stride_s", ctypes.c_int64), ("k_stride_h", ctypes.c_int64),
        ("v_stride_b", ctypes.c_int64), ("v_stride_h", ctypes.c_int64), ("v_stride_d", ctypes.c_int64),
        ("o_stride_b", ctypes.c_int64), ("o_stride_s", ctypes.c_int64), ("o_stride_h", ctypes.c_int64),
        ("B", ctypes.c_int32), ("Sq", ctypes.c_int32), ("Sk", ctypes.c_int32), ("Hq", ctypes.c_int32),
        ("Hkv", ctypes.c_int32), ("D", ctypes.c_int32), ("Dv", ctypes.c_int32),
        ("causal", ctypes.c_int32),
        ("q_scale", ctypes.c_float), ("k_scale", ctypes.c_float), ("v_scale", ctypes.c_float),
        ("softmax_scale", ctypes.c_float),
        ("wait_budget_ns", ctypes.c_uint64),
    ]


class Ext(ctypes.Structure):
    """Mirror of ``fa4_nvfp4_ext``."""
    _fields_ = [
        ("struct_size", ctypes.c_uint32), ("num_splits", ctypes.c_int32),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_uint64),
        ("window_left", ctypes.c_int32), ("window_right", ctypes.c_int32),
        ("sink", ctypes.c_void_p), ("softcap", ctypes.c_float), ("reserved", ctypes.c_uint32),
        ("seqused_k", ctypes.c_void_p), ("page_table", ctypes.c_void_p),
        ("page_size", ctypes.c_int32), ("pages_per_seq", ctypes.c_int32),
        ("num_pages", ctypes.c_int32), ("reserved2", ctypes.c_int32),
    ]


class Varlen(ctypes.Structure):
    """Mirror of ``fa4_nvfp4_varlen``."""
    _fields_ = [
        ("struct_size", ctypes.c_uint32), ("num_seqs", ctypes.c_int32),
        ("cu_seqlens_q", ctypes.c_void_p), ("cu_seqlens_k", ctypes.c_void_p), ("seqused_k", ctypes.c_void_p),
        ("total_q", ctypes.c_int32), ("total_k", ctypes.c_int32),
        ("max_seqlen_q", ctypes.c_int32), ("max_seqlen_k", ctypes.c_int32),
        ("window_left", ctypes.c_int32), ("window_right", ctypes.c_int32),
        ("sink", ctypes.c_void_p), ("softcap", ctypes.c_float), ("reserved", ctypes.c_uint32),
        ("cu_seqlens_v", ctypes.c_void_p), ("total_v", ctypes.c_int32), ("reserved2", ctypes.c_int32),
    ]


def _dependencies():
    """Every file the library is compiled from: all of csrc/ and the public header."""
    deps = sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cuh")))
    deps.append(os.path.join(_HERE, "..", "include", "fa4_nvfp4.h"))
    return deps


def _needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in _dependencies())


class _BuildLock:
    """Inter-process lock around build and load: the ranks of one node share the source tree, and
    a rank must never load a library another rank is still writing."""

    def __enter__(self):
        self.f = open(LOCK_PATH, "w")
        fcntl.flock(self.f, fcntl.LOCK_EX)
        return self

    def __exit__(self, *exc):
        fcntl.flock(self.f, fcntl.LOCK_UN)
        self.f.close()


def _compile(verbose: bool) -> None:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    tmp = f"{LIB_PATH}.{os.getpid()}.tmp"
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
          ["-o", tmp] + [os.path.join(CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    os.replace(tmp, LIB_PATH)       # readers see the old file or the complete new one
    if verbose:
        print(res.stderr)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the CUDA library for sm_100a (cross-compiles without a GPU)."""
    with _BuildLock():
        if force or _needs_build():
            _compile(verbose)
    return LIB_PATH


_lib = None
_lock = threading.Lock()


def lib() -> ctypes.CDLL:
    """The loaded library.  Raises if it is absent (built on demand only when nvcc is present)."""
    global _lib
    with _lock:
        if _lib is None:
            with _BuildLock():
                if _needs_build():
                    if shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc"):
                        _compile(False)
                    elif not os.path.exists(LIB_PATH):
                        raise RuntimeError(f"{LIB_PATH} is missing and nvcc is not available; "
                                           "run flash_attention_b200.build() first")
                L = ctypes.CDLL(LIB_PATH)
            L.fa4_nvfp4_fwd.argtypes = [ctypes.POINTER(Params), ctypes.c_void_p]
            L.fa4_nvfp4_fwd.restype = ctypes.c_int
            L.fa4_nvfp4_splitkv_workspace_bytes.argtypes = [ctypes.POINTER(Params), ctypes.c_int32]
            L.fa4_nvfp4_splitkv_workspace_bytes.restype = ctypes.c_int64
            L.fa4_nvfp4_fwd_splitkv.argtypes = [ctypes.POINTER(Params), ctypes.c_int32, ctypes.c_void_p,
                                                ctypes.c_uint64, ctypes.c_void_p]
            L.fa4_nvfp4_fwd_splitkv.restype = ctypes.c_int
            L.fa4_nvfp4_fwd_ex.argtypes = [ctypes.POINTER(Params), ctypes.POINTER(Ext), ctypes.c_void_p]
            L.fa4_nvfp4_fwd_ex.restype = ctypes.c_int
            L.fa4_nvfp4_fwd_varlen.argtypes = [ctypes.POINTER(Params), ctypes.POINTER(Varlen), ctypes.c_void_p]
            L.fa4_nvfp4_fwd_varlen.restype = ctypes.c_int
            L.fa4_nvfp4_sf_linear_to_tiled_packed.argtypes = [
                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
            L.fa4_nvfp4_sf_linear_to_tiled_packed.restype = ctypes.c_int
            L.fa4_nvfp4_sf_linear_to_tiled.argtypes = [
                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32,
                ctypes.c_void_p]
            L.fa4_nvfp4_sf_linear_to_tiled.restype = ctypes.c_int
            L.fa4_nvfp4_query.argtypes = [ctypes.c_int32]
            L.fa4_nvfp4_query.restype = ctypes.c_int
            L.fa4_nvfp4_debug_qk_tile.argtypes = [ctypes.c_void_p] * 5 + [
                ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]
            L.fa4_nvfp4_debug_qk_tile.restype = ctypes.c_int
            L.fa4_nvfp4_debug_wait_expiry.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p]
            L.fa4_nvfp4_debug_wait_expiry.restype = ctypes.c_int
            L.fa4_nvfp4_debug_mma_rate.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p,
                                                   ctypes.c_void_p, ctypes.c_void_p]
            L.fa4_nvfp4_debug_mma_rate.restype = ctypes.c_int
            L.fa4_nvfp4_debug_ex2_rate.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p,
                                                   ctypes.c_void_p, ctypes.c_void_p]
            L.fa4_nvfp4_debug_ex2_rate.restype = ctypes.c_int
            L.fa4_nvfp4_amax_bf16.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32,
                                              ctypes.c_int32, ctypes.c_int32, ctypes.c_int64,
                                              ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                              ctypes.c_void_p]
            L.fa4_nvfp4_amax_bf16.restype = ctypes.c_int
            for fn in (L.fa4_nvfp4_quantize_qk_bf16, L.fa4_nvfp4_quantize_v_bf16):
                fn.argtypes = [ctypes.c_void_p] + [ctypes.c_int32] * 4 + [ctypes.c_int64] * 3 + \
                              [ctypes.c_void_p] * 6
                fn.restype = ctypes.c_int
            L.fa4_nvfp4_fwd_linear_sf_noalloc.argtypes = [ctypes.POINTER(Params), ctypes.c_void_p]
            L.fa4_nvfp4_fwd_linear_sf_noalloc.restype = ctypes.c_int
            _lib = L
        return _lib


EXPORTS = ["fa4_nvfp4_fwd", "fa4_nvfp4_sf_linear_to_tiled", "fa4_nvfp4_query",
           "fa4_nvfp4_debug_qk_tile", "fa4_nvfp4_debug_wait_expiry", "fa4_nvfp4_debug_mma_rate",
           "fa4_nvfp4_debug_ex2_rate", "fa4_nvfp4_fwd_varlen", "fa4_nvfp4_sf_linear_to_tiled_packed",
           "fa4_nvfp4_fwd_linear_sf_noalloc", "fa4_nvfp4_amax_bf16", "fa4_nvfp4_quantize_qk_bf16",
           "fa4_nvfp4_quantize_v_bf16", "fa4_nvfp4_splitkv_workspace_bytes", "fa4_nvfp4_fwd_splitkv",
           "fa4_nvfp4_fwd_ex"]


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc < 0:
        raise ValueError(f"{what}: argument rejected ({ERROR_NAMES.get(-rc, rc)})")
    raise RuntimeError(f"{what}: CUDA error {rc}")
