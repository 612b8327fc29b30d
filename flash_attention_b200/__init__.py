"""B200 (sm_100a) NVFP4 fused attention forward behind the ``flash_attn.cute`` call surface.

Public names follow the reference's ``flash_attn/cute/__init__.py:11-18``.
"""
from ._lib import build, lib, LIB_PATH
from .interface import (flash_attn_func, flash_attn_fp4_func, check_status, measure_fp4_mma_rate, measure_ex2_rate,
                        VARIANT_AUTO,
                        VARIANT_WS, VARIANT_WS64, VARIANT_DECODE)
from .host_pipeline import HostPipeline, flash_attn_fp4_host
from .varlen import flash_attn_varlen_fp4_func, quantize_varlen_qkv, padded_key_offsets
from .quant import NVFP4Tensor, quantize_qkv, quantize_qkv_fused, quantize_lastdim, dequantize_lastdim, sf_to_tiled

__all__ = ["flash_attn_func", "flash_attn_fp4_func", "check_status", "HostPipeline", "flash_attn_fp4_host", "flash_attn_varlen_fp4_func", "quantize_varlen_qkv", "padded_key_offsets", "measure_fp4_mma_rate", "measure_ex2_rate", "NVFP4Tensor", "quantize_qkv", "quantize_qkv_fused",
           "quantize_lastdim", "dequantize_lastdim", "sf_to_tiled", "build", "lib", "LIB_PATH",
           "VARIANT_AUTO", "VARIANT_WS", "VARIANT_WS64", "VARIANT_DECODE"]
