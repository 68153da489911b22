"""TEST INFRASTRUCTURE ONLY - quantise-on-write / dequantise-on-read of the KV cache, restated.

Quantise (bytes must be bit-exact):
  INT8: int8 = cvt.rni.sat.s8.f32(float(x) * scale_f32)
        cpp/tensorrt_llm/kernels/decoderMaskedMultiheadAttentionUtils.h:3741-3749 (store), :3629-3639 (cvt)
  FP8 : scale is first rounded to the activation type T, the product scale_T * x_T is one
        multiplication in T (one rounding), then T -> e4m3 round-to-nearest-even, saturating
        decoderMaskedMultiheadAttentionUtils.h:3753-3763, :3824-3848 (scale type),
        decoderMaskedMultiheadAttention/decoderMaskedMultiheadAttentionTemplate.h:1510-1515 (scale convert)
  none: stored as T.
Dequantise: int8 -> float, e4m3 -> float; the per-tensor scale is applied by the caller.
"""
from __future__ import annotations

import torch

CACHE_T, CACHE_INT8, CACHE_FP8 = 0, 1, 2


def int8_from_f32(x: torch.Tensor) -> torch.Tensor:
    """cvt.rni.sat.s8.f32: round half to even, saturate to [-128, 127]."""
    return torch.round(x.to(torch.float32)).clamp_(-128, 127).to(torch.int8)


def fp8_from_f32(x: torch.Tensor) -> torch.Tensor:
    """float -> e4m3, round to nearest even, saturating to +-448 (__NV_SATFINITE); returns uint8."""
    return x.to(torch.float32).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)


def quantize_kv(x: torch.Tensor, scale_orig_quant: float, mode: int) -> torch.Tensor:
    """x: tensor of the activation dtype T (fp16/bf16), any shape [..., Dh].
    Returns uint8 bytes of shape [..., Dh * elem_bytes] exactly as the cache stores them."""
    assert x.dtype in (torch.float16, torch.bfloat16)
    if mode == CACHE_T:
        return x.contiguous().view(torch.uint8)
    s32 = torch.tensor(scale_orig_quant, dtype=torch.float32)
    if mode == CACHE_INT8:
        # one fp32 multiply, round half to even (torch.round), saturate
        return int8_from_f32(x.to(torch.float32) * s32).view(torch.uint8)
    if mode == CACHE_FP8:
        st = s32.to(x.dtype)
        prod = x * st  # one rounding to T (the exact product fits fp32)
        return fp8_from_f32(prod.to(torch.float32))
    raise ValueError(mode)


def dequantize_kv(raw: torch.Tensor, mode: int, dtype: torch.dtype) -> torch.Tensor:
    """raw: uint8 [..., Dh * elem_bytes] -> float32 [..., Dh], without the per-tensor scale."""
    if mode == CACHE_T:
        return raw.contiguous().view(dtype).to(torch.float32)
    if mode == CACHE_INT8:
        return raw.view(torch.int8).to(torch.float32)
    if mode == CACHE_FP8:
        return raw.view(torch.float8_e4m3fn).to(torch.float32)
    raise ValueError(mode)
