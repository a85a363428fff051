"""K-cache quantisers on the GPU, with the reference's function names and return values.

Each function is one or two streaming CUDA passes (``ffa_quantize_*`` in libffa_b200.so) that
reproduce the reference's torch implementation bit for bit on the same K:

====================================  =====================================================
this module                           reference
====================================  =====================================================
``quantize_k_2bit_fp8_residual``      ffa-q2fp8/fused_kproj_rope_q2fp8.py:40-68
``quantize_k_fp8_fp8_residual``       ffa-fp8fp8/fused_kproj_rope_fp8fp8.py:58-64
``encode_k_fp4_fp8_residual``         ffa-fp4fp8/fused_kproj_rope_fp4fp8.py:40-73
``encode_k_nf4_fp8_residual``         ffa-nf4fp8/fused_kproj_rope_nf4fp8.py:72-96
``encode_k_nvfp4_fp8_residual``       ffa-nvfp4fp8/fused_kproj_rope_nvfp4fp8.py:62-114
====================================  =====================================================
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib


def _prep(k: torch.Tensor, fp8_dtype: torch.dtype):
    if not k.is_cuda:
        raise ValueError("k must be a CUDA tensor (this build has no CPU path)")
    if k.dim() != 4 or k.shape[-1] != 128:
        raise ValueError(f"k must be [B, T, HKV, 128], got {tuple(k.shape)}")
    if k.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise ValueError(f"k must be float16, bfloat16 or float32, got {k.dtype}")
    k = k.contiguous()
    B, T, HKV, D = k.shape
    return k, B, T, HKV, _lib.float_code(k.dtype), _lib.fp8_code(fp8_dtype), _lib.current_stream(k.device)


def _scratch(B: int, HKV: int, device) -> torch.Tensor:
    return torch.empty(_lib.lib().ffa_quantize_scratch_bytes(B, HKV), dtype=torch.uint8, device=device)


def minmax_scratch(B: int, HKV: int, device) -> torch.Tensor:
    """Scratch buffer of the 2-bit / NF4 quantisers.  Passed as ``scratch=`` it holds, after the call,
    the per-channel (min, max) of K as ordered integers: the running statistics that
    ``quantize_append`` keeps up to date."""
    return _scratch(B, HKV, device)


def quantize_k_2bit_fp8_residual(k: torch.Tensor, fp8_dtype: torch.dtype, *, scratch: Optional[torch.Tensor] = None
                                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """-> (codes [B,T,HKV,32] u8, scale [B,HKV,128], zero [B,HKV,128], residual [B,T,HKV,128] fp8)."""
    k, B, T, HKV, dt, f8, st = _prep(k, fp8_dtype)
    codes = torch.empty((B, T, HKV, 32), dtype=torch.uint8, device=k.device)
    scale = torch.empty((B, HKV, 128), dtype=k.dtype, device=k.device)
    zero = torch.empty_like(scale)
    res = torch.empty((B, T, HKV, 128), dtype=fp8_dtype, device=k.device)
    if scratch is None:
        scratch = _scratch(B, HKV, k.device)
    _lib.check(_lib.lib().ffa_quantize_q2(k.data_ptr(), dt, B, T, HKV, f8, codes.data_ptr(), scale.data_ptr(),
                                          zero.data_ptr(), res.data_ptr(), scratch.data_ptr(), st), "ffa_quantize_q2")
    return codes, scale, zero, res


def quantize_k_fp8_fp8_residual(k: torch.Tensor, fp8_dtype: torch.dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (base [B,T,HKV,128] fp8, residual [B,T,HKV,128] fp8)."""
    k, B, T, HKV, dt, f8, st = _prep(k, fp8_dtype)
    base = torch.empty((B, T, HKV, 128), dtype=fp8_dtype, device=k.device)
    res = torch.empty_like(base)
    _lib.check(_lib.lib().ffa_quantize_fp8fp8(k.data_ptr(), dt, B, T, HKV, f8, base.data_ptr(), res.data_ptr(), st),
               "ffa_quantize_fp8fp8")
    return base, res


def encode_k_fp4_fp8_residual(k: torch.Tensor, fp8_dtype: torch.dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (nibbles [B,T,HKV,64] u8, residual fp8)."""
    k, B, T, HKV, dt, f8, st = _prep(k, fp8_dtype)
    codes = torch.empty((B, T, HKV, 64), dtype=torch.uint8, device=k.device)
    res = torch.empty((B, T, HKV, 128), dtype=fp8_dtype, device=k.device)
    _lib.check(_lib.lib().ffa_quantize_fp4(k.data_ptr(), dt, B, T, HKV, f8, codes.data_ptr(), res.data_ptr(), st),
               "ffa_quantize_fp4")
    return codes, res


def encode_k_nf4_fp8_residual(k: torch.Tensor, fp8_dtype: torch.dtype, *, scratch: Optional[torch.Tensor] = None
                              ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """-> (nibbles [B,T,HKV,64] u8, absmax [B,HKV,128] in k's dtype, residual fp8)."""
    k, B, T, HKV, dt, f8, st = _prep(k, fp8_dtype)
    codes = torch.empty((B, T, HKV, 64), dtype=torch.uint8, device=k.device)
    scale = torch.empty((B, HKV, 128), dtype=k.dtype, device=k.device)
    res = torch.empty((B, T, HKV, 128), dtype=fp8_dtype, device=k.device)
    if scratch is None:
        scratch = _scratch(B, HKV, k.device)
    _lib.check(_lib.lib().ffa_quantize_nf4(k.data_ptr(), dt, B, T, HKV, f8, codes.data_ptr(), scale.data_ptr(),
                                           res.data_ptr(), scratch.data_ptr(), st), "ffa_quantize_nf4")
    return codes, scale, res


def encode_k_nvfp4_fp8_residual(k: torch.Tensor, fp8_dtype: torch.dtype, page_size: int
                                ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """-> (nibbles [B,T,HKV,64] u8, scale [B, ceil(T/page), HKV] in k's dtype, residual fp8)."""
    if page_size <= 0:
        raise ValueError(f"page_size must be positive, got {page_size}")
    k, B, T, HKV, dt, f8, st = _prep(k, fp8_dtype)
    n_pages = -(-T // page_size)
    codes = torch.empty((B, T, HKV, 64), dtype=torch.uint8, device=k.device)
    scale = torch.empty((B, n_pages, HKV), dtype=k.dtype, device=k.device)
    res = torch.empty((B, T, HKV, 128), dtype=fp8_dtype, device=k.device)
    _lib.check(_lib.lib().ffa_quantize_nvfp4(k.data_ptr(), dt, B, T, HKV, f8, page_size, codes.data_ptr(),
                                             scale.data_ptr(), res.data_ptr(), st), "ffa_quantize_nvfp4")
    return codes, scale, res


def quantize_append(kind: str, k_new: torch.Tensor, codes_pool: torch.Tensor, residual_pool: torch.Tensor,
                    block_table: torch.Tensor, position: int, *, fp8_dtype: torch.dtype,
                    scale: Optional[torch.Tensor] = None, zero: Optional[torch.Tensor] = None,
                    running_minmax: Optional[torch.Tensor] = None) -> None:
    """Encode ``k_new [B, T_new, HKV, 128]`` against the scales the cache already has and write codes and
    residual into the page slots of positions ``position ..`` (``ffa_quantize_append``): q2 needs
    ``scale`` and ``zero``, nf4 ``scale``; fp8 / fp4 have none.  ``running_minmax`` is the scratch buffer
    of the whole-sequence quantiser; the new tokens' extremes are folded into it."""
    k_new, B, T_new, HKV, dt, f8, st = _prep(k_new, fp8_dtype)
    if kind not in ("q2", "nf4", "fp8", "fp4"):
        raise ValueError(f"quantize_append serves q2, nf4, fp8 and fp4, got {kind!r}")
    scratch = _scratch(B, HKV, k_new.device) if kind == "nf4" else None
    ptr = lambda t: 0 if t is None else t.data_ptr()
    _lib.check(_lib.lib().ffa_quantize_append(
        _lib.VARIANT_CODE[kind], k_new.data_ptr(), dt, B, T_new, HKV, f8, codes_pool.data_ptr(), ptr(scale), ptr(zero),
        residual_pool.data_ptr(), ptr(running_minmax), ptr(scratch), block_table.data_ptr(), block_table.shape[1],
        int(position), st), "ffa_quantize_append")


# variant directory name of the reference -> short name of its coarse-K format
VARIANTS = {"fp8fp8": "fp8", "q2fp8": "q2", "fp4fp8": "fp4", "nf4fp8": "nf4", "nvfp4fp8": "nvfp4"}


def quantize_variant(kind: str, k: torch.Tensor, fp8_dtype: torch.dtype, page_size: int = 64):
    """``(codes, scale, zero, residual)`` of K in the format ``kind`` (a value of ``VARIANTS``); the
    parts a format does not have are ``None``."""
    if kind == "fp8":
        c, r = quantize_k_fp8_fp8_residual(k, fp8_dtype)
        return c, None, None, r
    if kind == "q2":
        return quantize_k_2bit_fp8_residual(k, fp8_dtype)
    if kind == "fp4":
        c, r = encode_k_fp4_fp8_residual(k, fp8_dtype)
        return c, None, None, r
    if kind == "nf4":
        c, s, r = encode_k_nf4_fp8_residual(k, fp8_dtype)
        return c, s, None, r
    if kind == "nvfp4":
        c, s, r = encode_k_nvfp4_fp8_residual(k, fp8_dtype, page_size)
        return c, s, None, r
    raise ValueError(f"unknown coarse-K format {kind!r}")
