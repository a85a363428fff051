"""Fused K-projection + RoPE + fp8 cache quantisation.

Drop-in for ffa-fp8fp8/fused_kproj_rope_fp8fp8.py (67-135 there): ``kproj_rope_quantize_reference``, ``kproj_rope_quantize_triton`` and
``kproj_rope_quantize_fused`` with the reference's arguments and return tuple, plus the RoPE helpers and the
quantiser it re-exports.  ``_triton`` and ``_fused`` run the tcgen05 GEMM of libffa_b200 (the name is
kept for callers of the reference; no Triton is involved)."""
from __future__ import annotations

from typing import Optional

import torch

from ..kproj import (_normalize_k_weight, _resolve_fp8_dtype, apply_rope, build_rope_cache, kproj_fused,
                     kproj_reference, rotate_half)
from ..quantize import quantize_k_fp8_fp8_residual

__all__ = ["build_rope_cache", "rotate_half", "apply_rope", "quantize_k_fp8_fp8_residual", "kproj_rope_quantize_reference", "kproj_rope_quantize_triton",
           "kproj_rope_quantize_fused"]


def kproj_rope_quantize_reference(h, w_k, cos, sin, num_kv_heads: int, head_dim: int, bias: Optional[torch.Tensor] = None,
                                  fp8_dtype: Optional[torch.dtype] = None):
    return kproj_reference("fp8", h, w_k, cos, sin, num_kv_heads, head_dim, bias, fp8_dtype)


def kproj_rope_quantize_triton(h, w_k, cos, sin, num_kv_heads: int, head_dim: int, bias: Optional[torch.Tensor] = None,
                               fp8_dtype: Optional[torch.dtype] = None, block_table=None, out=None, return_k: bool = False,
                               **_tile_kwargs):
    """``_tile_kwargs`` swallows the Triton tile knobs of the reference (block_t, block_h, block_pair,
    num_warps, num_stages); the GEMM tile here is fixed."""
    return kproj_fused("fp8", h, w_k, cos, sin, num_kv_heads, head_dim, bias, fp8_dtype,
                       block_table=block_table, out=out, return_k=return_k)


def kproj_rope_quantize_fused(h, w_k, cos, sin, num_kv_heads: int, head_dim: int, bias: Optional[torch.Tensor] = None,
                              fp8_dtype: Optional[torch.dtype] = None, block_table=None, out=None, return_k: bool = False):
    return kproj_fused("fp8", h, w_k, cos, sin, num_kv_heads, head_dim, bias, fp8_dtype,
                       block_table=block_table, out=out, return_k=return_k)
