"""2-bit K + fp8 residual decode attention.

Drop-in for ffa-q2fp8/attn_kernel/attn_kernel_v1210_fused_bsz_q2fp8.py: same entry point
name, arguments, exceptions and return values (:191-309 there); the work is done by
``ffa_decode`` in libffa_b200.so.  ``workspace`` / ``allocate_q2fp8_decode_workspace`` follow
the H100-tuned sibling (ffa-q2fp8-h100/attn_kernel/attn_kernel_v1210_fused_bsz_q2fp8.py:232-277).
"""
from __future__ import annotations

import torch

from ...decode import DecodeWorkspace, allocate_decode_workspace, check_common, check_layout, decode_call

Q2FP8DecodeWorkspace = DecodeWorkspace
allocate_q2fp8_decode_workspace = allocate_decode_workspace


def _normalize_scale_zero(k_scale: torch.Tensor, k_zero: torch.Tensor, expect_shape):
    """Accept [B, 1, HKV, K] or [B, HKV, K]; return contiguous [B, HKV, K] (reference :174-188)."""
    if k_scale.ndim == 4 and k_scale.shape[1] == 1:
        k_scale = k_scale.squeeze(1)
    if k_zero.ndim == 4 and k_zero.shape[1] == 1:
        k_zero = k_zero.squeeze(1)
    if k_scale.shape != expect_shape or k_zero.shape != expect_shape:
        raise ValueError(
            f"Unsupported k_scale/k_zero shapes: {k_scale.shape=} {k_zero.shape=}, expected {expect_shape}")
    return k_scale.contiguous(), k_zero.contiguous()


def attn_forward_decode_quantized(
    q: torch.Tensor,            # [B, 1, HQ, K]
    k_q: torch.Tensor,          # [B, T, HKV, K/4] uint8, four 2-bit codes per byte, first code in the low bits
    k_scale: torch.Tensor,      # [B, HKV, K]
    k_zero: torch.Tensor,       # [B, HKV, K]
    v: torch.Tensor,            # [B, T, HKV, V]
    k_residual: torch.Tensor | None = None,   # [B, T, HKV, K] fp8
    k_bits: int = 2,
    scale: float = None,
    BS: int = 128,
    SBS: int | None = None,
    delta: float = 5.0,
    return_skip_ratio: bool = False,
    precomputed_threshold: torch.Tensor | None = None,
    use_fp8_residual: bool = True,
    *,
    block_table: torch.Tensor | None = None,
    seq_len: int | None = None,
    workspace: DecodeWorkspace | None = None,
    out: torch.Tensor | None = None,
    partial_out: torch.Tensor | None = None,
    pages_per_chunk: int = 0,
    kernel: str = "auto",
    mean_v: torch.Tensor | None = None,
    **kwargs,
):
    check_common(q, k_q, v, k_residual, "attn_forward_decode_quantized")
    if k_bits != 2:
        raise ValueError(f"attn_forward_decode_quantized currently supports 2-bit keys, got k_bits={k_bits}")
    assert k_scale.is_cuda and k_zero.is_cuda, "k_scale/k_zero must be CUDA tensors"
    if not k_scale.is_floating_point() or not k_zero.is_floating_point():
        raise ValueError("k_scale and k_zero must be floating point tensors for dequantization")
    if k_q.is_floating_point():
        raise ValueError("k_q must contain integer quantized values (e.g., uint8/int8)")
    B, _, HQ, K = q.shape
    HKV = k_q.shape[2]
    expected = (K + 3) // 4
    if k_q.shape[-1] != expected:
        raise ValueError(
            f"k_q packed dim mismatch: got {k_q.shape[-1]}, expected {expected} for K={K}, k_bits={k_bits}")
    check_layout(q, k_q, v, k_residual, expected, block_table is not None)
    k_scale, k_zero = _normalize_scale_zero(k_scale, k_zero, (B, HKV, K))
    if k_scale.dtype != k_zero.dtype:
        k_zero = k_zero.to(k_scale.dtype)
    if use_fp8_residual and k_residual is None:
        raise ValueError("use_fp8_residual=True requires k_residual")
    return decode_call(
        "q2", q, k_q, v, k_scale=k_scale, k_zero=k_zero, k_residual=k_residual, scale=scale, BS=BS, SBS=SBS,
        delta=delta, return_skip_ratio=return_skip_ratio, precomputed_threshold=precomputed_threshold,
        use_fp8_residual=use_fp8_residual, block_table=block_table, seq_len=seq_len, workspace=workspace, out=out,
        partial_out=partial_out, pages_per_chunk=pages_per_chunk, kernel=kernel, mean_v=mean_v)
