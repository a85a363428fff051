"""Unscaled e2m1 (fp4) K + fp8 residual decode attention.

Drop-in for ffa-fp4fp8/attn_kernel/attn_kernel_v1210_fused_bsz_fp4fp8.py (:182-294 there)."""
from __future__ import annotations

import torch

from ...decode import DecodeWorkspace, allocate_decode_workspace, check_common, check_layout, decode_call

allocate_fp4_decode_workspace = allocate_decode_workspace


def attn_forward_decode_fp4(
    q: torch.Tensor,        # [B, 1, HQ, K]
    k_fp4: torch.Tensor,    # [B, T, HKV, K/2] uint8, two e2m1 nibbles per byte, first in the low nibble
    v: torch.Tensor,        # [B, T, HKV, V]
    k_residual: torch.Tensor | None = None,
    k_bits: int = 4,
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
    **kwargs,
):
    check_common(q, k_fp4, v, k_residual, "attn_forward_decode_fp4")
    if k_bits != 4:
        raise ValueError(f"attn_forward_decode_fp4 supports 4-bit keys, got k_bits={k_bits}")
    if k_fp4.is_floating_point():
        raise ValueError("k_fp4 must contain packed FP4 (E2M1) nibbles in an integer tensor (e.g., uint8)")
    K = q.shape[-1]
    expected = (K + 1) // 2
    if k_fp4.shape[-1] != expected:
        raise ValueError(
            f"k_fp4 packed dim mismatch: got {k_fp4.shape[-1]}, expected {expected} for K={K}, k_bits={k_bits}")
    check_layout(q, k_fp4, v, k_residual, expected, block_table is not None)
    if use_fp8_residual and k_residual is None:
        raise ValueError("use_fp8_residual=True requires k_residual")
    return decode_call(
        "fp4", q, k_fp4, v, k_residual=k_residual, scale=scale, BS=BS, SBS=SBS, delta=delta,
        return_skip_ratio=return_skip_ratio, precomputed_threshold=precomputed_threshold,
        use_fp8_residual=use_fp8_residual, block_table=block_table, seq_len=seq_len, workspace=workspace, out=out,
        partial_out=partial_out, pages_per_chunk=pages_per_chunk, kernel=kernel)
