"""fp8 K + fp8 residual decode attention.

Drop-in for ffa-fp8fp8/attn_kernel/attn_kernel_v1210_fused_bsz_fp8fp8.py (:180-312 there)."""
from __future__ import annotations

import torch

from ...decode import DecodeWorkspace, allocate_decode_workspace, check_common, check_layout, decode_call

allocate_fp8fp8_decode_workspace = allocate_decode_workspace


def attn_forward_decode_fp8fp8(
    q: torch.Tensor,        # [B, 1, HQ, K]
    k_fp8: torch.Tensor,    # [B, T, HKV, K] fp8
    v: torch.Tensor,        # [B, T, HKV, V]
    *,
    k_residual: torch.Tensor | None = None,   # [B, T, HKV, K] fp8
    scale: float | None = None,
    BS: int = 128,
    SBS: int | None = None,
    delta: float = 5.0,
    return_skip_ratio: bool = False,
    precomputed_threshold: torch.Tensor | None = None,
    use_fp8_residual: bool = True,
    block_table: torch.Tensor | None = None,
    seq_len: int | None = None,
    workspace: DecodeWorkspace | None = None,
    out: torch.Tensor | None = None,
    partial_out: torch.Tensor | None = None,
    pages_per_chunk: int = 0,
    kernel: str = "auto",
    **kwargs,
):
    check_common(q, k_fp8, v, k_residual, "attn_forward_decode_fp8fp8")
    if not k_fp8.is_floating_point():
        raise ValueError("k_fp8 must be a floating point tensor (fp8/fp16/bf16)")
    check_layout(q, k_fp8, v, k_residual, q.shape[-1], block_table is not None)
    if q.shape[2] % k_fp8.shape[2] != 0:
        raise ValueError(f"HQ ({q.shape[2]}) must be divisible by HKV ({k_fp8.shape[2]}) for GQA")
    if use_fp8_residual and k_residual is None:
        raise ValueError("use_fp8_residual=True requires k_residual")
    return decode_call(
        "fp8", q, k_fp8, v, k_residual=k_residual, scale=scale, BS=BS, SBS=SBS, delta=delta,
        return_skip_ratio=return_skip_ratio, precomputed_threshold=precomputed_threshold,
        use_fp8_residual=use_fp8_residual, block_table=block_table, seq_len=seq_len, workspace=workspace, out=out,
        partial_out=partial_out, pages_per_chunk=pages_per_chunk, kernel=kernel)
