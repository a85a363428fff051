"""Block-scaled e2m1 (NVFP4-style, one scale per BS-token block and kv-head) K + fp8 residual
decode attention.

Drop-in for ffa-nvfp4fp8/attn_kernel/attn_kernel_v1210_fused_bsz_nvfp4fp8.py (:225-367 there)."""
from __future__ import annotations

import torch

from ...decode import DecodeWorkspace, allocate_decode_workspace, check_common, check_layout, decode_call

allocate_nvfp4fp8_decode_workspace = allocate_decode_workspace


def _normalize_k_scale(k_scale: torch.Tensor, expect_shape: tuple[int, int, int]) -> torch.Tensor:
    """Accept [B, NTB, HKV], [B, 1, NTB, HKV] or the transposed [B, HKV, NTB] (reference :213-222)."""
    if k_scale.ndim == 4 and k_scale.shape[1] == 1:
        k_scale = k_scale.squeeze(1)
    if k_scale.shape == (expect_shape[0], expect_shape[2], expect_shape[1]):
        k_scale = k_scale.permute(0, 2, 1)
    if k_scale.shape != expect_shape:
        raise ValueError(f"Unsupported k_scale shape: {k_scale.shape=} expected {expect_shape}")
    return k_scale.contiguous()


def attn_forward_decode_nvfp4fp8(
    q: torch.Tensor,        # [B, 1, HQ, K]
    k_fp4: torch.Tensor,    # [B, T, HKV, K/2] uint8 e2m1 nibbles
    k_scale: torch.Tensor,  # [B, NTB, HKV] (NTB = ceil(T/BS)) or [B, HKV, NTB]
    v: torch.Tensor,        # [B, T, HKV, V]
    *,
    k_residual: torch.Tensor | None = None,
    k_bits: int = 4,
    scale: float = None,
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
    assert k_scale.is_cuda
    check_common(q, k_fp4, v, k_residual, "attn_forward_decode_nvfp4fp8")
    if k_bits != 4:
        raise ValueError(f"attn_forward_decode_nvfp4fp8 supports 4-bit keys, got k_bits={k_bits}")
    if k_fp4.is_floating_point():
        raise ValueError("k_fp4 must contain packed FP4 (E2M1) nibbles in an integer tensor (e.g., uint8)")
    if not k_scale.is_floating_point():
        raise ValueError("k_scale must be a floating point tensor")
    B, _, HQ, K = q.shape
    expected = (K + 1) // 2
    if k_fp4.shape[-1] != expected:
        raise ValueError(
            f"k_fp4 packed dim mismatch: got {k_fp4.shape[-1]}, expected {expected} for K={K}, k_bits={k_bits}")
    check_layout(q, k_fp4, v, k_residual, expected, block_table is not None)
    T = seq_len if (block_table is not None and seq_len is not None) else (
        block_table.shape[1] * 64 if block_table is not None else k_fp4.shape[1])
    NTB = -(-T // BS)
    k_scale = _normalize_k_scale(k_scale, (B, NTB, k_fp4.shape[2]))
    if use_fp8_residual and k_residual is None:
        raise ValueError("use_fp8_residual=True requires k_residual")
    return decode_call(
        "nvfp4", q, k_fp4, v, k_scale=k_scale, k_residual=k_residual, scale=scale, BS=BS, SBS=SBS, delta=delta,
        return_skip_ratio=return_skip_ratio, precomputed_threshold=precomputed_threshold,
        use_fp8_residual=use_fp8_residual, block_table=block_table, seq_len=seq_len, workspace=workspace, out=out,
        partial_out=partial_out, pages_per_chunk=pages_per_chunk, kernel=kernel)
