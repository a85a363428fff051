"""NF4 K (per-channel absmax) + fp8 residual decode attention.

Drop-in for ffa-nf4fp8/attn_kernel/attn_kernel_v1210_fused_bsz_nf4fp8.py (:212-330 there)."""
from __future__ import annotations

import torch

from ...decode import DecodeWorkspace, allocate_decode_workspace, check_common, check_layout, decode_call

NF4_CODEBOOK_VALUES = (
    -1.0, -0.6961928009986877, -0.5229921340942383, -0.39491748809814453,
    -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
    0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
    0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0,
)
allocate_nf4_decode_workspace = allocate_decode_workspace


def _normalize_scale(k_scale: torch.Tensor, expect_shape):
    if k_scale.ndim == 4 and k_scale.shape[1] == 1:
        k_scale = k_scale.squeeze(1)
    if k_scale.shape != expect_shape:
        raise ValueError(f"Unsupported k_scale shape: {k_scale.shape=}, expected {expect_shape}")
    return k_scale.contiguous()


def attn_forward_decode_nf4(
    q: torch.Tensor,        # [B, 1, HQ, K]
    k_nf4: torch.Tensor,    # [B, T, HKV, K/2] uint8, two NF4 indices per byte, first in the low nibble
    k_scale: torch.Tensor,  # [B, HKV, K] absmax per channel
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
    check_common(q, k_nf4, v, k_residual, "attn_forward_decode_nf4")
    if k_bits != 4:
        raise ValueError(f"attn_forward_decode_nf4 supports 4-bit keys, got k_bits={k_bits}")
    assert k_scale.is_cuda, "k_scale must be a CUDA tensor"
    if not k_scale.is_floating_point():
        raise ValueError("k_scale must be a floating point tensor for dequantization")
    if k_nf4.is_floating_point():
        raise ValueError("k_nf4 must contain packed NF4 indices in an integer tensor (e.g., uint8)")
    B, _, HQ, K = q.shape
    expected = (K + 1) // 2
    if k_nf4.shape[-1] != expected:
        raise ValueError(
            f"k_nf4 packed dim mismatch: got {k_nf4.shape[-1]}, expected {expected} for K={K}, k_bits={k_bits}")
    check_layout(q, k_nf4, v, k_residual, expected, block_table is not None)
    k_scale = _normalize_scale(k_scale, (B, k_nf4.shape[2], K))
    if use_fp8_residual and k_residual is None:
        raise ValueError("use_fp8_residual=True requires k_residual")
    return decode_call(
        "nf4", q, k_nf4, v, k_scale=k_scale, k_residual=k_residual, scale=scale, BS=BS, SBS=SBS, delta=delta,
        return_skip_ratio=return_skip_ratio, precomputed_threshold=precomputed_threshold,
        use_fp8_residual=use_fp8_residual, block_table=block_table, seq_len=seq_len, workspace=workspace, out=out,
        partial_out=partial_out, pages_per_chunk=pages_per_chunk, kernel=kernel)
