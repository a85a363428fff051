"""2-bit K + fp8 residual decode attention, mean-V variant.

Takes the place of ffa-q2fp8-meanv/attn_kernel/attn_kernel_v1210_meanv_bsz_q2fp8.py (entry point
:222-343 there): pages whose coarse scores fall below the threshold are not dropped; each adds its
coarse softmax mass (relative maximum and sum of exp2 over its tokens, :107-119) to a scalar running
pair, and the merge adds that mass times the mean of V over the sequence (:169-200).  Same arguments
and return values as the plain 2-bit entry point; ``v_mean [B, HKV, V]`` may be passed to avoid the
pass over V that the reference makes on every call (:332).
"""
from __future__ import annotations

import torch

from ...decode import DecodeWorkspace, allocate_decode_workspace
from ...q2fp8.attn_kernel.attn_kernel_v1210_fused_bsz_q2fp8 import attn_forward_decode_quantized as _plain

Q2FP8DecodeWorkspace = DecodeWorkspace
allocate_q2fp8_decode_workspace = allocate_decode_workspace


def attn_forward_decode_quantized(q, k_q, k_scale, k_zero, v, k_residual=None, k_bits: int = 2, scale=None,
                                  BS: int = 128, SBS=None, delta: float = 5.0, return_skip_ratio: bool = False,
                                  precomputed_threshold=None, use_fp8_residual: bool = True, *,
                                  v_mean: torch.Tensor | None = None, **kwargs):
    if v_mean is None:
        if kwargs.get("block_table") is not None:
            raise ValueError("with a paged cache pass v_mean: the mean over a pool is not the mean over the sequence")
        v_mean = v.mean(dim=1, dtype=torch.float32).to(v.dtype).contiguous()
    return _plain(q, k_q, k_scale, k_zero, v, k_residual, k_bits, scale, BS, SBS, delta, return_skip_ratio,
                  precomputed_threshold, use_fp8_residual, mean_v=v_mean, **kwargs)
