"""CUDA-graph runner for the nvfp4fp8 decode call.

Drop-in for ffa-nvfp4fp8/attn_kernel/attn_kernel_v1210_fused_bsz_nvfp4fp8_cudagraph.py (11-178 there):
same constructor and ``replay`` arguments, ``output``, ``__call__`` and ``replay_only``."""
from __future__ import annotations

from typing import Optional

import torch

from ...cudagraph import GraphDecodeRunner
from .attn_kernel_v1210_fused_bsz_nvfp4fp8 import attn_forward_decode_nvfp4fp8


class CUDAGraphDecodeRunnerNVFP4FP8(GraphDecodeRunner):
    def __init__(
        self,
        q: torch.Tensor, k_fp4: torch.Tensor, k_scale: torch.Tensor, v: torch.Tensor,
        *,
        k_residual: Optional[torch.Tensor] = None,
        precomputed_threshold: Optional[torch.Tensor] = None,
        k_bits: int = 4,
        scale: Optional[float] = None,
        BS: int = 128,
        SBS: Optional[int] = None,
        delta: float = 5.0,
        use_fp8_residual: bool = True,
        warmup: int = 2,
        in_place: bool = False,
    ) -> None:
        if use_fp8_residual and k_residual is None:
            raise ValueError("use_fp8_residual=True requires k_residual")
        tensors = {"q": q, "k_fp4": k_fp4, "k_scale": k_scale, "v": v, "k_residual": k_residual if use_fp8_residual else None,
                   "precomputed_threshold": precomputed_threshold}
        super().__init__(attn_forward_decode_nvfp4fp8, tensors, "q", "v",
                         settings=dict(k_bits=k_bits, scale=scale, BS=BS, SBS=SBS, delta=delta,
                                       use_fp8_residual=use_fp8_residual),
                         warmup=warmup, in_place=in_place)

    def replay(
        self,
        q: torch.Tensor, k_fp4: torch.Tensor, k_scale: torch.Tensor, v: torch.Tensor,
        *,
        k_residual: Optional[torch.Tensor] = None,
        precomputed_threshold: Optional[torch.Tensor] = None,
        return_skip_ratio: bool = False,
    ):
        new = {"q": q, "k_fp4": k_fp4, "k_scale": k_scale, "v": v, "k_residual": k_residual, "precomputed_threshold": precomputed_threshold}
        return self._replay(new, return_skip_ratio)

    __call__ = replay
