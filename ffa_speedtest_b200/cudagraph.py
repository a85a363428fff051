"""CUDA-graph capture / replay of one decode step with static buffers.

Counterpart of the reference's ``CUDAGraphDecodeRunner*`` classes
(ffa-q2fp8/attn_kernel/attn_kernel_v1210_fused_bsz_q2fp8_cudagraph.py:11-183 and siblings): the
constructor copies every input into static buffers and captures one call; ``replay(...)`` copies
new inputs into those buffers and replays; ``replay_only()`` just replays; ``output`` is the
static output tensor (overwritten by every replay).

Differences that do not change results: the captured call uses a preallocated workspace, so the
graph contains exactly two kernels and no memset; a tensor passed to ``replay`` that already is
the static buffer is not copied; ``return_skip_ratio=True`` reads the kept mask the replay just
wrote instead of re-running the kernel eagerly as the reference does (:159-176).
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch

from .decode import DecodeWorkspace


class GraphDecodeRunner:
    """Shared machinery; the per-variant subclasses only name the tensors."""

    def __init__(self, entry: Callable, tensors: Dict[str, Optional[torch.Tensor]], q_name: str, v_name: str,
                 *, settings: dict, warmup: int = 2, in_place: bool = False):
        if not torch.cuda.is_available():
            raise RuntimeError("CUDA is required for CUDAGraph capture.")
        q, v = tensors[q_name], tensors[v_name]
        if q.device.type != "cuda":
            raise ValueError("q must be a CUDA tensor.")
        self._device = q.device
        self._entry = entry
        self._settings = dict(settings)
        self._names = [n for n, t in tensors.items() if t is not None]
        # static copies (or, with in_place=True, the caller's own tensors: a KV cache of many GiB
        # should not be duplicated just to be captured)
        self._static = {n: (tensors[n] if in_place else tensors[n].clone()) for n in self._names}
        BS = self._settings.get("BS", 128)
        SBS = self._settings.get("SBS") or BS
        self._ws = DecodeWorkspace.for_shape(q.shape[0], v.shape[1], q.shape[2], v.shape[2], v.shape[3], BS=BS, SBS=SBS,
                                             device=self._device, dtype=q.dtype)
        for _ in range(max(1, warmup)):
            self._call()
        torch.cuda.synchronize(self._device)
        self._graph = torch.cuda.CUDAGraph()
        self._pool = torch.cuda.graphs.graph_pool_handle()
        with torch.cuda.graph(self._graph, pool=self._pool):
            self._static_out = self._call()

    def _call(self):
        return self._entry(**self._static, **self._settings, return_skip_ratio=False, workspace=self._ws)

    @property
    def output(self) -> torch.Tensor:
        return self._static_out

    def _replay(self, new: Dict[str, Optional[torch.Tensor]], return_skip_ratio: bool):
        q = next(iter(new.values()))
        if q.device != self._device:
            raise ValueError("q must be on the same device as the captured graph.")
        for name in self._names:
            t = new.get(name)
            if t is None:
                raise ValueError(f"{name} is required for this captured graph.")
            dst = self._static[name]
            if t.data_ptr() != dst.data_ptr():
                dst.copy_(t)
        self._graph.replay()
        if not return_skip_ratio:
            return self._static_out
        kept = self._ws.mask.to(torch.int32).sum()
        return self._static_out, float((1.0 - kept.float() / float(self._ws.mask.numel())).item())

    def replay_only(self) -> torch.Tensor:
        """Replay without updating static inputs."""
        self._graph.replay()
        return self._static_out
