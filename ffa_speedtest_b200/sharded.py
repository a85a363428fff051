"""Multi-GPU decode: one process per GPU, work partitioned with no data-path collective
(batch x kv-head sharding) or split along the sequence with one small all-gather of
(partial output, LSE) pairs followed by the merge kernel.

The reference has no distributed code; this module is new.  The merge reuses the recurrence
of its stage-2 kernel (ffa-q2fp8/attn_kernel/attn_kernel_v1210_fused_bsz_q2fp8.py:142-171) in
LSE form."""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from . import _lib


def unit_slice(n_units: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous slice [lo, hi) of ``n_units`` (batch x kv-head) work units owned by ``rank``;
    the first ``n_units % world`` ranks get one extra unit."""
    base, extra = divmod(n_units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def page_slice(n_pages: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous slice of the pages of every sequence owned by ``rank`` (sequence split)."""
    return unit_slice(n_pages, rank, world)


def shard_batch_heads(rank: int, world: int, B: int, HKV: int) -> Tuple[slice, slice]:
    """Batch x kv-head sharding when ``world`` divides B*HKV along whole batches or whole heads:
    returns (batch slice, kv-head slice).  Batches are split first; if there are fewer batches
    than ranks, each batch's kv-heads are split over ``world // B`` ranks."""
    if B % world == 0:
        per = B // world
        return slice(rank * per, (rank + 1) * per), slice(0, HKV)
    if world % B == 0 and HKV % (world // B) == 0:
        per_b = world // B
        hp = HKV // per_b
        b, j = divmod(rank, per_b)
        return slice(b, b + 1), slice(j * hp, (j + 1) * hp)
    raise ValueError(f"cannot shard B={B}, HKV={HKV} over {world} ranks in whole batches or heads")


def merge_partials(parts: torch.Tensor, out_dtype: torch.dtype, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """parts ``[R, B, HQ, 129]`` fp32 (normalised output + base-2 LSE per row) -> ``[B, HQ, 128]``."""
    if parts.dim() != 4 or parts.shape[-1] != 129 or parts.dtype != torch.float32 or not parts.is_cuda:
        raise ValueError("parts must be a CUDA fp32 tensor of shape [R, B, HQ, 129]")
    parts = parts.contiguous()
    R, B, HQ, _ = parts.shape
    if out is None:
        out = torch.empty((B, HQ, 128), dtype=out_dtype, device=parts.device)
    _lib.check(_lib.lib().ffa_merge_partials(parts.data_ptr(), R, B * HQ, out.data_ptr(), _lib.float_code(out.dtype),
                                             _lib.current_stream(parts.device)), "ffa_merge_partials")
    return out


class SequenceShardedDecode:
    """Sequence-split decode step for one rank.

    Every rank holds pages ``page_slice(NP, rank, world)`` of every sequence and the same
    thresholds (passed in, or computed once by rank-local sampling of replicated codes by the
    caller).  ``step`` runs the local decode into a ``[B, HQ, 129]`` partial, all-gathers the
    partials over the process group (NCCL over NVLink for CUDA groups) and merges them."""

    def __init__(self, group, B: int, HQ: int, device, out_dtype: torch.dtype, merge_fn=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.world = dist.get_world_size(group)
        self.local = torch.empty((B, HQ, 129), dtype=torch.float32, device=device)
        self.gathered = torch.empty((self.world, B, HQ, 129), dtype=torch.float32, device=device)
        self.out = torch.empty((B, HQ, 128), dtype=out_dtype, device=device)
        # the CUDA merge kernel by default; CPU-rank tests of the protocol pass their own
        self._merge = merge_fn or (lambda parts, out: merge_partials(parts, out.dtype, out=out))

    def step(self, local_decode) -> torch.Tensor:
        """``local_decode(partial_out=...)`` must enqueue this rank's decode writing the partial
        ``[B, HQ, 129]`` (normalised output, base-2 LSE; LSE = -inf if the rank kept nothing)."""
        local_decode(partial_out=self.local)
        # rank r's partial lands in gathered[r]; the flat view is the form every backend accepts
        self.dist.all_gather_into_tensor(self.gathered.view(-1, *self.local.shape[1:]), self.local, group=self.group)
        return self._merge(self.gathered, self.out)
