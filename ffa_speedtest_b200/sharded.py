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


def sample_token_rows(T: int, BS: int) -> Tuple[range, range]:
    """The two 16-token blocks the prune thresholds are computed from: tokens ``[0, 16)`` and
    ``[(NTB-1)*16, +16)`` with ``NTB = ceil(T / BS)`` (reference ...q2fp8.py:55-82)."""
    ntb = -(-T // BS)
    if ntb * 16 > T:
        raise ValueError(f"T={T} is shorter than the sample blocks of {ntb} x 16 tokens")
    return range(0, 16), range((ntb - 1) * 16, (ntb - 1) * 16 + 16)


def global_threshold(variant: str, q: torch.Tensor, k_codes: torch.Tensor, *, delta: float,
                     k_scale: Optional[torch.Tensor] = None, k_zero: Optional[torch.Tensor] = None,
                     scale: Optional[float] = None) -> torch.Tensor:
    """Prune thresholds ``[B, HQ]`` of a sequence from its two sample blocks alone.

    The thresholds depend on the coarse codes of the token rows ``sample_token_rows(T, BS)`` only, so
    a rank that owns other pages can compute them from a replicated copy of those 32 rows: ``k_codes``
    is ``[B, 32, HKV, code_bytes]`` (first block, then second block).  The two blocks are placed in a
    short stand-in sequence at the positions the kernel samples and one decode call over it writes the
    thresholds.  For nvfp4 ``k_scale`` is the sequence's ``[B, NTB, HKV]`` page scales (or just its
    first and last block, ``[B, 2, HKV]``): the kernel scales the first sample by block 0 and the
    second by block NTB-1 (reference ...nvfp4fp8.py:80,99), and the stand-in carries those two."""
    from .decode import DecodeWorkspace, decode_call
    if k_codes.dim() != 4 or k_codes.shape[1] != 32:
        raise ValueError("k_codes must be [B, 32, HKV, code_bytes]: the two 16-token sample blocks")
    B, _, HKV, W = k_codes.shape
    HQ = q.shape[2]
    # five pages: the second sample sits at (5-1)*16 = 64; six when a 5 x 5 nvfp4 scale would be
    # ambiguous between [NTB, HKV] and its transpose
    n_pages = 6 if (variant == "nvfp4" and HKV == 5) else 5
    T_s = n_pages * 64
    second = (n_pages - 1) * 16
    mini = torch.zeros((B, T_s, HKV, W), dtype=k_codes.dtype, device=k_codes.device)
    mini.view(torch.uint8)[:, 0:16] = k_codes.view(torch.uint8)[:, 0:16]
    mini.view(torch.uint8)[:, second:second + 16] = k_codes.view(torch.uint8)[:, 16:32]
    if variant == "nvfp4":
        if k_scale is None or k_scale.dim() != 3 or k_scale.shape[0] != B or k_scale.shape[2] != HKV or k_scale.shape[1] < 1:
            raise ValueError("nvfp4 needs k_scale [B, NTB, HKV] (or its first and last block)")
        mini_scale = torch.ones((B, n_pages, HKV), dtype=k_scale.dtype, device=k_scale.device)
        mini_scale[:, 0] = k_scale[:, 0]
        mini_scale[:, n_pages - 1] = k_scale[:, -1]
        k_scale = mini_scale
    v = torch.zeros((B, T_s, HKV, 128), dtype=q.dtype if q.dtype != torch.float32 else torch.float16, device=q.device)
    ws = DecodeWorkspace.for_shape(B, T_s, HQ, HKV, 128, BS=64, SBS=64, device=q.device, dtype=q.dtype)
    decode_call(variant, q, mini, v, k_scale=k_scale, k_zero=k_zero, k_residual=None, scale=scale, BS=64, SBS=64,
                delta=delta, use_fp8_residual=False, workspace=ws)
    return ws.threshold.clone()


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
        self.rank = dist.get_rank(group)
        self.gathered = torch.empty((self.world, B, HQ, 129), dtype=torch.float32, device=device)
        # this rank's partial is written straight into its slot of the gathered buffer, so the
        # all-gather runs in place (no staging copy of the send buffer)
        self.local = self.gathered[self.rank]
        self.out = torch.empty((B, HQ, 128), dtype=out_dtype, device=device)
        # the CUDA merge kernel by default; CPU-rank tests of the protocol pass their own
        self._merge = merge_fn or (lambda parts, out: merge_partials(parts, out.dtype, out=out))

    def gather(self) -> None:
        """All-gather the partials: rank r's lands in ``gathered[r]`` on every rank."""
        self.dist.all_gather_into_tensor(self.gathered.view(-1, *self.local.shape[1:]), self.local, group=self.group)

    def merge(self) -> torch.Tensor:
        return self._merge(self.gathered, self.out)

    def step(self, local_decode) -> torch.Tensor:
        """``local_decode(partial_out=...)`` must enqueue this rank's decode writing the partial
        ``[B, HQ, 129]`` (normalised output, base-2 LSE; LSE = -inf if the rank kept nothing)."""
        local_decode(partial_out=self.local)
        self.gather()
        return self.merge()


class _DeviceArray:
    """A device buffer owned by the library, seen by torch through the CUDA array interface."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2}


class PeerShardedDecode:
    """Sequence-split decode step whose exchange runs over peer memory, fused with the merge.

    Same contract as ``SequenceShardedDecode`` (every rank holds a page range of every sequence and the
    same thresholds; ``step`` returns the merged ``[B, HQ, 128]`` output on every rank), but instead of an
    NCCL all-gather followed by the merge kernel, each rank stores its ``[B, HQ, 129]`` partial straight
    into its slot of every peer's buffer (plain peer stores over NVLink, buffers mapped through CUDA
    IPC) and raises a flag there; the merge kernel waits, for at most a second, for all flags of the step
    and merges from local memory (``ffa_peer_exchange_merge``).  One box only: every rank must be able
    to map every other rank's memory.  ``close()`` unmaps and frees; call it on every rank."""

    def __init__(self, group, B: int, HQ: int, device, out_dtype: torch.dtype):
        import ctypes as C
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 16:
            raise ValueError("at most 16 ranks")
        self.rows = B * HQ
        self.device = torch.device(device)
        L = _lib.lib()
        n_part = self.rows * 129
        self._gather_bytes = 2 * self.world * n_part * 4
        total = self._gather_bytes + 256                       # + the flags, one int per rank
        # Set-up is collective and every rank takes every collective step whatever happens on it, so that
        # a rank that cannot allocate or map ends in the same exception on all ranks, not in a hang.
        import contextlib
        on_device = torch.cuda.device(self.device) if self.device.type == "cuda" else contextlib.nullcontext()
        with on_device:
            ptr, handle = C.c_void_p(), C.create_string_buffer(64)
            rc = L.ffa_peer_alloc(total, C.byref(ptr), handle)
            self._own = ptr.value if rc == 0 else None
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.raw) if rc == 0 else None, group=group)
            self._bases, failed = [], rc != 0                     # `failed`: this rank's own steps
            if not failed and all(h is not None for h in handles):
                for r, h in enumerate(handles):
                    if r == self.rank:
                        self._bases.append(self._own)
                        continue
                    p = C.c_void_p()
                    if L.ffa_peer_open(h, C.byref(p)) != 0:
                        failed = True
                        break
                    self._bases.append(p.value)
            oks = [None] * self.world
            dist.all_gather_object(oks, not failed, group=group)
            if not all(oks):
                for r, b in enumerate(self._bases):
                    if r != self.rank:
                        L.ffa_peer_close(b)
                dist.barrier(group=group)
                if self._own is not None:
                    L.ffa_peer_free(self._own)
                self._own = None
                raise RuntimeError("peer-memory set-up failed on rank(s) "
                                   f"{[r for r, ok in enumerate(oks) if not ok]}: {L.ffa_last_cuda_error().decode()!r}")
        self._gathered_ptrs = (C.c_void_p * self.world)(*self._bases)
        self._flag_ptrs = (C.c_void_p * self.world)(*[b + self._gather_bytes for b in self._bases])
        # this rank's two slots, as tensors the decode kernel writes its partial into
        holder = _DeviceArray(self._own, (2, self.world, B, HQ, 129), "<f4")
        self.gathered = torch.as_tensor(holder, device=self.device)
        self._holder = holder
        self.out = torch.empty((B, HQ, 128), dtype=out_dtype, device=self.device)
        self.status = torch.zeros(8, dtype=torch.int32, device=self.device)
        self.step_no = 0
        dist.barrier(group=group)

    def local_slot(self) -> torch.Tensor:
        """Where the NEXT step's local partial goes: ``[B, HQ, 129]``."""
        return self.gathered[(self.step_no + 1) & 1, self.rank]

    def step(self, local_decode, fused: bool = False) -> torch.Tensor:
        """``fused=False``: ``local_decode(partial_out=...)`` as for ``SequenceShardedDecode``, then one call
        pushes the partial to the peers, waits and merges.  ``fused=True``: ``local_decode(partial_out=...,
        peer=...)`` must hand ``peer`` to the decode entry point (warp-specialised kernel); the kernel then
        stores every partial row on the peers as it is produced and only the wait-and-merge remains."""
        if not fused:
            local_decode(partial_out=self.local_slot())
            return self.exchange_and_merge()
        slot = self.local_slot()
        self.step_no += 1
        args = _lib.FfaPeerArgs(world=self.world, rank=self.rank, step=self.step_no,
                                peer_gathered=self._gathered_ptrs, peer_flags=self._flag_ptrs)
        local_decode(partial_out=slot, peer=args)
        _lib.check(_lib.lib().ffa_peer_wait_merge(
            self._own, self._own + self._gather_bytes, self.world, self.rows, self.step_no, self.out.data_ptr(),
            _lib.float_code(self.out.dtype), self.status.data_ptr(), _lib.current_stream(self.device)),
            "ffa_peer_wait_merge")
        return self.out

    def exchange_and_merge(self) -> torch.Tensor:
        """The part of a step after the local decode: push the partial in ``local_slot()`` to every peer,
        wait for theirs, merge.  Every rank must call it the same number of times."""
        slot = self.local_slot()
        self.step_no += 1
        _lib.check(_lib.lib().ffa_peer_exchange_merge(
            slot.data_ptr(), self.rows, self.rank, self.world, self._gathered_ptrs, self._flag_ptrs, self.step_no,
            self.out.data_ptr(), _lib.float_code(self.out.dtype), self.status.data_ptr(),
            _lib.current_stream(self.device)), "ffa_peer_exchange_merge")
        return self.out

    def close(self) -> None:
        if getattr(self, "_own", None) is None:
            return
        torch.cuda.synchronize(self.device)
        self.dist.barrier(group=self.group)                  # nobody is still storing into a peer
        L = _lib.lib()
        with torch.cuda.device(self.device):
            for r, b in enumerate(self._bases):
                if r != self.rank:
                    L.ffa_peer_close(b)
            self.dist.barrier(group=self.group)              # every mapping is gone before the owners free
            del self.gathered
            L.ffa_peer_free(self._own)
        self._own = None
