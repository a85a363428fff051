"""Multi-rank host logic on CPU ranks (gloo, world size 2 and 3): unit sharding without any
collective, and the sequence split with one all-gather of (O, LSE) partials.  The oracle stands in
for the CUDA kernels; what is under test is the partitioning, the partial layout and the merge
protocol of ffa_speedtest_b200/sharded.py."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ffa_oracle as fo
from ffa_speedtest_b200 import sharded
from ffa_speedtest_b200.synth import make_decode_inputs

LN2 = 0.6931471805599453


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_slices_partition_exactly():
    for n, w in ((256, 8), (64, 3), (5, 8), (7, 2)):
        spans = [sharded.unit_slice(n, r, w) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [hi - lo for lo, hi in spans]
        assert max(sizes) - min(sizes) <= 1
    assert sharded.shard_batch_heads(3, 8, 32, 8) == (slice(12, 16), slice(0, 8))
    assert sharded.shard_batch_heads(5, 8, 2, 8) == (slice(1, 2), slice(2, 4))
    with pytest.raises(ValueError):
        sharded.shard_batch_heads(0, 3, 2, 8)


def oracle_partial(q, coarse, v, res, th, lo, hi):
    """(normalised O, base-2 LSE) of tokens [lo, hi) with the global thresholds - what the CUDA
    decode writes into partial_out for a rank that owns those pages."""
    B, _, HQ, K = q.shape
    HKV = v.shape[2]
    sub = fo.CoarseK(coarse.kind, coarse.codes[:, lo:hi], coarse.scale, coarse.zero, K)
    o, keep = fo.decode_attention_fast(q, sub, v[:, lo:hi], res[:, lo:hi], BS=64, precomputed_threshold=th,
                                       out_dtype=torch.float32)
    q16 = q[:, 0].to(torch.float16).reshape(B, HKV, HQ // HKV, K)
    kk = sub.tile(torch.arange(hi - lo)) + res[:, lo:hi].to(torch.float16)
    s = fo._scores(q16, kk, K ** -0.5)
    s = torch.where(keep.repeat_interleave(64, dim=-1).bool().unsqueeze(2), s, torch.tensor(float("-inf")))
    lse = torch.logsumexp(s * LN2, dim=-1) / LN2
    return torch.cat([o, lse.reshape(B, HQ, 1)], dim=-1)


def _seq_split_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        B, T, HQ, HKV = 2, 64 * 11, 8, 2
        q, k, v = make_decode_inputs(B, T, HQ, HKV, 128, seed=3, n_heavy=3)      # same seed on every rank
        coarse, res = fo.make_coarse("fp8", k, torch.float8_e4m3fn, 64)
        # thresholds are global: every rank derives them from the (replicated) sample tokens
        th = fo.decode_threshold(q[:, 0].to(torch.float16).reshape(B, HKV, 4, 128), coarse, T, 64, 128 ** -0.5,
                                 5.0).reshape(B, HQ)
        lo, hi = sharded.page_slice(T // 64, rank, world)
        runner = sharded.SequenceShardedDecode(
            dist.group.WORLD, B, HQ, "cpu", torch.float32,
            merge_fn=lambda parts, out: out.copy_(fo.merge_partials(parts[..., :128], parts[..., 128])))

        def local_decode(partial_out):
            partial_out.copy_(oracle_partial(q, coarse, v, res, th, lo * 64, hi * 64))

        got = runner.step(local_decode)
        want = fo.decode_attention(q, coarse, v, res, BS=64, precomputed_threshold=th, out_dtype=torch.float32)
        ret[rank] = float((got - want).abs().max())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_split_all_gather_merge(world):
    port = free_port()
    ret = mp.Manager().dict()
    mp.spawn(_seq_split_worker, args=(world, port, ret), nprocs=world, join=True)
    assert len(ret) == world
    assert max(ret.values()) <= 2e-3, dict(ret)


def _unit_shard_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        B, T, HQ, HKV = 2, 256, 16, 4
        q, k, v = make_decode_inputs(B, T, HQ, HKV, 128, seed=4, n_heavy=2)
        coarse, res = fo.make_coarse("q2", k, torch.float8_e5m2, 64)
        bs, hs = sharded.shard_batch_heads(rank, world, B, HKV)
        G = HQ // HKV
        qs = q[bs][:, :, hs.start * G:hs.stop * G]
        sub = fo.CoarseK("q2", coarse.codes[bs][:, :, hs], coarse.scale[bs][:, hs], coarse.zero[bs][:, hs], 128)
        mine = fo.decode_attention(qs, sub, v[bs][:, :, hs], res[bs][:, :, hs], BS=64, delta=5.0,
                                   out_dtype=torch.float32)
        # no collective on the data path; gather only to check the result
        full = fo.decode_attention(q, coarse, v, res, BS=64, delta=5.0, out_dtype=torch.float32)
        ret[rank] = float((mine - full[bs][:, hs.start * G:hs.stop * G]).abs().max())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_batch_head_sharding_needs_no_collective(world):
    port = free_port()
    ret = mp.Manager().dict()
    mp.spawn(_unit_shard_worker, args=(world, port, ret), nprocs=world, join=True)
    # identical work on a slice of the tensors: only the CPU matmul blocking may differ
    assert len(ret) == world and max(ret.values()) <= 1e-5, dict(ret)


def _failing_rank_worker(rank, world, port, ret):
    """A rank that dies before the all-gather: the survivor's collective ends with an error
    within the process-group timeout instead of hanging."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        if rank == 1:
            ret[rank] = "left"
            return                       # leaves between steps, nothing in flight
        runner = sharded.SequenceShardedDecode(dist.group.WORLD, 1, 4, "cpu", torch.float32,
                                               merge_fn=lambda parts, out: out)
        try:
            runner.step(lambda partial_out: partial_out.zero_())
            ret[rank] = "no error"
        except Exception as e:           # noqa: BLE001 - any backend error is the expected outcome
            ret[rank] = "error: " + type(e).__name__
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_missing_rank_surfaces_as_error_not_hang():
    port = free_port()
    ret = mp.Manager().dict()
    mp.spawn(_failing_rank_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret[1] == "left" and str(ret[0]).startswith("error"), dict(ret)


def test_sample_token_rows_match_the_oracle_sampling():
    """The rows a rank replicates for the global threshold are the ones the oracle samples."""
    from ffa_speedtest_b200.sharded import sample_token_rows
    for T, BS in ((4096, 64), (2373, 128), (524288, 64), (64, 64)):
        ntb = -(-T // BS)
        r0, r1 = sample_token_rows(T, BS)
        assert list(r0) == list(range(16))
        assert list(r1) == [(ntb - 1) * fo.THRESHOLD_SAMPLE + i for i in range(fo.THRESHOLD_SAMPLE)]
    with pytest.raises(ValueError):
        sample_token_rows(10, 64)


class _FakePeerLib:
    """Stands in for the CUDA library in the peer-memory set-up: host-side buffers, and an allocation
    that fails on one chosen rank."""

    def __init__(self, fail_alloc: bool, fail_open: bool):
        self.fail_alloc, self.fail_open = fail_alloc, fail_open
        self.opened, self.closed, self.freed = 0, 0, 0

    def ffa_peer_alloc(self, nbytes, ptr_ref, handle):
        if self.fail_alloc:
            return -5
        ptr_ref._obj.value = 0x1000
        return 0

    def ffa_peer_open(self, handle, ptr_ref):
        if self.fail_open:
            return -5
        self.opened += 1
        ptr_ref._obj.value = 0x2000 + self.opened
        return 0

    def ffa_peer_close(self, ptr):
        self.closed += 1
        return 0

    def ffa_peer_free(self, ptr):
        self.freed += 1
        return 0

    def ffa_last_cuda_error(self):
        return b"out of memory (injected)"


def _peer_setup_worker(rank, world, port, mode, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ffa_speedtest_b200 import _lib
        fake = _FakePeerLib(fail_alloc=(mode == "alloc" and rank == 1), fail_open=(mode == "open" and rank == 0))
        _lib.lib = lambda: fake
        try:
            sharded.PeerShardedDecode(dist.group.WORLD, 1, 8, "cpu", torch.float32)
            ret[rank] = ("built", fake.opened, fake.closed, fake.freed)
        except RuntimeError as exc:
            ret[rank] = ("raised", str(exc), fake.closed, fake.freed)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["alloc", "open"])
def test_peer_setup_failure_on_one_rank_raises_on_every_rank(mode):
    """The set-up of the peer-memory transport is collective: when one rank cannot allocate its buffer,
    or cannot map a peer's, every rank must leave with the same exception (and give back what it had
    taken) instead of waiting for the failed rank in a later collective.  The failure is injected on
    the host, through a stand-in for the library."""
    world, port = 3, free_port()
    ret = mp.Manager().dict()
    mp.spawn(_peer_setup_worker, args=(world, port, mode, ret), nprocs=world, join=True)
    assert len(ret) == world
    failed = 1 if mode == "alloc" else 0
    for rank in range(world):
        kind, msg = ret[rank][0], ret[rank][1]
        assert kind == "raised" and f"[{failed}]" in msg, dict(ret)
    if mode == "open":
        # ranks that had mapped their peers unmapped them again, and everyone freed its own buffer
        assert ret[1][2] == world - 1 and all(ret[r][3] == 1 for r in range(world))
