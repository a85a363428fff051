"""Two-rank NCCL runs of the sharded decode paths (skipped with fewer than two GPUs): sequence
split with one all-gather of (O, LSE) partials + merge kernel, and batch x kv-head sharding."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    from oracle import ffa_oracle as fo
    from ffa_speedtest_b200 import sharded
    from ffa_speedtest_b200.decode import allocate_decode_workspace
    from ffa_speedtest_b200.fp8fp8.attn_kernel.attn_kernel_v1210_fused_bsz_fp8fp8 import attn_forward_decode_fp8fp8
    from ffa_speedtest_b200.synth import make_decode_inputs

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        B, T, HQ, HKV = 2, 64 * 40, 32, 8
        q, k, v = make_decode_inputs(B, T, HQ, HKV, 128, seed=8, n_heavy=6)       # replicated inputs
        coarse, res = fo.make_coarse("fp8", k, torch.float8_e4m3fn, 64)
        want = fo.decode_attention_fast(q, coarse, v, res, BS=64, delta=6.0, out_dtype=torch.float32)[0]
        qd = q.to(dev)

        # --- sequence split: rank r owns pages [lo, hi) of every sequence; thresholds are global ----
        full_ws = allocate_decode_workspace(qd, v.to(dev), BS=64)
        attn_forward_decode_fp8fp8(qd, coarse.codes.to(dev), v.to(dev), k_residual=res.to(dev), BS=64, delta=6.0,
                                   workspace=full_ws)
        th = full_ws.threshold.clone()      # in production: sampled once from the replicated sample tokens
        lo, hi = sharded.page_slice(T // 64, rank, world)
        ck, rk, vk = (x[:, lo * 64:hi * 64].contiguous().to(dev) for x in (coarse.codes, res, v))
        runner = sharded.SequenceShardedDecode(dist.group.WORLD, B, HQ, dev, torch.bfloat16)
        out = runner.step(lambda partial_out: attn_forward_decode_fp8fp8(
            qd, ck, vk, k_residual=rk, BS=64, precomputed_threshold=th, partial_out=partial_out))
        torch.cuda.synchronize()
        err_seq = float((out.float().cpu() - want).abs().max())

        # --- the same step with the exchange over peer memory, fused with the merge: three steps, so
        # that both halves of the double buffer and the step-numbered flags are exercised
        peer = sharded.PeerShardedDecode(dist.group.WORLD, B, HQ, dev, torch.bfloat16)
        same = True
        for _ in range(3):
            o_peer = peer.step(lambda partial_out: attn_forward_decode_fp8fp8(
                qd, ck, vk, k_residual=rk, BS=64, precomputed_threshold=th, partial_out=partial_out))
            torch.cuda.synchronize()
            close = float((o_peer.float() - out.float()).abs().max()) <= 2.0 ** -8      # one bf16 ulp at |o| <= 1
            same = same and close and int(peer.status[0]) == 0
        # ... and with the push fused into the decode kernel (warp-specialised kernel), three more steps
        from ffa_speedtest_b200.decode import decode_call
        ws_local = allocate_decode_workspace(qd, vk, BS=64)
        for _ in range(3):
            o_peer = peer.step(lambda partial_out, peer: decode_call(
                "fp8", qd, ck, vk, k_residual=rk, BS=64, SBS=64, precomputed_threshold=th, partial_out=partial_out,
                peer=peer, kernel="ws", workspace=ws_local), fused=True)
            torch.cuda.synchronize()
            close = float((o_peer.float() - out.float()).abs().max()) <= 2.0 ** -8
            same = same and close and int(peer.status[0]) == 0 and ws_local.status() == 0
        peer.close()

        # --- batch x kv-head sharding: disjoint outputs, no collective ------------------------------
        bs, hs = sharded.shard_batch_heads(rank, world, B, HKV)
        G = HQ // HKV
        o = attn_forward_decode_fp8fp8(
            q[bs][:, :, hs.start * G:hs.stop * G].contiguous().to(dev), coarse.codes[bs][:, :, hs].contiguous().to(dev),
            v[bs][:, :, hs].contiguous().to(dev), k_residual=res[bs][:, :, hs].contiguous().to(dev), BS=64, delta=6.0)
        err_unit = float((o.float().cpu() - want[bs][:, hs.start * G:hs.stop * G]).abs().max())
        ret[rank] = (err_seq, err_unit, same)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_sequence_split_and_unit_sharding():
    import torch.multiprocessing as mp
    port = free_port()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert len(ret) == 2
    for rank, (err_seq, err_unit, peer_same) in ret.items():
        assert err_seq <= 2e-2 and err_unit <= 2e-2, dict(ret)
        assert peer_same, "peer-memory exchange + merge differs from all-gather + merge"
