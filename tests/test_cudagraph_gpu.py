"""The CUDA-graph runners, driven the way the reference's benches drive theirs
(ffa-q2fp8/attn_kernel/attn_kernel_v1210_fused_bsz_q2fp8_cudagraph.py:19-36, 122-183 and the four
siblings): constructor with the reference's arguments, ``replay`` with new tensors,
``replay_only``, ``output`` - each compared bit for bit with the eager entry point."""
import importlib

import pytest
import torch

from oracle import ffa_oracle as fo
from tests.helpers import KINDS
from ffa_speedtest_b200.synth import make_decode_inputs

pytestmark = pytest.mark.gpu

RUNNERS = {
    "q2": ("q2fp8", "CUDAGraphDecodeRunnerQ2FP8", "attn_forward_decode_quantized"),
    "fp8": ("fp8fp8", "CUDAGraphDecodeRunnerFP8FP8", "attn_forward_decode_fp8fp8"),
    "fp4": ("fp4fp8", "CUDAGraphDecodeRunnerFP4FP8", "attn_forward_decode_fp4"),
    "nf4": ("nf4fp8", "CUDAGraphDecodeRunnerNF4FP8", "attn_forward_decode_nf4"),
    "nvfp4": ("nvfp4fp8", "CUDAGraphDecodeRunnerNVFP4FP8", "attn_forward_decode_nvfp4fp8"),
}


def tensors_of(kind, coarse, dev):
    """Positional K tensors of the variant's call, after q and before v."""
    codes = coarse.codes.to(dev)
    if kind == "q2":
        return [codes, coarse.scale.to(dev), coarse.zero.to(dev)]
    if kind in ("nf4", "nvfp4"):
        return [codes, coarse.scale.to(dev)]
    return [codes]


@pytest.mark.parametrize("kind", KINDS)
def test_runner_matches_eager_entry_point(kind):
    variant, cls_name, fn_name = RUNNERS[kind]
    base = f"ffa_speedtest_b200.{variant}.attn_kernel.attn_kernel_v1210_fused_bsz_{variant}"
    Runner = getattr(importlib.import_module(base + "_cudagraph"), cls_name)
    entry = getattr(importlib.import_module(base), fn_name)
    dev = "cuda"
    B, T, HQ, HKV, BS, SBS, delta = 2, 64 * 20, 8, 2, 128, 64, 4.0
    q, k, v = make_decode_inputs(B, T, HQ, HKV, 128, seed=70, n_heavy=4)
    q2 = make_decode_inputs(B, T, HQ, HKV, 128, seed=71, n_heavy=4)[0]
    coarse, res = fo.make_coarse(kind, k, torch.float8_e5m2, BS)
    kt = tensors_of(kind, coarse, dev)
    qd, q2d, vd, rd = q.to(dev), q2.to(dev), v.to(dev), res.to(dev)

    def eager(qq):
        return entry(qq, *kt, vd, k_residual=rd, BS=BS, SBS=SBS, delta=delta).clone()

    runner = Runner(qd, *kt, vd, k_residual=rd, precomputed_threshold=None, k_bits=2 if kind == "q2" else 4,
                    scale=None, BS=BS, SBS=SBS, delta=delta, use_fp8_residual=True, warmup=2) if kind != "fp8" else \
        Runner(qd, *kt, vd, k_residual=rd, precomputed_threshold=None, scale=None, BS=BS, SBS=SBS, delta=delta,
               use_fp8_residual=True, warmup=2)
    want = eager(qd)
    assert runner.output.shape == (B, HQ, 128) and runner.output.dtype == qd.dtype
    assert torch.equal(runner.output, want)                       # the capture itself ran the step
    assert torch.equal(runner.replay_only(), want)

    # new query: replay copies it into the static buffers; __call__ is replay
    want2 = eager(q2d)
    out = runner.replay(q2d, *kt, vd, k_residual=rd)
    assert out.data_ptr() == runner.output.data_ptr() and torch.equal(out, want2)
    out, skip = runner(qd, *kt, vd, k_residual=rd, return_skip_ratio=True)
    o_e, skip_e = entry(qd, *kt, vd, k_residual=rd, BS=BS, SBS=SBS, delta=delta, return_skip_ratio=True)
    assert torch.equal(out, want) and torch.equal(o_e, want) and skip == skip_e
    assert torch.equal(runner.replay_only(), want)

    with pytest.raises(ValueError, match="k_residual is required"):
        runner.replay(qd, *kt, vd)


def test_runner_with_precomputed_threshold_and_without_residual():
    from ffa_speedtest_b200.fp8fp8.attn_kernel.attn_kernel_v1210_fused_bsz_fp8fp8 import attn_forward_decode_fp8fp8
    from ffa_speedtest_b200.fp8fp8.attn_kernel.attn_kernel_v1210_fused_bsz_fp8fp8_cudagraph import CUDAGraphDecodeRunnerFP8FP8
    dev = "cuda"
    q, k, v = make_decode_inputs(1, 64 * 9 + 3, 8, 2, 128, seed=72, n_heavy=2, dtype=torch.float16)
    coarse, res = fo.make_coarse("fp8", k, torch.float8_e4m3fn, 64)
    th = torch.full((1, 8), -3.0, device=dev)
    qd, cd, vd = q.to(dev), coarse.codes.to(dev), v.to(dev)
    runner = CUDAGraphDecodeRunnerFP8FP8(qd, cd, vd, precomputed_threshold=th, BS=64, use_fp8_residual=False, warmup=1)
    want = attn_forward_decode_fp8fp8(qd, cd, vd, precomputed_threshold=th, BS=64, use_fp8_residual=False)
    assert torch.equal(runner.replay_only(), want)
    th2 = torch.full((1, 8), 2.0, device=dev)
    want2 = attn_forward_decode_fp8fp8(qd, cd, vd, precomputed_threshold=th2, BS=64, use_fp8_residual=False).clone()
    assert torch.equal(runner.replay(qd, cd, vd, precomputed_threshold=th2), want2)
    with pytest.raises(ValueError, match="precomputed_threshold is required"):
        runner.replay(qd, cd, vd)
