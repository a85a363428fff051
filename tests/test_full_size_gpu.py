"""Benchmark-sized decode steps against the CPU oracle at their own shape.

BASELINE configs 1 (fp8fp8, B=8, T=32K), 2 (fp4 / nf4 / nvfp4, B=16, T=64K) and 4 (q2, T=128K; the
batch is cut to 4 sequences to bound memory and time - the kernel's work per sequence is the same):
the GPU runs the whole paged batch behind a seeded permutation of pages, the way bench.py does, and
the oracle then decodes one or two whole sequences of that batch on the CPU from the very tensors
the GPU read.  Kept set: identical outside the 1e-3 band around a threshold.  Output: within the
north-star tolerance (2e-2 max abs, 1e-2 mean relative) of the oracle run on the GPU's kept set.
"""
import pytest
import torch

from oracle import ffa_oracle as fo
from tests.helpers import band_ok
from ffa_speedtest_b200 import quantize as Q
from ffa_speedtest_b200.decode import allocate_decode_workspace, decode_call
from ffa_speedtest_b200.synth import make_block_table, make_decode_inputs

pytestmark = pytest.mark.gpu
HQ, HKV, D, PAGE = 32, 8, 128, 64
MAX_ABS, MEAN_REL = 2e-2, 1e-2


def quantise(kind, k, f8):
    if kind == "fp8":
        c, r = Q.quantize_k_fp8_fp8_residual(k, f8)
        return c, None, None, r
    if kind == "q2":
        return Q.quantize_k_2bit_fp8_residual(k, f8)
    if kind == "fp4":
        c, r = Q.encode_k_fp4_fp8_residual(k, f8)
        return c, None, None, r
    if kind == "nf4":
        c, s, r = Q.encode_k_nf4_fp8_residual(k, f8)
        return c, s, None, r
    c, s, r = Q.encode_k_nvfp4_fp8_residual(k, f8, PAGE)
    return c, s, None, r


@pytest.mark.parametrize("kind,B,T,check,SBS", [
    ("fp8", 8, 32768, (0, 5), 64),       # config 1
    ("fp4", 16, 65536, (3,), 64),        # config 2
    ("nf4", 16, 65536, (9,), 64),
    ("nvfp4", 16, 65536, (15,), 64),
    ("q2", 4, 131072, (2,), 64),         # config 4 at 128K, four of the 32 sequences
    ("q2", 4, 65536, (1,), 128),         # the reference's default block sizes (BS = SBS = 128): pages pruned in pairs
    ("fp8", 4, 65536, (3,), 32),         # prune blocks of half a page
])
def test_bench_workload_against_oracle(kind, B, T, check, SBS):
    dev = torch.device("cuda")
    f8 = torch.float8_e4m3fn
    delta = 8.0
    q, k, v = make_decode_inputs(B, T, HQ, HKV, D, seed=1, device=dev)
    codes, scale, zero, res = quantise(kind, k, f8)
    del k
    NP = T // PAGE
    BS = max(PAGE, SBS)
    NTBS = T // SBS
    bt = make_block_table(B, NP, seed=7).to(dev)

    def to_pool(x):
        xp = x.reshape(B * NP, PAGE, *x.shape[2:])
        pool = torch.empty_like(xp)
        view = torch.uint8 if x.dtype.itemsize == 1 else torch.int16
        pool.view(view)[bt.reshape(-1).long()] = xp.view(view)
        return pool

    codes_p, res_p, v_p = to_pool(codes), to_pool(res), to_pool(v)
    ws = allocate_decode_workspace(q, v_p, BS=BS, SBS=SBS, seq_len=T)
    o = decode_call(kind, q, codes_p, v_p, k_scale=scale, k_zero=zero, k_residual=res_p, BS=BS, SBS=SBS, delta=delta,
                    block_table=bt, seq_len=T, workspace=ws).clone()
    torch.cuda.synchronize()
    assert ws.status() == 0
    mask = ws.mask_view(B, HKV, NTBS).cpu()
    th = ws.threshold.cpu()
    del codes_p, res_p, v_p

    for b in check:
        sl = slice(b, b + 1)
        coarse = fo.CoarseK(kind, codes[sl].cpu(), None if scale is None else scale[sl].cpu(),
                            None if zero is None else zero[sl].cpu(), D)
        qb, vb, rb = q[sl].cpu(), v[sl].cpu(), res[sl].cpu()
        _, keep_ref, parts = fo.decode_attention_fast(qb, coarse, vb, rb, BS=BS, SBS=SBS, delta=delta,
                                                      out_dtype=torch.float32, return_parts=True)
        torch.testing.assert_close(th[sl], parts["threshold"], rtol=1e-5, atol=1e-4)
        assert band_ok(mask[sl], keep_ref, parts["block_max"], parts["threshold"], HQ // HKV)
        flips = int((mask[sl] != keep_ref).sum())
        assert flips <= 0.001 * keep_ref.numel(), f"{flips} pages decided differently"
        # the output, on the kept set the GPU used
        o_ref, _ = fo.decode_attention_fast(qb, coarse, vb, rb, BS=BS, SBS=SBS, delta=delta, out_dtype=torch.float32,
                                            keep_override=mask[sl])
        a = o[sl].float().cpu()
        assert torch.isfinite(a).all()
        max_abs = (a - o_ref).abs().max().item()
        mean_rel = ((a - o_ref).abs().mean() / o_ref.abs().mean().clamp_min(1e-6)).item()
        assert max_abs <= MAX_ABS, f"sequence {b}: max abs err {max_abs}"
        assert mean_rel <= MEAN_REL, f"sequence {b}: mean rel err {mean_rel}"
