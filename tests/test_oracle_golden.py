"""The CPU oracle against the committed outputs of the reference's own code (tests/golden)."""
import hashlib

import numpy as np
import pytest
import torch

from oracle import ffa_oracle as fo
from tests.helpers import FP8, GOLDEN, KINDS, SMALL_CASES, GoldenCase, band_ok, digest, from_raw
from ffa_speedtest_b200.synth import make_decode_inputs, make_kproj_inputs


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("name", SMALL_CASES)
def test_quantiser_bit_exact(kind, name):
    """Oracle quantiser == reference quantiser, bit for bit (digests of codes, scales, residual)."""
    c = GoldenCase(kind, name)
    assert digest(c.q, c.k, c.v) == c.sha["inputs"], "seeded inputs drifted from the ones the goldens were made on"
    coarse, res = c.quantise()
    assert digest(coarse.codes) == c.sha["codes"]
    assert digest(res) == c.sha["res"]
    if "scale" in c.sha:
        assert digest(coarse.scale) == c.sha["scale"]
    if "zero" in c.sha:
        assert digest(coarse.zero) == c.sha["zero"]


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("name", SMALL_CASES)
def test_decode_matches_reference_kernels(kind, name):
    """Oracle decode == reference Triton stage 1 + 2 (interpreter): same kept set, fp32 output
    equal up to accumulation order."""
    c = GoldenCase(kind, name)
    coarse, res = c.quantise()
    o, parts = fo.decode_attention(c.q, coarse, c.v, res, BS=c.BS, SBS=c.SBS, delta=c.delta,
                                   precomputed_threshold=c.th, use_fp8_residual=c.use_res, return_parts=True,
                                   out_dtype=torch.float32)
    assert band_ok(parts["mask"], c.mask_ref, parts["block_max"], parts["threshold"], c.HQ // c.HKV, tol=1e-5)
    assert torch.equal(parts["mask"], c.mask_ref)
    torch.testing.assert_close(o, c.o_ref, rtol=1e-4, atol=2e-5)


@pytest.mark.parametrize("fp8", ["e5m2", "e4m3"])
def test_config0_q2fp8(fp8):
    """benchmark config 0 (B=1, 32/8 heads, T=4096, page 64, delta 8): oracle vs reference."""
    z = np.load(GOLDEN / f"decode_q2_config0_{fp8}.npz")
    q, k, v = make_decode_inputs(1, 4096, 32, 8, 128, seed=0, dtype=torch.bfloat16)
    coarse, res = fo.make_coarse("q2", k, FP8[fp8], 64)
    assert digest(q, k, v, coarse.codes, coarse.scale, coarse.zero, res) == str(z["sha256"])
    o, keep = fo.decode_attention_fast(q, coarse, v, res, BS=64, SBS=64, delta=8.0, out_dtype=torch.float32)
    assert torch.equal(keep, torch.from_numpy(z["mask"]))
    torch.testing.assert_close(o, torch.from_numpy(z["o"]), rtol=1e-4, atol=2e-5)


def test_fast_and_serial_oracles_agree():
    q, k, v = make_decode_inputs(2, 512, 8, 2, 128, seed=11, n_heavy=2)
    for kind in KINDS:
        coarse, res = fo.make_coarse(kind, k, torch.float8_e4m3fn, 64)
        a, parts = fo.decode_attention(q, coarse, v, res, BS=64, delta=4.5, out_dtype=torch.float32,
                                       return_parts=True)
        b, keep = fo.decode_attention_fast(q, coarse, v, res, BS=64, delta=4.5, out_dtype=torch.float32)
        assert torch.equal(parts["mask"], keep)
        assert 0 < int(keep.sum()) < keep.numel()
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)


def test_merge_partials_equals_single_pass():
    """Splitting the sequence and merging (O, LSE) pairs reproduces the unsplit result."""
    q, k, v = make_decode_inputs(1, 512, 8, 2, 128, seed=12, n_heavy=2)
    coarse, res = fo.make_coarse("fp8", k, torch.float8_e4m3fn, 64)
    th = fo.decode_threshold(q[:, 0].to(torch.float16).reshape(1, 2, 4, 128), coarse, 512, 64, 128 ** -0.5, 5.0)
    th = th.reshape(1, 8)
    full = fo.decode_attention(q, coarse, v, res, BS=64, precomputed_threshold=th, out_dtype=torch.float32)
    outs, lses = [], []
    for lo, hi in ((0, 192), (192, 512)):
        sub = fo.CoarseK("fp8", coarse.codes[:, lo:hi])
        o, keep = fo.decode_attention_fast(q, sub, v[:, lo:hi], res[:, lo:hi], BS=64, precomputed_threshold=th,
                                           out_dtype=torch.float32)
        # recover the LSE of the part from a second pass with V = 1
        ones = torch.ones_like(v[:, lo:hi])
        q16 = q[:, 0].to(torch.float16).reshape(1, 2, 4, 128)
        kk = (sub.tile(torch.arange(hi - lo)) + res[:, lo:hi].to(torch.float16))
        s = fo._scores(q16, kk, 128 ** -0.5)                                  # [1,2,4,n]
        keep_tok = keep.repeat_interleave(64, dim=-1).bool().unsqueeze(2)     # [1,2,1,n]
        s = torch.where(keep_tok, s, torch.tensor(float("-inf")))
        lse = torch.logsumexp(s * 0.6931471805599453, dim=-1) * 1.4426950408889634
        outs.append(o)
        lses.append(lse.reshape(1, 8))
    merged = fo.merge_partials(torch.stack(outs), torch.stack(lses))
    torch.testing.assert_close(merged, full, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("T", [1, 70])
def test_kproj_reference_goldens(kind, T):
    """Oracle K-proj + RoPE + quantiser == the reference's torch kproj_rope_*_reference on CPU."""
    z = np.load(GOLDEN / f"kproj_{kind}_T{T}.npz")
    B, T_, H, HKV, D, seed, start = (int(x) for x in z["meta"])
    h, w = make_kproj_inputs(T_, H, HKV, D, B=B, seed=seed, dtype=torch.bfloat16)
    w = w * 4.0
    cos, sin = fo.rope_tables(T_ + start, D, base=500000.0)
    cos, sin = cos[start:].contiguous(), sin[start:].contiguous()
    assert digest(h, w, cos, sin) == str(z["sha_inputs"])
    k = fo.kproj_rope(h, w, cos, sin, HKV, D)
    if kind == "nvfp4":
        outs = fo.quantize_nvfp4(k, torch.float8_e4m3fn, 64)
    else:
        outs = fo.QUANTIZERS[kind](k, torch.float8_e4m3fn)
    for i, t in enumerate(outs):
        ref = z[f"out{i}"]
        got = t.view(torch.uint8).numpy() if t.dtype == torch.float8_e4m3fn else (
            t.view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.numpy())
        assert np.array_equal(got, ref), f"output {i} differs"


@pytest.mark.parametrize("name", ["meanv_ragged", "meanv_fp16", "meanv_sbs128"])
def test_mean_v_variant_matches_the_reference(name):
    """Pruned blocks folded in as coarse mass x mean(V): oracle against the reference's mean-V kernels."""
    z = np.load(GOLDEN / f"decode_q2_{name}.npz")
    B, T, HQ, HKV, D, BS, SBS, seed, n_heavy = (int(x) for x in z["meta"])
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16}[str(z["dtype"])]
    q, k, v = make_decode_inputs(B, T, HQ, HKV, D, seed=seed, dtype=dt, n_heavy=n_heavy)
    assert digest(q, k, v) == str(z["sha_inputs"])
    coarse, res = fo.make_coarse("q2", k, FP8[str(z["fp8"])], BS)
    mean_v = v.mean(dim=1, dtype=torch.float32).to(v.dtype)
    o, parts = fo.decode_attention(q, coarse, v, res, BS=BS, SBS=SBS, delta=float(z["delta"]), mean_v=mean_v,
                                   out_dtype=torch.float32, return_parts=True)
    approx = torch.from_numpy(z["approx"])
    # a block is approximated exactly when it holds tokens and was pruned
    n_sub = -(-T // SBS)
    has_tokens = (torch.arange(approx.shape[-1]) < n_sub).view(1, 1, -1)
    assert torch.equal((parts["mask"] == 0) & has_tokens, approx.bool())
    torch.testing.assert_close(o, torch.from_numpy(z["o"]), rtol=0, atol=1e-4)
