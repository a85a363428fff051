"""Fused K-projection + RoPE (tcgen05 GEMM) and the quantise/scatter pass behind it."""
import numpy as np
import pytest
import torch

from oracle import ffa_oracle as fo
from tests.helpers import GOLDEN, KINDS
from ffa_speedtest_b200 import kproj as KP
from ffa_speedtest_b200.synth import make_block_table, make_kproj_inputs

pytestmark = pytest.mark.gpu
E4 = torch.float8_e4m3fn


def status():
    """Device status word of the last call: 0 unless a bounded wait inside the GEMM gave up."""
    return int(KP.kproj_fused.last_workspace[-256:-252].view(torch.int32).item())


def rope_tables(T, start, dtype=torch.float32):
    cos, sin = fo.rope_tables(T + start, 128, base=500000.0)
    return cos[start:].contiguous().to(dtype), sin[start:].contiguous().to(dtype)


@pytest.mark.parametrize("T,H,HKV,B", [(1, 512, 2, 2), (70, 512, 2, 2), (300, 4096, 8, 1), (129, 1024, 1, 3)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rope32", [True, False])
def test_post_rope_k_matches_torch(T, H, HKV, B, dtype, rope32):
    """K = rope(h W^T + b): same op order and roundings as the reference recipe; only the GEMM's
    accumulation order differs, which can flip the last bit of the 16-bit K_lin."""
    h, w = make_kproj_inputs(T, H, HKV, 128, B=B, seed=40 + T, dtype=dtype)
    w = w * 4.0
    bias = (0.1 * torch.randn(HKV * 128, generator=torch.Generator().manual_seed(1))).to(dtype)
    cos, sin = rope_tables(T, 7, torch.float32 if rope32 else dtype)
    want = fo.kproj_rope(h, w, cos, sin, HKV, 128, bias=bias)
    (got,) = KP.kproj_fused(None, h.cuda(), w.cuda(), cos.cuda(), sin.cuda(), HKV, 128, bias=bias.cuda())
    assert status() == 0
    assert got.dtype == want.dtype and got.shape == want.shape
    err = (got.float().cpu() - want.float()).abs()
    ulp = 2.0 ** (-7 if dtype == torch.bfloat16 else -10)
    scale = want.float().abs().max().item()
    assert err.max().item() <= 2.5 * ulp * scale, err.max().item()
    assert err.mean().item() <= 0.05 * ulp * scale, err.mean().item()


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("T", [1, 70])
def test_against_reference_goldens_with_its_smoke_tolerances(kind, T):
    """Reference kproj_rope_*_reference outputs (CPU, bf16) vs the fused path, judged with the
    reference's own smoke-test tolerances (ffa-q2fp8/fused_kproj_rope_q2fp8.py:606-615):
    packed-byte mismatch <= 1 %, scale / zero max error <= 0.05, residual mean error <= 0.05."""
    z = np.load(GOLDEN / f"kproj_{kind}_T{T}.npz")
    B, T_, H, HKV, D, seed, start = (int(x) for x in z["meta"])
    h, w = make_kproj_inputs(T_, H, HKV, D, B=B, seed=seed, dtype=torch.bfloat16)
    w = w * 4.0
    cos, sin = rope_tables(T_, start)
    outs = KP.kproj_fused(kind, h.cuda(), w.cuda(), cos.cuda(), sin.cuda(), HKV, D, fp8_dtype=E4, page_size=64)
    assert status() == 0
    refs = [z[f"out{i}"] for i in range(len(outs))]
    for i, (got, ref) in enumerate(zip(outs, refs)):
        got = got.cpu()
        last = i == len(outs) - 1
        if last:                                    # fp8 residual
            r = torch.from_numpy(ref).view(E4).float()
            assert (got.float() - r).abs().mean().item() <= 0.05
        elif i == 0:                                # packed codes (fp8 base for fp8fp8)
            g = got.view(torch.uint8).numpy()
            assert (g != ref).mean() <= 0.01, f"{(g != ref).mean():.4f} of packed bytes differ"
        else:                                       # scales / zeros (fp32: the tables are fp32)
            assert got.dtype == torch.float32
            r = torch.from_numpy(ref.view(np.float32) if ref.dtype != np.float32 else ref)
            assert (got - r).abs().max().item() <= 0.05


@pytest.mark.parametrize("kind", KINDS)
def test_fused_equals_reference_recipe_given_same_k(kind):
    """Quantising the K returned by the fused kernel with the standalone quantiser reproduces the
    fused outputs bit for bit (the epilogue adds nothing of its own)."""
    from ffa_speedtest_b200 import quantize as Q
    T, H, HKV, B = 200, 1024, 2, 2
    h, w = make_kproj_inputs(T, H, HKV, 128, B=B, seed=77, dtype=torch.bfloat16)
    cos, sin = rope_tables(T, 3)
    *outs, k = KP.kproj_fused(kind, h.cuda(), (w * 4).cuda(), cos.cuda(), sin.cuda(), HKV, 128, fp8_dtype=E4,
                              return_k=True)
    again = KP._QUANT[kind](k, E4, 64)
    for a, b in zip(outs, again):
        assert torch.equal(a.view(torch.uint8) if a.dtype.itemsize == 1 else a, b.view(torch.uint8) if b.dtype.itemsize == 1 else b)
    ref = fo.QUANTIZERS[kind](k.cpu(), E4) if kind != "nvfp4" else fo.quantize_nvfp4(k.cpu(), E4, 64)
    for a, b in zip(outs, ref):
        a = a.cpu()
        assert torch.equal(a.view(torch.uint8) if a.dtype.itemsize == 1 else a, b.view(torch.uint8) if b.dtype.itemsize == 1 else b)


def test_scatter_into_paged_cache():
    """Codes and residual written through a random slot table land where the decode kernel's
    block table will look for them."""
    T, H, HKV, B = 64 * 3 + 20, 512, 2, 2
    h, w = make_kproj_inputs(T, H, HKV, 128, B=B, seed=5, dtype=torch.bfloat16)
    cos, sin = rope_tables(T, 0)
    args = (h.cuda(), (w * 4).cuda(), cos.cuda(), sin.cuda(), HKV, 128)
    codes, res = KP.kproj_fused("fp8", *args, fp8_dtype=E4)
    NP = 4
    bt = make_block_table(B, NP, seed=9).cuda()
    pool_c = torch.zeros(B * NP, 64, HKV, 128, dtype=torch.uint8, device="cuda")
    pool_r = torch.zeros_like(pool_c)
    KP.kproj_fused("fp8", *args, fp8_dtype=E4, block_table=bt, out=(pool_c, pool_r))
    for b in range(B):
        for pg in range(NP):
            t0, t1 = pg * 64, min(T, pg * 64 + 64)
            slot = int(bt[b, pg])
            assert torch.equal(pool_c[slot, : t1 - t0], codes.view(torch.uint8)[b, t0:t1])
            assert torch.equal(pool_r[slot, : t1 - t0], res.view(torch.uint8)[b, t0:t1])


@pytest.mark.parametrize("rows,H,HKV", [(1, 4096, 8), (3, 4096, 8), (8, 4096, 8), (5, 512, 2), (8, 1024, 1),
                                        (2, 8192, 8), (4, 384, 1), (7, 128, 2), (9, 4096, 8), (16, 4096, 8),
                                        (24, 4096, 8), (20, 512, 2), (24, 8192, 8), (17, 384, 1)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_few_token_rows_one_launch_kernel(rows, H, HKV, dtype):
    """One decode step of a batch (at most 24 token rows) takes the cluster kernel: every cluster size
    it picks (hidden 128 ... 8192), row counts in one and in several blocks of eight, against the
    oracle's recipe and against the same rows inside a call large enough to take the tensor-memory GEMM."""
    h, w = make_kproj_inputs(1, H, HKV, 128, B=rows, seed=90 + rows, dtype=dtype)
    w = w * 4.0
    bias = (0.1 * torch.randn(HKV * 128, generator=torch.Generator().manual_seed(2))).to(dtype)
    cos, sin = rope_tables(1, 33, dtype)
    want = fo.kproj_rope(h, w, cos, sin, HKV, 128, bias=bias)
    (got,) = KP.kproj_fused(None, h.cuda(), w.cuda(), cos.cuda(), sin.cuda(), HKV, 128, bias=bias.cuda())
    assert status() == 0
    ulp = 2.0 ** (-7 if dtype == torch.bfloat16 else -10)
    scale = want.float().abs().max().item()
    err = (got.float().cpu() - want.float()).abs()
    assert err.max().item() <= 2.5 * ulp * scale, err.max().item()
    assert err.mean().item() <= 0.05 * ulp * scale, err.mean().item()
    # the same rows as the first token of 70 sequences (70 rows: the other kernel), same RoPE position
    hb = torch.cat([h, h[:1].expand(70 - rows, -1, -1)], 0).contiguous()
    (big,) = KP.kproj_fused(None, hb.cuda(), w.cuda(), cos.cuda(), sin.cuda(), HKV, 128, bias=bias.cuda())
    diff = (got.float() - big[:rows].float()).abs()
    assert diff.max().item() <= 2.5 * ulp * scale and (diff > 0).float().mean().item() <= 0.02


@pytest.mark.parametrize("kind", ["fp8", "fp4"])
def test_few_token_rows_append_into_paged_cache(kind):
    """The fused quantiser of the few-row kernel appends at slot_pos0 through the block table and
    writes what the standalone quantiser makes of the K it returns."""
    from ffa_speedtest_b200 import quantize as Q
    B, H, HKV, pos = 4, 4096, 8, 64 * 2 + 37
    h, w = make_kproj_inputs(1, H, HKV, 128, B=B, seed=12, dtype=torch.bfloat16)
    cos, sin = rope_tables(1, pos, torch.bfloat16)
    args = (h.cuda(), (w * 4).cuda(), cos.cuda(), sin.cuda(), HKV, 128)
    codes, res, k = KP.kproj_fused(kind, *args, fp8_dtype=E4, return_k=True)
    again = KP._QUANT[kind](k, E4, 64)
    assert torch.equal(codes.view(torch.uint8), again[0].view(torch.uint8))
    assert torch.equal(res.view(torch.uint8), again[1].view(torch.uint8))
    NP = 4
    bt = make_block_table(B, NP, seed=4).cuda()
    cw = codes.view(torch.uint8).shape[-1]
    pool_c = torch.zeros(B * NP, 64, HKV, cw, dtype=torch.uint8, device="cuda")
    pool_r = torch.zeros(B * NP, 64, HKV, 128, dtype=torch.uint8, device="cuda")
    KP.kproj_fused(kind, *args, fp8_dtype=E4, block_table=bt, out=(pool_c, pool_r), position=pos)
    assert status() == 0
    for b in range(B):
        slot = int(bt[b, pos // 64])
        assert torch.equal(pool_c[slot, pos % 64], codes.view(torch.uint8)[b, 0])
        assert torch.equal(pool_r[slot, pos % 64], res.view(torch.uint8)[b, 0])
    assert int((pool_c != 0).any(dim=-1).any(dim=-1).sum()) == B      # nothing else was written


def test_short_chunk_takes_the_few_row_kernel_with_positions():
    """B x T <= 24 with T > 1: RoPE rows and cache slots follow (row % T), per sequence."""
    B, T, H, HKV, pos = 2, 12, 4096, 8, 64 + 55          # the chunk crosses a page boundary
    h, w = make_kproj_inputs(T, H, HKV, 128, B=B, seed=31, dtype=torch.bfloat16)
    cos, sin = rope_tables(T, pos, torch.bfloat16)
    args = (h.cuda(), (w * 4).cuda(), cos.cuda(), sin.cuda(), HKV, 128)
    codes, res, k = KP.kproj_fused("fp8", *args, fp8_dtype=E4, return_k=True)
    want = fo.kproj_rope(h, w * 4, cos, sin, HKV, 128)
    err = (k.float().cpu() - want.float()).abs()
    scale = want.float().abs().max().item()
    assert err.max().item() <= 2.5 * 2.0 ** -7 * scale and err.mean().item() <= 0.05 * 2.0 ** -7 * scale
    NP = 3
    bt = make_block_table(B, NP, seed=6).cuda()
    pool_c = torch.zeros(B * NP, 64, HKV, 128, dtype=torch.uint8, device="cuda")
    pool_r = torch.zeros_like(pool_c)
    KP.kproj_fused("fp8", *args, fp8_dtype=E4, block_table=bt, out=(pool_c, pool_r), position=pos)
    assert status() == 0
    for b in range(B):
        for t in range(T):
            slot, off = int(bt[b, (pos + t) // 64]), (pos + t) % 64
            assert torch.equal(pool_c[slot, off], codes.view(torch.uint8)[b, t])
            assert torch.equal(pool_r[slot, off], res.view(torch.uint8)[b, t])


@pytest.mark.parametrize("kind", ["q2", "nf4"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,T,H,HKV", [(2, 1024, 512, 8), (1, 2048, 256, 8), (3, 512, 256, 8), (1, 4864, 128, 8)])
def test_minmax_reduced_in_the_epilogue_equals_the_standalone_quantiser(kind, dtype, B, T, H, HKV):
    """Whole tiles of one sequence (T a multiple of 128, enough tiles for an unsplit GEMM): the epilogue
    leaves per-32-row min/max, a fold kernel finishes the scales.  Same bits as quantising the returned
    K with the standalone quantiser and with the oracle, per sequence of the batch."""
    h, w = make_kproj_inputs(T, H, HKV, 128, B=B, seed=61, dtype=dtype)
    cos, sin = rope_tables(T, 5, dtype)
    *outs, k = KP.kproj_fused(kind, h.cuda(), (w * 4).cuda(), cos.cuda(), sin.cuda(), HKV, 128, fp8_dtype=E4,
                              return_k=True)
    assert status() == 0
    again = KP._QUANT[kind](k, E4, 64)
    ref = fo.QUANTIZERS[kind](k.cpu(), E4)
    for a, b, c in zip(outs, again, ref):
        view = (lambda x: x.view(torch.uint8) if x.dtype.itemsize == 1 else x)
        assert torch.equal(view(a), view(b))
        assert torch.equal(view(a.cpu()), view(c))


def test_large_tile_count_against_cublas():
    """T = 8192 (benchmark config 3): 512 output tiles; cuBLAS + eager RoPE on the same GPU as a
    second opinion (not the oracle: its accumulation order is its own)."""
    T, H, HKV = 8192, 4096, 8
    h, w = make_kproj_inputs(T, H, HKV, 128, B=1, seed=3, device="cuda")
    cos, sin = KP.build_rope_cache(T + 11, 128, base=500000.0, device="cuda")
    cos, sin = cos[11:].contiguous(), sin[11:].contiguous()
    (got,) = KP.kproj_fused(None, h, w, cos, sin, HKV, 128)
    assert status() == 0
    want = KP.apply_rope(torch.nn.functional.linear(h, w).view(1, T, HKV, 128), cos, sin)
    err = (got - want).abs()
    scale = want.abs().max().item()
    assert err.max().item() <= 2.5 * 2.0 ** -7 * scale and err.mean().item() <= 0.05 * 2.0 ** -7 * scale
