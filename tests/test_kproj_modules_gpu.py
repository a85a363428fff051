"""The per-variant ``fused_kproj_rope_<variant>`` modules, called by the reference's names and argument
order (ffa-q2fp8/fused_kproj_rope_q2fp8.py:402-566, ffa-fp4fp8/...:390-522, ffa-nf4fp8/...:415-580,
ffa-fp8fp8/...:67-135, ffa-nvfp4fp8/...:117-190) on the shape of the reference's own smoke test
(:569-625: B=2, T=32, H=256, HKV=4, seed 0, randn h and W, rope tables in the activation dtype) and
judged by its tolerances: packed mismatch <= 1 %, scale / zero max error <= 0.05, residual mean
error <= 0.05.  Head_dim is 128 here (the reference's smoke uses 64; this build has one head size),
and W is divided by sqrt(H) so that K is of order one: with K of order fifty, as randn W gives at
H = 256, one float16 ulp of a scale (0.03) is already most of the absolute tolerance."""
import importlib

import pytest
import torch

pytestmark = pytest.mark.gpu

MODULES = {
    # variant dir: (function stem, extra positional args after head_dim, outputs: kinds)
    "q2fp8": ("kproj_rope_quantize", (), ("codes", "scale", "scale", "res")),
    "fp8fp8": ("kproj_rope_quantize", (), ("fp8", "res")),
    "fp4fp8": ("kproj_rope_fp4", (), ("codes", "res")),
    "nf4fp8": ("kproj_rope_nf4", (), ("codes", "scale", "res")),
    "nvfp4fp8": ("kproj_rope_quantize", (64,), ("codes", "scale", "res")),
}
TILE_KWARGS = dict(block_t=16, block_h=32, block_pair=16, num_warps=4, num_stages=2)


def compare(kinds, got, ref):
    assert len(got) == len(ref) == len(kinds)
    for kind, g, r in zip(kinds, got, ref):
        assert g.shape == r.shape and g.dtype == r.dtype, (kind, g.shape, r.shape, g.dtype, r.dtype)
        if kind == "codes":
            assert (g != r).float().mean().item() <= 0.01
        elif kind == "fp8":
            assert (g.view(torch.uint8) != r.view(torch.uint8)).float().mean().item() <= 0.01
        elif kind == "scale":
            assert (g.float() - r.float()).abs().max().item() <= 0.05
        else:
            assert (g.float() - r.float()).abs().mean().item() <= 0.05


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("variant", sorted(MODULES))
def test_module_functions_by_reference_names(variant, dtype):
    stem, extra, kinds = MODULES[variant]
    mod = importlib.import_module(f"ffa_speedtest_b200.{variant}.fused_kproj_rope_{variant}")
    reference, triton, fused = (getattr(mod, f"{stem}_{s}") for s in ("reference", "triton", "fused"))
    dev = torch.device("cuda")
    B, T, H, HKV, K = 2, 32, 256, 4, 128
    torch.manual_seed(0)
    h = torch.randn(B, T, H, device=dev, dtype=dtype)
    w_k = (torch.randn(HKV * K, H, device=dev) / H ** 0.5).to(dtype)
    cos, sin = mod.build_rope_cache(T, K, device=dev, dtype=dtype)
    f8 = torch.float8_e5m2

    ref = reference(h, w_k, cos, sin, HKV, K, *extra, fp8_dtype=f8)
    compare(kinds, fused(h, w_k, cos, sin, HKV, K, *extra, fp8_dtype=f8), ref)
    # the Triton tile knobs of the reference are accepted (and have no meaning for the tcgen05 tile)
    tile = {} if variant in ("fp8fp8", "nvfp4fp8") else TILE_KWARGS
    compare(kinds, triton(h=h, w_k=w_k, cos=cos, sin=sin, num_kv_heads=HKV, head_dim=K, fp8_dtype=f8,
                          **({"page_size": 64} if extra else {}), **tile), ref)
    # weight given as [in, out] is transposed like the reference's _normalize_k_weight does
    compare(kinds, fused(h, w_k.t().contiguous(), cos, sin, HKV, K, *extra, fp8_dtype=f8), ref)
    # with a bias, default fp8 type (e5m2, reference _resolve_fp8_dtype)
    bias = (0.1 * torch.randn(HKV * K, device=dev)).to(dtype)
    ref_b = reference(h, w_k, cos, sin, HKV, K, *extra, bias)
    compare(kinds, fused(h, w_k, cos, sin, HKV, K, *extra, bias), ref_b)
    assert ref_b[-1].dtype == torch.float8_e5m2


def test_rope_helpers_follow_the_reference_convention():
    """cos/sin = cat([freqs, freqs]); pairs are interleaved (2j, 2j+1): ffa-q2fp8/fused_kproj_rope_q2fp8.py:10-37."""
    from ffa_speedtest_b200.q2fp8.fused_kproj_rope_q2fp8 import apply_rope, build_rope_cache, rotate_half
    cos, sin = build_rope_cache(5, 8, base=10000.0)
    assert cos.shape == (5, 8) and torch.equal(cos[:, :4], cos[:, 4:])
    inv = 1.0 / (10000.0 ** (torch.arange(0, 8, 2).float() / 8))
    assert torch.allclose(cos[3, :4], torch.cos(3 * inv))
    x = torch.arange(8.0).view(1, 1, 1, 8)
    assert rotate_half(x).flatten().tolist() == [-1, 0, -3, 2, -5, 4, -7, 6]
    y = apply_rope(x.expand(1, 5, 1, 8), cos, sin)
    assert torch.allclose(y[0, 2, 0, 0], x[0, 0, 0, 0] * cos[2, 0] - x[0, 0, 0, 1] * sin[2, 0])
    assert torch.allclose(y[0, 2, 0, 1], x[0, 0, 0, 1] * cos[2, 1] + x[0, 0, 0, 0] * sin[2, 1])
