"""Paged append-in-place fp8fp8 cache against the contiguous call on the same tokens."""
import pytest
import torch

from ffa_speedtest_b200 import quantize as Q
from ffa_speedtest_b200.fp8fp8.attn_kernel.attn_kernel_v1210_fused_bsz_fp8fp8 import attn_forward_decode_fp8fp8
from ffa_speedtest_b200.fp8fp8.e2e.fp8fp8_cache import PagedFP8Fp8Cache
from ffa_speedtest_b200.synth import make_decode_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("f8", [torch.float8_e5m2, torch.float8_e4m3fn])
def test_prefill_then_token_by_token_matches_contiguous(f8):
    B, T, HQ, HKV, D = 2, 333, 32, 8, 128
    q, k, v = make_decode_inputs(B, T, HQ, HKV, D, seed=11, device="cuda")
    cache = PagedFP8Fp8Cache(B, HKV, max_seq_len=512, fp8_dtype=f8)
    prefill = 300
    cache.update(k[:, :prefill], v[:, :prefill], layer_idx=0)
    for t in range(prefill, T):
        cache.update(k[:, t:t + 1], v[:, t:t + 1], layer_idx=0)
        if t in (prefill, 319, 320, T - 1):        # page boundary at 320
            base, res = Q.quantize_k_fp8_fp8_residual(k[:, :t + 1].contiguous(), f8)
            want = attn_forward_decode_fp8fp8(q, base, v[:, :t + 1].contiguous(), k_residual=res, BS=64, SBS=64, delta=8.0)
            got = cache.decode(q, layer_idx=0, delta=8.0)
            assert cache.get_seq_length() == t + 1
            assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_crop_reset_and_capacity():
    B, HKV, D = 1, 8, 128
    q, k, v = make_decode_inputs(B, 130, 32, HKV, D, seed=3, device="cuda")
    cache = PagedFP8Fp8Cache(B, HKV, max_seq_len=128)
    cache.update(k[:, :100], v[:, :100], 0)
    with pytest.raises(ValueError, match="capacity"):
        cache.update(k[:, 100:130], v[:, 100:130], 0)
    a = cache.decode(q, 0, delta=8.0).clone()
    cache.update(k[:, 100:120], v[:, 100:120], 0)
    cache.crop(100)
    assert torch.equal(cache.decode(q, 0, delta=8.0), a)
    cache.reset()
    assert cache.get_seq_length() == 0
    with pytest.raises(RuntimeError):
        cache.decode(q, 0)


def test_append_from_hidden_states_equals_append_of_projected_keys():
    """hidden -> fused K-proj + RoPE + quantise + scatter at the cache position, against projecting
    first (same kernel, K only) and appending the keys."""
    from ffa_speedtest_b200.kproj import build_rope_cache, kproj_fused
    from ffa_speedtest_b200.synth import make_kproj_inputs
    B, HKV, D, H, T = 2, 8, 128, 512, 150
    f8 = torch.float8_e4m3fn
    h, w = make_kproj_inputs(T, H, HKV, D, B=B, seed=5, device="cuda")
    cos, sin = build_rope_cache(T, D, base=500000.0, device="cuda")
    cos, sin = cos.to(h.dtype), sin.to(h.dtype)
    q, _, v = make_decode_inputs(B, T, 32, HKV, D, seed=6, device="cuda")
    fused = PagedFP8Fp8Cache(B, HKV, max_seq_len=256, fp8_dtype=f8)
    plain = PagedFP8Fp8Cache(B, HKV, max_seq_len=256, fp8_dtype=f8)
    steps = [(0, 100), (100, 101), (101, 129), (129, 150)]          # crosses the page boundary at 128
    for a, b in steps:
        fused.update_from_hidden(h[:, a:b].contiguous(), w, cos[a:b].contiguous(), sin[a:b].contiguous(), v[:, a:b], 0)
        (k,) = kproj_fused(None, h[:, a:b].contiguous(), w, cos[a:b].contiguous(), sin[a:b].contiguous(), HKV, D)
        plain.update(k, v[:, a:b], 0)
        for name in ("key_base", "key_residual", "value"):
            x, y = getattr(fused.layers[0], name), getattr(plain.layers[0], name)
            assert torch.equal(x.view(torch.uint8), y.view(torch.uint8)), (name, a, b)
    assert torch.equal(fused.decode(q, 0, delta=8.0), plain.decode(q, 0, delta=8.0))
