"""Streaming scale maintenance: tokens appended at decode time to a paged cache in every coarse-K format."""
import pytest
import torch

from ffa_speedtest_b200 import quantize as Q
from ffa_speedtest_b200.decode import decode_call
from ffa_speedtest_b200.streaming import StreamingKVCache
from ffa_speedtest_b200.synth import make_decode_inputs

pytestmark = pytest.mark.gpu
F8 = torch.float8_e4m3fn


def gather(cache, pool, T):
    """Pool rows of tokens [0, T) of every sequence, back in the reference layout [B, T, HKV, W]."""
    rows = cache._rows(0, T)
    flat = pool.view(-1, *pool.shape[2:]).view(torch.uint8)
    return flat[rows].view(cache.batch, T, *flat.shape[1:])


def whole(kind, k):
    codes, scale, zero, res = Q.quantize_variant(kind, k.contiguous(), F8, 64)
    return codes, scale, zero, res


@pytest.mark.parametrize("kind", ["q2", "nf4", "nvfp4", "fp4", "fp8"])
def test_appends_inside_the_range_equal_whole_sequence_quantisation(kind):
    """Prompt of 200 tokens, then 70 tokens one by one and in chunks (crossing two page boundaries).  The
    appended tokens lie inside the prompt's per-channel range, so the whole-sequence quantiser of the
    lengthened sequence has the same scales: codes, residual, scales and the decode output must be
    identical bit for bit."""
    B, T0, T1, HQ, HKV = 2, 200, 270, 8, 2
    q, k, v = make_decode_inputs(B, T1, HQ, HKV, 128, seed=4, device="cuda", n_heavy=3)
    k[:, T0:] *= 0.5                                    # stay inside the range of the prompt
    if kind in ("q2", "nf4"):
        lo, hi = k[:, :T0].amin(1, keepdim=True), k[:, :T0].amax(1, keepdim=True)
        k[:, T0:] = torch.minimum(torch.maximum(k[:, T0:], lo), hi)
    cache = StreamingKVCache(kind, B, HKV, 512, fp8_dtype=F8)
    cache.prefill(k[:, :T0], v[:, :T0])
    t = T0
    for step in (1, 1, 7, 1, 30, 1, 29):
        cache.append(k[:, t:t + step], v[:, t:t + step])
        t += step
    assert t == T1 and cache.get_seq_length() == T1
    codes, scale, zero, res = whole(kind, k)
    assert torch.equal(gather(cache, cache.codes, T1), codes.view(torch.uint8))
    assert torch.equal(gather(cache, cache.residual, T1), res.view(torch.uint8))
    assert torch.equal(gather(cache, cache.value, T1).view(torch.bfloat16), v)
    if kind == "q2":
        assert torch.equal(cache.scale, scale) and torch.equal(cache.zero, zero)
    elif kind == "nf4":
        assert torch.equal(cache.scale, scale)
    elif kind == "nvfp4":
        assert torch.equal(cache.scale[:, :scale.shape[1]], scale)
    assert cache.drift() <= 1.01          # the frozen range is (max - min) rounded to K's dtype
    want = decode_call(kind, q, codes, v, k_scale=scale, k_zero=zero, k_residual=res, BS=64, SBS=64, delta=5.0)
    got = cache.decode(q, delta=5.0)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("kind", ["q2", "nf4"])
def test_tokens_outside_the_range_saturate_and_the_residual_carries_the_rest(kind):
    """New tokens twice as large as anything in the prompt: the scales stay frozen, the codes saturate,
    code + residual still reconstruct K to fp8-residual accuracy, and drift() reports the move."""
    B, T0, n_new, HKV = 1, 128, 16, 2
    _, k, v = make_decode_inputs(B, T0 + n_new, 8, HKV, 128, seed=9, device="cuda", n_heavy=0)
    k[:, T0:] *= 2.5
    cache = StreamingKVCache(kind, B, HKV, 256, fp8_dtype=F8)
    cache.prefill(k[:, :T0], v[:, :T0])
    scale0 = cache.scale.clone()
    cache.append(k[:, T0:], v[:, T0:])
    assert torch.equal(cache.scale, scale0)                     # frozen
    assert cache.drift() > 1.5
    T = T0 + n_new
    codes = gather(cache, cache.codes, T)[:, T0:]
    res = gather(cache, cache.residual, T)[:, T0:].view(F8).float()
    nib = torch.stack([(codes >> s) & (3 if kind == "q2" else 15) for s in ((0, 2, 4, 6) if kind == "q2" else (0, 4))],
                      dim=-1).flatten(-2).float()
    if kind == "q2":
        deq = nib * cache.scale.float()[:, None] + cache.zero.float()[:, None]
    else:
        from oracle.ffa_oracle import NF4_LEVELS
        book = torch.tensor(NF4_LEVELS, device="cuda")
        deq = book[nib.long()] * cache.scale.float()[:, None]
    kf = k[:, T0:].float()
    err = (deq + res - kf).abs()
    # e4m3 keeps 4 significant bits: the residual is off by at most 1/16 of its size (2^-10 in its
    # subnormal range), plus the bf16 rounding of K's arithmetic
    assert bool((err <= (kf - deq).abs() / 16 + 2e-2 * kf.abs() + 2e-3).all())


def test_append_before_prefill_is_refused_for_sequence_scaled_formats():
    cache = StreamingKVCache("q2", 1, 2, 128)
    _, k, v = make_decode_inputs(1, 4, 8, 2, 128, seed=1, device="cuda")
    with pytest.raises(RuntimeError, match="prefill"):
        cache.append(k, v)
    with pytest.raises(ValueError, match="capacity"):
        StreamingKVCache("fp8", 1, 2, 64).append(*make_decode_inputs(1, 65, 8, 2, 128, seed=1, device="cuda")[1:])
