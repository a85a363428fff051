"""The model-side half of the end-to-end integration: a decoder whose attention routes single-token
steps to the pruned decode op on the paged fp8 + fp8-residual cache, against the same model on an
unquantised cache."""
import pytest
import torch

from ffa_speedtest_b200.fp8fp8.e2e.fp8fp8_cache import PagedFP8Fp8Cache
from ffa_speedtest_b200.fp8fp8.e2e.modeling_llama import DenseCache, LlamaConfig, LlamaForCausalLM

pytestmark = pytest.mark.gpu


def build(layers=2, hidden=512, heads=4, kv=2, vocab=97, seed=0, dtype=torch.bfloat16):
    torch.manual_seed(seed)
    cfg = LlamaConfig(hidden_size=hidden, num_attention_heads=heads, num_key_value_heads=kv, num_hidden_layers=layers,
                      max_position_embeddings=512, vocab_size=vocab)
    return cfg, LlamaForCausalLM(cfg).to(device="cuda", dtype=dtype).eval()


@pytest.mark.parametrize("fused_append", [True, False])
def test_ffa_decode_steps_track_the_dense_model(fused_append):
    """Prefill 70 tokens, decode 80 more (crossing the page boundary at 128) with nothing pruned
    (delta = 1e4): logits stay within the error of storing K as fp8 + fp8 residual."""
    B, T0, steps = 2, 70, 80
    cfg, model = build()
    ids = torch.randint(0, cfg.vocab_size, (B, T0 + steps), generator=torch.Generator().manual_seed(1)).cuda()
    dense = DenseCache(B, cfg.num_key_value_heads, 256, 128, torch.bfloat16, "cuda")
    cfg.attn_settings = {}
    ref = [model(ids[:, :T0], past_key_values=dense, use_cache=True)[:, -1]]
    for t in range(T0, T0 + steps):
        ref.append(model(ids[:, t:t + 1], past_key_values=dense, use_cache=True)[:, -1])

    cache = PagedFP8Fp8Cache(B, cfg.num_key_value_heads, 256, fp8_dtype=torch.float8_e4m3fn)
    cfg.attn_settings = {"use_ffa_decode": True, "BS": 64, "SBS": 64, "delta": 1e4, "fused_append": fused_append}
    got = [model(ids[:, :T0], past_key_values=cache, use_cache=True)[:, -1]]
    for t in range(T0, T0 + steps):
        got.append(model(ids[:, t:t + 1], past_key_values=cache, use_cache=True)[:, -1])
    assert cache.get_seq_length() == T0 + steps
    torch.testing.assert_close(got[0].float(), ref[0].float(), atol=2e-2, rtol=0)   # prefill: the same dense computation
    ref_t, got_t = torch.stack(ref).float(), torch.stack(got).float()
    assert torch.isfinite(got_t).all()
    err = (got_t - ref_t).abs().max().item()
    assert err <= 2e-2 * max(1.0, ref_t.abs().max().item()), err


def test_fused_append_equals_projected_append():
    """The two ways of appending a decode token (one fused kernel from the hidden state; torch
    projection + RoPE, then the append kernel) leave the same bytes in the cache up to the rounding of
    K before quantisation, and pruning decisions at the default delta agree on all but a few pages."""
    B, T0, steps = 1, 130, 10
    cfg, model = build(layers=1, seed=3)
    ids = torch.randint(0, cfg.vocab_size, (B, T0 + steps), generator=torch.Generator().manual_seed(2)).cuda()
    outs = {}
    for fused in (True, False):
        cache = PagedFP8Fp8Cache(B, cfg.num_key_value_heads, 256, fp8_dtype=torch.float8_e4m3fn)
        cfg.attn_settings = {"use_ffa_decode": True, "BS": 64, "SBS": 64, "delta": 5.0, "fused_append": fused}
        model(ids[:, :T0], past_key_values=cache, use_cache=True)
        last = None
        for t in range(T0, T0 + steps):
            last = model(ids[:, t:t + 1], past_key_values=cache, use_cache=True)
        outs[fused] = (last.float(), cache.layers[0].value.clone(), cache.layers[0].key_base.clone().view(torch.uint8))
    assert torch.equal(outs[True][1], outs[False][1])                           # V pages identical
    same = (outs[True][2] == outs[False][2]).float().mean().item()
    assert same > 0.99                                                        # K codes: GEMM rounding only
    assert (outs[True][0] - outs[False][0]).abs().max().item() <= 5e-2


def test_bench_driver_runs_and_reports(capsys):
    from ffa_speedtest_b200.fp8fp8.e2e import bench_llama_fp8fp8 as drv
    out = drv.main(["--compare", "--batch", "2", "--seq-len", "24", "--hidden-size", "512", "--heads", "4", "--kv-heads", "2",
                    "--layers", "1", "--iters", "1", "--warmup", "1", "--bs", "64", "--json"])
    text = capsys.readouterr().out
    assert "[Baseline][Decode]" in text and "[FP8FP8][Decode]" in text and "[FP8FP8][Prefill][cache]" in text
    assert out["FP8FP8_decode_tok_s"] > 0 and out["Baseline_decode_tok_s"] > 0
    out = drv.main(["--ffa-decode", "--context", "4096", "--decode-steps", "4", "--batch", "2", "--hidden-size", "1024",
                    "--heads", "8", "--kv-heads", "2", "--layers", "2", "--iters", "1", "--warmup", "1", "--bs", "64",
                    "--delta", "8", "--json"])
    assert out["FP8FP8_decode_tok_s"] > 0 and 0.0 <= out["skip_ratio_layer0"] < 1.0


def test_import_shim_exports_the_entry_point():
    from ffa_speedtest_b200.fp8fp8.e2e.ffa_fwd_decode_fp8fp8 import attn_forward_decode_fp8fp8
    from ffa_speedtest_b200.fp8fp8.attn_kernel.attn_kernel_v1210_fused_bsz_fp8fp8 import attn_forward_decode_fp8fp8 as direct
    assert callable(attn_forward_decode_fp8fp8) and callable(direct)
