"""End-to-end tok/s driver: a Llama-style decoder over the paged fp8 + fp8-residual cache.

    python -m ffa_speedtest_b200.fp8fp8.e2e.bench_llama_fp8fp8 --ffa-decode --batch 2 --seq-len 128 \\
        --hidden-size 512 --heads 4 --kv-heads 2 --layers 2
    python -m ffa_speedtest_b200.fp8fp8.e2e.bench_llama_fp8fp8 --compare --context 32768 --decode-steps 64 \\
        --batch 8 --hidden-size 4096 --heads 32 --kv-heads 8 --layers 2 --bs 64 --delta 8

Arguments, modes and output lines are those of the reference driver
(ffa-fp8fp8/e2e/bench_llama_fp8fp8.py:20-44 arguments, :148-161 the decode loop, :238-261 the
``[tag][Prefill]`` / ``[tag][Decode]`` lines): ``--mode decode`` feeds ``--seq-len`` tokens one by one
through the model with a fresh cache per iteration; ``--compare`` runs the dense baseline and the FFA
path one after the other.  Head dimension must be 128 (``hidden-size = 128 x heads``).

Added here: ``--context N`` fills every layer's cache with N synthetic tokens (seeded post-RoPE keys
and values written straight into the pages, no model pass) and then times ``--decode-steps`` decode
steps on top of it - the long-context regime the decode op is for; ``--json`` prints one JSON line
with the figures.  Token ids are seeded random numbers.
"""
from __future__ import annotations

import argparse
import gc
import json
import time

import torch

from ...synth import make_decode_inputs
from .fp8fp8_cache import PagedFP8Fp8Cache, resolve_fp8_dtype
from .modeling_llama import DenseCache, LlamaConfig, LlamaForCausalLM


def parse_args(argv=None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="End-to-end benchmark for the fp8+fp8 cache on a Llama-style model.")
    p.add_argument("--device", type=str, default="cuda")
    p.add_argument("--dtype", type=str, default="bf16", choices=["fp16", "bf16"])
    p.add_argument("--batch", type=int, default=2)
    p.add_argument("--seq-len", type=int, default=128)
    p.add_argument("--hidden-size", type=int, default=512)
    p.add_argument("--heads", type=int, default=4)
    p.add_argument("--kv-heads", type=int, default=2)
    p.add_argument("--layers", type=int, default=1)
    p.add_argument("--intermediate-size", type=int, default=0)
    p.add_argument("--vocab-size", type=int, default=128)
    p.add_argument("--warmup", type=int, default=2)
    p.add_argument("--iters", type=int, default=5)
    p.add_argument("--mode", type=str, default="both", choices=["prefill", "decode", "both"])
    p.add_argument("--compare", action="store_true", help="dense baseline, then the FFA decode path")
    p.add_argument("--ffa-decode", action="store_true", help="route single-token steps to the FFA decode op")
    p.add_argument("--bs", type=int, default=128, help="block size of the decode op")
    p.add_argument("--sbs", type=int, default=None, help="prune-group size of the decode op")
    p.add_argument("--delta", type=float, default=5.0)
    p.add_argument("--no-residual", action="store_true")
    p.add_argument("--no-fused-append", action="store_true", help="project K with torch and append the keys instead")
    p.add_argument("--context", type=int, default=0, help="synthetic tokens already in the cache before decoding")
    p.add_argument("--decode-steps", type=int, default=32, help="decode steps timed on top of --context")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--json", action="store_true")
    return p.parse_args(argv)


def clear_cuda() -> None:
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()


def benchmark_ms(fn, iters: int, warmup: int) -> float:
    """Mean milliseconds per call: CUDA events around ``iters`` calls after ``warmup`` calls
    (reference :86-106)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters


def main(argv=None) -> dict:
    args = parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    torch.manual_seed(args.seed)
    device = torch.device(args.device)
    dtype = {"fp16": torch.float16, "bf16": torch.bfloat16}[args.dtype]
    if args.hidden_size % args.heads != 0 or args.heads % args.kv_heads != 0:
        raise ValueError("hidden-size must be divisible by heads, heads by kv-heads")
    if args.hidden_size // args.heads != 128:
        raise ValueError("the decode op is built for head_dim 128: choose hidden-size = 128 x heads")
    use_residual = not args.no_residual
    fp8_dtype = resolve_fp8_dtype(device)
    capacity = max(args.seq_len, args.context + args.decode_steps, 64)
    cfg = LlamaConfig(hidden_size=args.hidden_size, num_attention_heads=args.heads, num_key_value_heads=args.kv_heads,
                      num_hidden_layers=args.layers, intermediate_size=args.intermediate_size,
                      max_position_embeddings=capacity, vocab_size=args.vocab_size)
    model = LlamaForCausalLM(cfg).to(device=device, dtype=dtype).eval()
    gen = torch.Generator().manual_seed(args.seed)
    input_ids = torch.randint(0, args.vocab_size, (args.batch, max(args.seq_len, args.decode_steps)), generator=gen).to(device)
    bs = args.bs
    sbs = args.sbs if args.sbs is not None else bs
    print(f"[Info] device={device.type} dtype={dtype} fp8_dtype={fp8_dtype} batch={args.batch} seq_len={args.seq_len} "
          f"hidden={args.hidden_size} heads={args.heads} kv_heads={args.kv_heads} layers={args.layers} "
          f"use_residual={use_residual} compare={args.compare} ffa_decode={args.ffa_decode} context={args.context}")
    out: dict = {"batch": args.batch, "layers": args.layers, "hidden": args.hidden_size, "context": args.context}

    def new_cache(use_ffa: bool):
        if use_ffa:
            return PagedFP8Fp8Cache(args.batch, args.kv_heads, capacity, use_fp8_residual=use_residual,
                                    fp8_dtype=fp8_dtype, dtype=dtype, device=device)
        return DenseCache(args.batch, args.kv_heads, capacity, 128, dtype, device)

    def set_attn_settings(use_ffa: bool) -> None:
        cfg.attn_settings = ({"use_ffa_decode": True, "BS": bs, "SBS": sbs, "delta": args.delta,
                              "use_fp8_residual": use_residual, "fused_append": not args.no_fused_append}
                             if use_ffa else {})

    def run_prefill(use_ffa: bool) -> None:
        model(input_ids[:, :args.seq_len], past_key_values=new_cache(use_ffa), use_cache=True)

    def run_decode(use_ffa: bool) -> None:
        cache = new_cache(use_ffa)
        for t in range(args.seq_len):
            model(input_ids[:, t:t + 1], past_key_values=cache, use_cache=True)

    def run_variant(tag: str, use_ffa: bool) -> None:
        set_attn_settings(use_ffa)
        clear_cuda()
        tokens = args.batch * args.seq_len
        if args.context <= 0 and args.mode in ("prefill", "both"):
            ms = benchmark_ms(lambda: run_prefill(use_ffa), args.iters, args.warmup)
            print(f"[{tag}][Prefill][cache] {ms:.3f} ms/iter, {tokens / (ms / 1000.0):.1f} tok/s")
            out[f"{tag}_prefill_ms"] = ms
        clear_cuda()
        if args.context <= 0 and args.mode in ("decode", "both"):
            ms = benchmark_ms(lambda: run_decode(use_ffa), args.iters, args.warmup)
            print(f"[{tag}][Decode] {ms:.3f} ms/iter, {ms / args.seq_len:.3f} ms/token, {tokens / (ms / 1000.0):.1f} tok/s")
            out[f"{tag}_decode_ms_per_token"] = ms / args.seq_len
            out[f"{tag}_decode_tok_s"] = tokens / (ms / 1000.0)
        if args.context > 0:
            # long-context decode: seeded keys / values in every layer's cache, then timed decode steps
            cache = new_cache(use_ffa)
            _, k, v = make_decode_inputs(args.batch, args.context, args.heads, args.kv_heads, 128, seed=args.seed + 1,
                                         dtype=dtype, device=device)
            for layer in range(args.layers):
                cache.update(k, v, layer)
            del k, v
            steps = args.decode_steps

            def rewind() -> None:
                if use_ffa:
                    cache.crop(args.context)
                else:
                    cache.len = [args.context] * len(cache.len)

            def decode_steps() -> None:
                rewind()
                for t in range(steps):
                    model(input_ids[:, t:t + 1], past_key_values=cache, use_cache=True)

            ms = benchmark_ms(decode_steps, args.iters, args.warmup)
            per_tok = ms / steps
            tps = args.batch * steps / (ms / 1000.0)
            print(f"[{tag}][Decode@{args.context}] {ms:.3f} ms/iter, {per_tok:.3f} ms/token, {tps:.1f} tok/s")
            out[f"{tag}_decode_ms_per_token"] = per_tok
            out[f"{tag}_decode_tok_s"] = tps
            if use_ffa:
                ws = cache.layers[0]._workspace
                if ws is not None:
                    NTB = -(-cache.layers[0].seq_len // bs) * (bs // sbs)
                    out["skip_ratio_layer0"] = 1.0 - float(ws.mask_view(args.batch, args.kv_heads, NTB).float().mean())
            del cache
        clear_cuda()

    t0 = time.time()
    if args.compare:
        run_variant("Baseline", False)
        run_variant("FP8FP8", True)
    elif args.ffa_decode:
        run_variant("FP8FP8", True)
    else:
        run_variant("Baseline", False)
    out["wall_s"] = time.time() - t0
    if args.json:
        print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
