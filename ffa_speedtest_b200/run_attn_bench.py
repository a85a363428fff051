"""Length sweep of one decode variant, in the shape of the reference's bench drivers.

    python -m ffa_speedtest_b200.run_attn_bench --variant q2fp8 --dtype fp16 --BS 128 --SBS 128 \
        --delta 5 --bsz 1 --max-length 32768 --step 4096 --iters 100 --warmup 50
    python -m ffa_speedtest_b200.run_attn_bench --variant q2fp8 --cudagraph --cg-warmup 2 ...
    python -m ffa_speedtest_b200.run_attn_bench --variant q2fp8 --kernel some.module.path ...

The reference drivers (ffa-q2fp8/run_attn_bench_q2.py:33-60 for the arguments, :208-262 for the
per-length measurement, utils/cache.py:36-58 for the result file) sweep a recorded Llama layer over
prefix lengths, quantise K for each length, time the decode call against a dense attention call and
store ``{"meta", "lengths", "fused_ms", "flash_ms", "skip_ratios"}`` as JSON.  This driver keeps the
arguments, the measurement protocol (CUDA events around ``iters`` calls after ``warmup`` calls) and
the result schema, on seeded synthetic activations (the recordings are not available): ``--layer``
selects the seed and ``--bsz`` the batch.  The dense column ``flash_ms`` is FlashAttention's
``flash_attn_func`` on the unquantised K, as in the reference, where that package is installed and runs
(torch's scaled-dot-product attention otherwise; ``meta["dense_baseline"]`` says which), and
``meta["sdpa_ms"]`` holds torch's own dense decode next to it; ``--no-flash`` leaves both out, like the
reference's flag.

``--kernel`` is the reference's plug-in point (run_attn_bench_q2.py:34-39, 108-113): a Python module
path that exports the variant's entry point (``attn_forward_decode_quantized`` for q2fp8, ...); it
is imported and called with the reference's keyword arguments.  The default is this package's
module for the variant.

``--cudagraph`` is the reference's second driver (run_attn_bench_q2_cudagraph.py): each length is
timed eagerly and through the variant's ``CUDAGraphDecodeRunner*`` (``replay_only()`` unless
``--cg-with-copies``), and the result file holds ``{"meta", "lengths", "<v>_ms", "<v>_cg_ms",
"flash_ms", "skip_ratios"}`` with the reference's key prefix per variant (:148-173 there) and its
``_cudagraph_replay`` / ``_cudagraph`` file-name suffix.
"""
from __future__ import annotations

import argparse
import importlib
import json
import math
from pathlib import Path

import torch

from .quantize import VARIANTS, quantize_variant
from .synth import make_decode_inputs

DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}
# variant -> (entry point, runner class, key prefix of the cudagraph result file)
ENTRY = {
    "q2fp8": ("attn_forward_decode_quantized", "CUDAGraphDecodeRunnerQ2FP8", "q2"),
    "fp8fp8": ("attn_forward_decode_fp8fp8", "CUDAGraphDecodeRunnerFP8FP8", "fp8"),
    "fp4fp8": ("attn_forward_decode_fp4", "CUDAGraphDecodeRunnerFP4FP8", "fp4"),
    "nf4fp8": ("attn_forward_decode_nf4", "CUDAGraphDecodeRunnerNF4FP8", "nf4"),
    "nvfp4fp8": ("attn_forward_decode_nvfp4fp8", "CUDAGraphDecodeRunnerNVFP4FP8", "nvfp4"),
}


def default_kernel(variant: str) -> str:
    return f"ffa_speedtest_b200.{variant}.attn_kernel.attn_kernel_v1210_fused_bsz_{variant}"


def load_kernel_components(kernel_path: str, variant: str):
    """The entry point of ``kernel_path`` for the variant (reference run_attn_bench_q2.py:108-113)."""
    module = importlib.import_module(kernel_path)
    name = ENTRY[variant][0]
    if not hasattr(module, name):
        raise AttributeError(f"Module {kernel_path} does not define '{name}'")
    return module, getattr(module, name)


def load_runner(kernel_path: str, variant: str):
    """The CUDA-graph runner class that sits next to the kernel module (``<module>_cudagraph``)."""
    module = importlib.import_module(kernel_path + "_cudagraph")
    return getattr(module, ENTRY[variant][1])


def k_args(kind: str, codes, scale, zero):
    """Positional K tensors of the variant's call, between q and v."""
    if kind == "q2":
        return [codes, scale, zero]
    if kind in ("nf4", "nvfp4"):
        return [codes, scale]
    return [codes]


def benchmark(fn, iters: int, warmup: int) -> float:
    """Milliseconds per call: CUDA events around ``iters`` calls after ``warmup`` calls
    (the reference's utils/bench.py:7-20)."""
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


def dense_attention(q, k, v, sm_scale: float, prefer):
    """The dense baseline on the unquantised K, V ``[B, L, HKV, D]`` and q ``[B, 1, HQ, D]``: FlashAttention's
    ``flash_attn_func`` as in the reference (utils/flash.py) where it is installed and runs on this GPU,
    torch's scaled_dot_product_attention otherwise.  Returns ``(callable, name)``; ``prefer`` is the name a
    previous length settled on."""
    if prefer in (None, "flash_attn"):
        try:
            from flash_attn import flash_attn_func
            fn = lambda: flash_attn_func(q, k, v, softmax_scale=sm_scale, causal=False)
            fn()
            torch.cuda.synchronize()
            return fn, "flash_attn"
        except Exception:
            pass
    qd, kd, vd = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)          # [B, H, L, D]
    return (lambda: torch.nn.functional.scaled_dot_product_attention(qd, kd, vd, scale=sm_scale, enable_gqa=True),
            "torch_sdpa")


def to_k(n: int) -> str:
    val = n / 1024.0
    return f"{int(val)}k" if abs(val - int(val)) < 1e-9 else f"{val:.1f}k"


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--variant", default="q2fp8", choices=sorted(VARIANTS))
    ap.add_argument("--kernel", default=None, help="Python module path of the variant's decode entry point")
    ap.add_argument("--dtype", default="fp16", choices=sorted(DTYPES))
    ap.add_argument("--BS", type=int, default=128)
    ap.add_argument("--SBS", type=int, default=None)
    ap.add_argument("--delta", type=float, default=5.0)
    ap.add_argument("--layer", type=int, default=1, help="seed of the synthetic activations")
    ap.add_argument("--bsz", type=int, default=1)
    ap.add_argument("--max-length", type=int, default=32768)
    ap.add_argument("--step", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--fp8", default="e5m2", choices=["e5m2", "e4m3"])
    ap.add_argument("--no-flash", "--no-dense", dest="no_flash", action="store_true", help="skip the dense baseline")
    ap.add_argument("--cudagraph", action="store_true", help="also time the CUDA-graph runner (second reference driver)")
    ap.add_argument("--cg-warmup", type=int, default=2, help="CUDAGraph warmup calls before capture")
    ap.add_argument("--cg-replay-only", action="store_true", default=True,
                    help="measure CUDAGraph replay time only (the reference's default)")
    ap.add_argument("--cg-with-copies", dest="cg_replay_only", action="store_false",
                    help="time runner(...) including the copies into its static buffers")
    ap.add_argument("--no-plot", action="store_true", help="accepted for compatibility: this driver never plots")
    ap.add_argument("--out-dir", default="plot_attn_bench/raw")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    dev = torch.device("cuda", 0)
    dtype = DTYPES[args.dtype]
    f8 = {"e5m2": torch.float8_e5m2, "e4m3": torch.float8_e4m3fn}[args.fp8]
    BS, SBS = args.BS, args.SBS or args.BS
    kind = VARIANTS[args.variant]
    kernel_path = args.kernel or default_kernel(args.variant)
    _, entry = load_kernel_components(kernel_path, args.variant)
    Runner = load_runner(kernel_path, args.variant) if args.cudagraph else None
    HQ, HKV, D = 32, 8, 128
    T_full = args.max_length
    # V (and the K that is quantised) are 16-bit like the reference's recordings; --dtype fp32 only
    # changes q, which the kernels round to float16 as the reference's do
    kv_dtype = torch.float16 if dtype == torch.float32 else dtype
    q_all, k_all, v_all = make_decode_inputs(args.bsz, T_full, HQ, HKV, D, seed=args.layer, device=dev, dtype=kv_dtype)
    q_all = q_all.to(dtype)
    sm_scale = 1.0 / math.sqrt(D)
    lengths = list(range(args.step, T_full, args.step)) + [T_full]
    bits = {} if kind == "fp8" else {"k_bits": 2 if kind == "q2" else 4}

    fused_ms, cg_ms, dense_ms, skip_ratios = [], [], [], []
    dense_name, sdpa_ms = None, []
    for L in lengths:
        k, v = k_all[:, :L].contiguous(), v_all[:, :L].contiguous()
        codes, scale, zero, res = quantize_variant(kind, k, f8, BS)
        kt = k_args(kind, codes, scale, zero)
        kw = dict(k_residual=res, scale=sm_scale, BS=BS, SBS=SBS, delta=args.delta, **bits)

        def run():
            return entry(q_all, *kt, v, return_skip_ratio=False, **kw)

        _, skip = entry(q_all, *kt, v, return_skip_ratio=True, **kw)
        fused_ms.append(benchmark(run, args.iters, args.warmup))
        skip_ratios.append(skip)
        if Runner is not None:
            runner = Runner(q_all, *kt, v, use_fp8_residual=True, warmup=args.cg_warmup, **kw)
            if args.cg_replay_only:
                cg_ms.append(benchmark(runner.replay_only, args.iters, args.warmup))
            else:
                cg_ms.append(benchmark(lambda: runner(q_all, *kt, v, k_residual=res), args.iters, args.warmup))
            del runner
        if args.no_flash:
            dense_ms.append(None)
        else:
            dense_fn, dense_name = dense_attention(q_all.to(kv_dtype), k, v, sm_scale, dense_name)
            dense_ms.append(benchmark(dense_fn, args.iters, args.warmup))
            if dense_name != "torch_sdpa":          # torch's own dense decode, as a second dense column
                sdpa_fn, _ = dense_attention(q_all.to(kv_dtype), k, v, sm_scale, "torch_sdpa")
                sdpa_ms.append(benchmark(sdpa_fn, args.iters, args.warmup))
        line = f"L={to_k(L):>6}  fused {fused_ms[-1] * 1e3:8.1f} us"
        if cg_ms:
            line += f"  cudagraph {cg_ms[-1] * 1e3:8.1f} us"
        if dense_ms[-1] is not None:
            line += f"  dense ({dense_name}) {dense_ms[-1] * 1e3:8.1f} us"
            if sdpa_ms:
                line += f"  dense (torch_sdpa) {sdpa_ms[-1] * 1e3:8.1f} us"
        print(line + f"  skip {skip:.3f}", flush=True)

    meta = dict(layer_indices=[args.layer], T_full=T_full, Hq=HQ, Hkv=HKV, D=D, Dv=D, BS=BS, SBS=SBS,
                delta=args.delta, dtype=args.dtype, step=args.step, iters=args.iters, warmup=args.warmup,
                attn_kernel=kernel_path, bsz=args.bsz, data="synthetic", fp8=args.fp8, dense_baseline=dense_name)
    stem = (f"layer_{args.layer}_Tmax{to_k(T_full)}_Hq{HQ}_Hkv{HKV}_D{D}_Dv{D}_BS{BS}_SBS{SBS}_delta{args.delta:g}_"
            f"{args.dtype}_step{args.step}_it{args.iters}_wu{args.warmup}_bsz{args.bsz}")
    if args.cudagraph:
        prefix = ENTRY[args.variant][2]
        meta["cudagraph_replay_only"] = bool(args.cg_replay_only)
        payload = {"meta": meta, "lengths": lengths, f"{prefix}_ms": fused_ms, f"{prefix}_cg_ms": cg_ms,
                   "flash_ms": dense_ms, "skip_ratios": skip_ratios}
        stem += "_cudagraph_replay" if args.cg_replay_only else "_cudagraph"
    else:
        payload = {"meta": meta, "lengths": lengths, "fused_ms": fused_ms,
                   "flash_ms": [float("nan") if x is None else x for x in dense_ms], "skip_ratios": skip_ratios}
    if sdpa_ms:
        payload["meta"]["sdpa_ms"] = sdpa_ms            # inside meta: the top-level keys stay the reference's
    path = Path(args.out_dir) / args.variant / (stem + ".json")
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps(payload, indent=2))
    print(f"saved {path}")


if __name__ == "__main__":
    main()
