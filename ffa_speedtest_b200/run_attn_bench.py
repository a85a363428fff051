"""Length sweep of one decode variant, in the shape of the reference's bench drivers.

    python -m ffa_speedtest_b200.run_attn_bench --variant q2fp8 --dtype fp16 --BS 128 --SBS 128 \
        --delta 5 --bsz 1 --max-length 32768 --step 4096 --iters 100 --warmup 50

The reference drivers (ffa-q2fp8/run_attn_bench_q2.py:33-60 for the arguments, :208-262 for the
per-length measurement, utils/cache.py:36-58 for the result file) sweep a recorded Llama layer over
prefix lengths, quantise K for each length, time the decode call against a dense attention call and
store ``{"meta", "lengths", "fused_ms", "flash_ms", "skip_ratios"}`` as JSON.  This driver keeps the
arguments, the measurement protocol (CUDA events around ``iters`` calls after ``warmup`` calls) and
the result schema, on seeded synthetic activations (the recordings are not available): ``--layer``
selects the seed and ``--bsz`` the batch.  The dense column is torch's scaled-dot-product attention
on the unquantised K (``--no-dense`` leaves it out).
"""
from __future__ import annotations

import argparse
import json
import math
from pathlib import Path

import torch

from .decode import decode_call
from .run_case import KINDS, quantise
from .synth import make_decode_inputs

DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16}


def benchmark(fn, iters: int, warmup: int) -> float:
    """Milliseconds per call: CUDA events around ``iters`` calls after ``warmup`` calls."""
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


def to_k(n: int) -> str:
    val = n / 1024.0
    return f"{int(val)}k" if abs(val - int(val)) < 1e-9 else f"{val:.1f}k"


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--variant", default="q2fp8", choices=sorted(KINDS))
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
    ap.add_argument("--no-dense", action="store_true")
    ap.add_argument("--out-dir", default="plot_attn_bench/raw")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    dev = torch.device("cuda", 0)
    dtype = DTYPES[args.dtype]
    f8 = {"e5m2": torch.float8_e5m2, "e4m3": torch.float8_e4m3fn}[args.fp8]
    BS, SBS = args.BS, args.SBS or args.BS
    kind = KINDS[args.variant]
    HQ, HKV, D = 32, 8, 128
    T_full = args.max_length
    q_all, k_all, v_all = make_decode_inputs(args.bsz, T_full, HQ, HKV, D, seed=args.layer, device=dev, dtype=dtype)
    sm_scale = 1.0 / math.sqrt(D)
    lengths = list(range(args.step, T_full, args.step)) + [T_full]

    fused_ms, dense_ms, skip_ratios = [], [], []
    for L in lengths:
        k, v = k_all[:, :L].contiguous(), v_all[:, :L].contiguous()
        codes, scale, zero, res = quantise(kind, k, f8, BS)

        def run():
            return decode_call(kind, q_all, codes, v, k_scale=scale, k_zero=zero, k_residual=res, scale=sm_scale,
                               BS=BS, SBS=SBS, delta=args.delta)

        _, skip = decode_call(kind, q_all, codes, v, k_scale=scale, k_zero=zero, k_residual=res, scale=sm_scale,
                              BS=BS, SBS=SBS, delta=args.delta, return_skip_ratio=True)
        fused_ms.append(benchmark(run, args.iters, args.warmup))
        skip_ratios.append(skip)
        if args.no_dense:
            dense_ms.append(float("nan"))
        else:
            qd = q_all.transpose(1, 2)                                   # [B, HQ, 1, D]
            kd, vd = k.transpose(1, 2), v.transpose(1, 2)                # [B, HKV, L, D]
            dense_ms.append(benchmark(
                lambda: torch.nn.functional.scaled_dot_product_attention(qd, kd, vd, scale=sm_scale, enable_gqa=True),
                args.iters, args.warmup))
        print(f"L={to_k(L):>6}  fused {fused_ms[-1] * 1e3:8.1f} us  dense {dense_ms[-1] * 1e3:8.1f} us  "
              f"skip {skip:.3f}", flush=True)

    meta = dict(layer_indices=[args.layer], T_full=T_full, Hq=HQ, Hkv=HKV, D=D, Dv=D, BS=BS, SBS=SBS,
                delta=args.delta, dtype=args.dtype, step=args.step, iters=args.iters, warmup=args.warmup,
                attn_kernel=f"ffa_speedtest_b200.{args.variant}", bsz=args.bsz, data="synthetic", fp8=args.fp8)
    name = (f"layer_{args.layer}_Tmax{to_k(T_full)}_Hq{HQ}_Hkv{HKV}_D{D}_Dv{D}_BS{BS}_SBS{SBS}_delta{args.delta:g}_"
            f"{args.dtype}_step{args.step}_it{args.iters}_wu{args.warmup}_bsz{args.bsz}.json")
    path = Path(args.out_dir) / args.variant / name
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps({"meta": meta, "lengths": lengths, "fused_ms": fused_ms, "flash_ms": dense_ms,
                                "skip_ratios": skip_ratios}, indent=2))
    print(f"saved {path}")


if __name__ == "__main__":
    main()
