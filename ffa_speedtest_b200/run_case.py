"""Run one decode or K-projection case on synthetic inputs a few times.

    python -m ffa_speedtest_b200.run_case decode --variant fp8fp8 --B 2 --T 32768 --iters 3
    python -m ffa_speedtest_b200.run_case kproj  --variant q2fp8  --T 8192 --iters 3

The command behind the profiler captures of this package (their summaries quote it): it builds the
seeded inputs, quantises K with this package's quantisers, calls the public entry point ``iters``
times and prints the kept-page fraction (decode) or the output shapes (kproj).  Sizes are whatever
is asked for; for a profiler pick a case it can replay (a few hundred MB of cache).
"""
from __future__ import annotations

import argparse

import torch

from . import quantize as Q
from .decode import allocate_decode_workspace, decode_call
from .kproj import build_rope_cache, kproj_fused
from .synth import make_decode_inputs, make_kproj_inputs

KINDS = Q.VARIANTS
quantise = Q.quantize_variant


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("what", choices=["decode", "kproj"])
    ap.add_argument("--variant", default="fp8fp8", choices=sorted(KINDS))
    ap.add_argument("--B", type=int, default=2)
    ap.add_argument("--T", type=int, default=32768)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--delta", type=float, default=8.0)
    ap.add_argument("--fp8", default="e4m3", choices=["e4m3", "e5m2"])
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--kernel", default="auto", choices=["auto", "ws", "pipe", "fp16"], help="decode kernel")
    ap.add_argument("--SBS", type=int, default=64, help="tokens per prune group (decode)")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    dev = torch.device("cuda", 0)
    f8 = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}[args.fp8]
    kind = KINDS[args.variant]

    if args.what == "decode":
        q, k, v = make_decode_inputs(args.B, args.T, 32, 8, 128, seed=args.seed, device=dev)
        BS = max(64, args.SBS)
        codes, scale, zero, res = quantise(kind, k, f8, BS)
        del k
        ws = allocate_decode_workspace(q, v, BS=BS, SBS=args.SBS)
        for _ in range(args.iters):
            decode_call(kind, q, codes, v, k_scale=scale, k_zero=zero, k_residual=res, BS=BS, SBS=args.SBS,
                        delta=args.delta, workspace=ws, kernel=args.kernel)
        torch.cuda.synchronize()
        print(f"decode {args.variant} B={args.B} T={args.T}: kept fraction {float(ws.mask.float().mean()):.4f}, "
              f"status {ws.status()}")
    else:
        h, w = make_kproj_inputs(args.T, 4096, 8, 128, B=args.B if args.B else 1, seed=args.seed, device=dev)
        cos, sin = build_rope_cache(args.T, 128, base=500000.0, device=dev)
        cos, sin = cos.to(h.dtype), sin.to(h.dtype)
        outs = None
        for _ in range(args.iters):
            outs = kproj_fused(kind, h, w, cos, sin, 8, 128, fp8_dtype=f8)
        torch.cuda.synchronize()
        print(f"kproj {args.variant} B={h.shape[0]} T={args.T}: outputs {[tuple(o.shape) for o in outs]}")


if __name__ == "__main__":
    main()
