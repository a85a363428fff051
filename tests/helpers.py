"""Shared helpers of the test-suite: golden cases, input regeneration, digests."""
from __future__ import annotations

import hashlib
from pathlib import Path

import numpy as np
import torch

from ffa_speedtest_b200.synth import make_decode_inputs
from oracle import ffa_oracle as fo

GOLDEN = Path(__file__).resolve().parent / "golden"
FP8 = {"e5m2": torch.float8_e5m2, "e4m3": torch.float8_e4m3fn}
FLT = {"bf16": torch.bfloat16, "fp16": torch.float16}
KINDS = ("q2", "fp8", "fp4", "nf4", "nvfp4")
SMALL_CASES = ("ragged", "g8_e4m3", "nores_extth", "bs128", "sbs128", "sbs256_fp16", "sbs32", "sbs16_fp16")


def raw(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype in (torch.float8_e5m2, torch.float8_e4m3fn):
        return t.view(torch.uint8).numpy()
    return t.numpy()


def digest(*tensors: torch.Tensor) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(raw(t).tobytes())
    return h.hexdigest()


def from_raw(a: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(dtype)


class GoldenCase:
    """One decode golden: regenerated inputs plus the reference's outputs."""

    def __init__(self, kind: str, name: str):
        z = np.load(GOLDEN / f"decode_{kind}_{name}.npz")
        self.kind, self.name = kind, name
        B, T, HQ, HKV, D, BS, SBS, seed, n_heavy = (int(x) for x in z["meta"])
        self.B, self.T, self.HQ, self.HKV, self.D, self.BS, self.SBS = B, T, HQ, HKV, D, BS, SBS
        self.delta = float(z["delta"])
        self.dtype = FLT[str(z["dtype"])]
        self.fp8 = FP8[str(z["fp8"])]
        self.use_res = bool(z["use_res"])
        self.q, self.k, self.v = make_decode_inputs(B, T, HQ, HKV, D, seed=seed, dtype=self.dtype, n_heavy=n_heavy)
        self.sha = {key[4:]: str(z[key]) for key in z.files if key.startswith("sha_")}
        self.th = torch.from_numpy(z["th"]) if "th" in z.files else None
        self.o_ref = torch.from_numpy(z["o"])          # fp32, not rounded to the I/O dtype
        self.mask_ref = torch.from_numpy(z["mask"])

    def quantise(self):
        """Oracle quantiser on the regenerated K -> (CoarseK, residual)."""
        return fo.make_coarse(self.kind, self.k, self.fp8, self.BS)


def band_ok(mask_a: torch.Tensor, mask_b: torch.Tensor, block_max: torch.Tensor, th: torch.Tensor, G: int,
            tol: float = 1e-3) -> bool:
    """Kept sets must agree except for pages whose decisive coarse maximum lies within `tol`
    of its threshold.  block_max [B,HQ,NTBS], th [B,HQ], masks [B,HKV,NTBS]."""
    diff = mask_a.to(torch.int8) != mask_b.to(torch.int8)
    if not bool(diff.any()):
        return True
    B, HQ, N = block_max.shape
    margin = (block_max - th.unsqueeze(-1)).abs().view(B, HQ // G, G, N).amin(dim=2)   # closest head decides
    return bool((margin[diff] <= tol).all())
