"""Seeded synthetic Q/K/V with the qualitative features of recorded Llama activations.

The reference benchmarks run on recorded Llama-3.2-3B activations of a LongBench
document (ffa-q2fp8/run_attn_bench_q2.py:26-30, loaded by utils/load.py).  Those
recordings are not redistributable, so the benches and tests here use inputs of the
same shapes and layouts drawn from a distribution with the features that make pruning
meaningful: per-channel outlier scales on K, an attention-sink token at position 0 and
a handful of heavy-hitter tokens whose keys line up with the queries.
"""
from __future__ import annotations

import torch


def make_decode_inputs(
    B: int,
    T: int,
    HQ: int = 32,
    HKV: int = 8,
    D: int = 128,
    *,
    seed: int = 0,
    device="cpu",
    dtype: torch.dtype = torch.bfloat16,
    n_heavy: int = 16,
    sink_gain: float = 3.0,
    heavy_gain: float = 4.0,
):
    """Return ``q [B,1,HQ,D]``, ``k [B,T,HKV,D]``, ``v [B,T,HKV,D]`` in ``dtype``.

    q, k, v ~ N(0,1); K is multiplied per (kv-head, channel) by exp(0.5*N(0,1)); token 0
    gets K = sink_gain * mean of the group's queries; ``n_heavy`` seeded positions get
    K = heavy_gain * that mean."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    G = HQ // HKV
    q = torch.randn(B, 1, HQ, D, generator=g, device=dev)
    chan = torch.exp(0.5 * torch.randn(HKV, D, generator=g, device=dev))
    k = torch.randn(B, T, HKV, D, generator=g, device=dev)
    k.mul_(chan)
    v = torch.randn(B, T, HKV, D, generator=g, device=dev)
    q_mean = q.view(B, HKV, G, D).mean(dim=2)                    # [B,HKV,D]
    k[:, 0] = sink_gain * q_mean
    n_heavy = min(n_heavy, max(T - 1, 0))
    if n_heavy:
        pos = torch.randperm(T - 1, generator=g, device=dev)[:n_heavy] + 1
        k[:, pos] = heavy_gain * q_mean.unsqueeze(1)
    return q.to(dtype), k.to(dtype), v.to(dtype)


def make_block_table(B: int, n_pages: int, *, seed: int = 0, device="cpu", identity: bool = False) -> torch.Tensor:
    """Block table ``[B, n_pages]`` int32 mapping (sequence, logical page) to a slot of a
    pool of ``B*n_pages`` pages: the identity layout, or one seeded permutation of the
    whole pool."""
    n = B * n_pages
    if identity:
        return torch.arange(n, dtype=torch.int32, device=device).view(B, n_pages)
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randperm(n, generator=g).to(torch.int32).view(B, n_pages).to(device)


def make_kproj_inputs(T: int, H: int = 4096, HKV: int = 8, D: int = 128, *, B: int = 1, seed: int = 3,
                      device="cpu", dtype: torch.dtype = torch.bfloat16):
    """hidden ``[B,T,H]`` ~ N(0,1) and ``W_k [HKV*D, H]`` ~ N(0, 0.02) in ``dtype``."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    h = torch.randn(B, T, H, generator=g, device=dev).to(dtype)
    w = (0.02 * torch.randn(HKV * D, H, generator=g, device=dev)).to(dtype)
    return h, w
