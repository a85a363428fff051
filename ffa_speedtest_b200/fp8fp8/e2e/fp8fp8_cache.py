"""Paged, append-in-place fp8 + fp8-residual KV cache for decode.

Takes the place of ffa-fp8fp8/e2e/fp8fp8_cache.py (FP8Fp8DynamicLayer :36-183, FP8Fp8Cache
:186-224 there).  The reference appends with ``torch.cat`` (a full copy of the cache per token)
and keeps a dequantised shadow copy of all keys (``_refresh_fp_cache``, :63-72).  Here every
layer owns three page pools - fp8 base, fp8 residual, V - of ``[pages, 64, HKV, 128]`` behind a
block table; ``update`` quantises only the new tokens and writes them into their slots, and
``decode`` runs the pruned decode kernel straight on the pools.  No dequantised copy exists.

Layout choices: all sequences of the batch have the same length (as in the reference's batched
decode); page p of sequence b lives in pool slot ``p * B + b`` so that a decode step of the whole
batch appends into B neighbouring slots; capacity is fixed at construction (``max_seq_len``),
sized by the caller for the memory it wants to give the cache.
"""
from __future__ import annotations

from typing import Any, Optional

import torch

from ... import _lib
from ...decode import DecodeWorkspace, allocate_decode_workspace
from ...kproj import kproj_fused
from ..attn_kernel.attn_kernel_v1210_fused_bsz_fp8fp8 import attn_forward_decode_fp8fp8

PAGE = 64


def resolve_fp8_dtype(device=None) -> torch.dtype:
    """fp8 storage type; the reference prefers float8_e5m2 (fp8fp8_cache.py:14-21)."""
    return torch.float8_e5m2


class PagedFP8Fp8Layer:
    """One layer's quantised K/V pages (the role of FP8Fp8DynamicLayer)."""

    is_sliding = False

    def __init__(self, batch: int, num_kv_heads: int, max_seq_len: int, *, head_dim: int = 128,
                 use_fp8_residual: bool = True, fp8_dtype: Optional[torch.dtype] = None,
                 dtype: torch.dtype = torch.bfloat16, device="cuda"):
        if head_dim != 128:
            raise ValueError(f"this build supports head_dim 128, got {head_dim}")
        self.batch, self.num_kv_heads, self.head_dim = batch, num_kv_heads, head_dim
        self.use_fp8_residual = use_fp8_residual
        self.fp8_dtype = fp8_dtype or resolve_fp8_dtype(device)
        self.dtype, self.device = dtype, torch.device(device)
        self.pages_per_seq = -(-max_seq_len // PAGE)
        self.max_seq_len = self.pages_per_seq * PAGE
        n_pages = batch * self.pages_per_seq
        shape = (n_pages, PAGE, num_kv_heads, head_dim)
        self.key_base = torch.zeros(shape, dtype=self.fp8_dtype, device=self.device)
        self.key_residual = torch.zeros(shape, dtype=self.fp8_dtype, device=self.device) if use_fp8_residual else None
        self.value = torch.zeros(shape, dtype=dtype, device=self.device)
        pages = torch.arange(self.pages_per_seq, dtype=torch.int32, device=self.device)
        seqs = torch.arange(batch, dtype=torch.int32, device=self.device)
        self.block_table = (pages[None, :] * batch + seqs[:, None]).contiguous()          # [B, pages_per_seq]
        self.seq_len = 0
        self._workspace: Optional[DecodeWorkspace] = None

    # ---- append ----------------------------------------------------------------------------------
    def _rows(self, start: int, count: int) -> torch.Tensor:
        """Pool rows (flattened page*64 + offset) of tokens [start, start+count) of every sequence."""
        t = torch.arange(start, start + count, device=self.device)
        page = self.block_table[:, (t // PAGE)].long()                                     # [B, count]
        return (page * PAGE + (t % PAGE)[None, :]).reshape(-1)

    def _append(self, key_states: Optional[torch.Tensor], value_states: torch.Tensor, T_new: int) -> None:
        """One library call: quantise K (if given) into the base and residual pools and copy V into
        its pool, all at the page slots of positions ``seq_len .. seq_len + T_new - 1``."""
        value_states = value_states.to(self.dtype).contiguous()
        k_ptr = 0
        if key_states is not None and self.key_residual is None:
            # no residual pool: quantise to a temporary and place the base codes with torch
            from ... import quantize as Q
            base, _ = Q.quantize_k_fp8_fp8_residual(key_states.to(self.dtype).contiguous(), self.fp8_dtype)
            rows = self._rows(self.seq_len, T_new)
            self.key_base.view(-1, self.num_kv_heads, self.head_dim).view(torch.uint8)[rows] = \
                base.view(torch.uint8).reshape(-1, self.num_kv_heads, self.head_dim)
        elif key_states is not None:
            key_states = key_states.to(self.dtype).contiguous()
            k_ptr = key_states.data_ptr()
        _lib.check(_lib.lib().ffa_cache_append(
            _lib.VARIANT_CODE["fp8"], k_ptr, value_states.data_ptr(), _lib.float_code(self.dtype), self.batch, T_new,
            self.num_kv_heads, _lib.fp8_code(self.fp8_dtype), self.key_base.data_ptr(),
            self.key_residual.data_ptr() if self.key_residual is not None else 0,
            self.value.data_ptr(), self.block_table.data_ptr(), self.block_table.shape[1], self.seq_len,
            _lib.current_stream(self.device)), "ffa_cache_append")

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor,
               cache_kwargs: Optional[dict[str, Any]] = None) -> None:
        """Append ``key_states, value_states [B, T_new, HKV, D]`` (post-RoPE K)."""
        B, T_new, HKV, D = key_states.shape
        if (B, HKV, D) != (self.batch, self.num_kv_heads, self.head_dim) or value_states.shape != key_states.shape:
            raise ValueError(f"expected [B={self.batch}, T, HKV={self.num_kv_heads}, D={self.head_dim}] keys and values")
        if self.seq_len + T_new > self.max_seq_len:
            raise ValueError(f"cache capacity {self.max_seq_len} exceeded ({self.seq_len} + {T_new})")
        self._append(key_states, value_states, T_new)
        self.seq_len += T_new

    def update_from_hidden(self, hidden: torch.Tensor, w_k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                           value_states: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        """Append the tokens whose hidden states are ``hidden [B, T_new, H]``: K projection, RoPE
        (``cos, sin [T_new, D]`` are the rows of the new positions) and quantisation run as one fused
        kernel that writes the codes and the residual into this layer's pages; V is copied in."""
        if not self.use_fp8_residual:
            raise ValueError("the fused append writes base and residual; build the cache with use_fp8_residual=True")
        B, T_new, _ = hidden.shape
        HKV, D = self.num_kv_heads, self.head_dim
        if B != self.batch or value_states.shape != (B, T_new, HKV, D):
            raise ValueError(f"expected hidden [B={self.batch}, T, H] and values [B, T, {HKV}, {D}]")
        if self.seq_len + T_new > self.max_seq_len:
            raise ValueError(f"cache capacity {self.max_seq_len} exceeded ({self.seq_len} + {T_new})")
        kproj_fused("fp8", hidden, w_k, cos, sin, HKV, D, bias=bias, fp8_dtype=self.fp8_dtype,
                    block_table=self.block_table, out=(self.key_base, self.key_residual), position=self.seq_len)
        self._append(None, value_states, T_new)
        self.seq_len += T_new

    # ---- decode ----------------------------------------------------------------------------------
    def decode(self, q: torch.Tensor, **kwargs) -> torch.Tensor:
        """Pruned decode attention of ``q [B, 1, HQ, D]`` over the cached tokens; keyword arguments
        are those of ``attn_forward_decode_fp8fp8`` (scale, BS, SBS, delta, ...)."""
        if self.seq_len == 0:
            raise RuntimeError("the cache is empty")
        kwargs.setdefault("BS", PAGE)
        kwargs.setdefault("SBS", PAGE)
        kwargs.setdefault("use_fp8_residual", self.use_fp8_residual)
        if self._workspace is None:
            self._workspace = allocate_decode_workspace(q, self.value, BS=kwargs["BS"], SBS=kwargs["SBS"],
                                                        seq_len=self.max_seq_len)
        return attn_forward_decode_fp8fp8(q, self.key_base, self.value, k_residual=self.key_residual,
                                          block_table=self.block_table, seq_len=self.seq_len,
                                          workspace=self._workspace, **kwargs)

    # ---- bookkeeping (names of the reference layer) --------------------------------------------------
    def get_seq_length(self) -> int:
        return self.seq_len

    def get_max_cache_shape(self) -> int:
        return self.max_seq_len

    def crop(self, max_length: int) -> None:
        if max_length < 0:
            max_length = self.seq_len - abs(max_length)
        self.seq_len = max(0, min(self.seq_len, max_length))

    def reset(self) -> None:
        self.seq_len = 0


class PagedFP8Fp8Cache:
    """All layers' caches (the role of FP8Fp8Cache); layers are created on first use."""

    def __init__(self, batch: int, num_kv_heads: int, max_seq_len: int, *, head_dim: int = 128,
                 use_fp8_residual: bool = True, fp8_dtype: Optional[torch.dtype] = None,
                 dtype: torch.dtype = torch.bfloat16, device="cuda"):
        self._args = dict(batch=batch, num_kv_heads=num_kv_heads, max_seq_len=max_seq_len, head_dim=head_dim,
                          use_fp8_residual=use_fp8_residual, fp8_dtype=fp8_dtype, dtype=dtype, device=device)
        self.use_fp8_residual = use_fp8_residual
        self.layers: list[PagedFP8Fp8Layer] = []

    def _ensure_layer(self, layer_idx: int) -> None:
        while len(self.layers) <= layer_idx:
            self.layers.append(PagedFP8Fp8Layer(**self._args))

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs: Optional[dict[str, Any]] = None) -> None:
        self._ensure_layer(layer_idx)
        self.layers[layer_idx].update(key_states, value_states, cache_kwargs)

    def update_from_hidden(self, hidden, w_k, cos, sin, value_states, layer_idx: int, bias=None) -> None:
        self._ensure_layer(layer_idx)
        self.layers[layer_idx].update_from_hidden(hidden, w_k, cos, sin, value_states, bias)

    def decode(self, q: torch.Tensor, layer_idx: int, **kwargs) -> torch.Tensor:
        return self.layers[layer_idx].decode(q, **kwargs)

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.layers[layer_idx].get_seq_length() if len(self.layers) > layer_idx else 0

    def crop(self, max_length: int) -> None:
        for layer in self.layers:
            layer.crop(max_length)

    def reset(self) -> None:
        for layer in self.layers:
            layer.reset()
