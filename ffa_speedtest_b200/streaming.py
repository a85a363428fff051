"""A paged, appendable K/V cache for every coarse-K format - streaming scale maintenance.

The reference quantises K for a whole sequence at a time; for the formats whose scales span the
sequence (2-bit: scale and zero per channel; NF4: absmax per channel) and for nvfp4 (absmax per
page) it lists incremental updates as future work (ffa-q2fp8/OPTIMIZATION_NOTES.md:23-27: "avoid
full-sequence min/max recompute each decode step by maintaining per-(B,HKV,K) running min/max or
block-wise scales for new tokens").  This module is that update, for one layer:

* ``prefill(k, v)`` quantises the prompt exactly like the reference's quantiser and scatters codes,
  residual and V into page pools behind a block table;
* ``append(k_new, v_new)`` adds tokens at decode time:
    - fp8 / fp4 have no statistics: the new tokens are encoded on their own;
    - q2 / nf4 keep the prompt's scales **frozen** and encode the new tokens against them; codes
      saturate at the ends of the old range and the fp8 residual carries the rest, so refined scores
      keep their accuracy.  The per-channel running min/max is updated alongside (``drift()``), so a
      caller can requantise when the range has moved.  While new tokens stay inside the old range the
      cache is bit-identical to quantising the lengthened sequence from scratch;
    - nvfp4 scales are page-local: the raw K of the open (partly filled) page is kept in a small
      staging buffer and the page is re-encoded on every append, which reproduces the whole-sequence
      quantiser bit for bit at any length;
* ``decode(q, ...)`` runs the pruned decode kernel on the pools.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib, quantize as Q
from .decode import DecodeWorkspace, allocate_decode_workspace, decode_call

PAGE = 64
_CODE_BYTES = {"fp8": 128, "q2": 32, "fp4": 64, "nf4": 64, "nvfp4": 64}


class StreamingKVCache:
    def __init__(self, kind: str, batch: int, num_kv_heads: int, max_seq_len: int, *,
                 fp8_dtype: torch.dtype = torch.float8_e5m2, dtype: torch.dtype = torch.bfloat16, device="cuda"):
        if kind not in _CODE_BYTES:
            raise ValueError(f"unknown coarse-K format {kind!r}")
        self.kind, self.batch, self.num_kv_heads = kind, batch, num_kv_heads
        self.fp8_dtype, self.dtype, self.device = fp8_dtype, dtype, torch.device(device)
        self.pages_per_seq = -(-max_seq_len // PAGE)
        self.max_seq_len = self.pages_per_seq * PAGE
        n_pages = batch * self.pages_per_seq
        code_dtype = fp8_dtype if kind == "fp8" else torch.uint8
        self.codes = torch.zeros((n_pages, PAGE, num_kv_heads, _CODE_BYTES[kind]), dtype=code_dtype, device=self.device)
        self.residual = torch.zeros((n_pages, PAGE, num_kv_heads, 128), dtype=fp8_dtype, device=self.device)
        self.value = torch.zeros((n_pages, PAGE, num_kv_heads, 128), dtype=dtype, device=self.device)
        pages = torch.arange(self.pages_per_seq, dtype=torch.int32, device=self.device)
        seqs = torch.arange(batch, dtype=torch.int32, device=self.device)
        self.block_table = (pages[None, :] * batch + seqs[:, None]).contiguous()
        self.scale: Optional[torch.Tensor] = None       # q2 / nf4: [B, HKV, 128]; nvfp4: [B, pages_per_seq, HKV]
        self.zero: Optional[torch.Tensor] = None
        self.minmax: Optional[torch.Tensor] = None      # q2 / nf4: running per-channel extremes (ordered integers)
        if kind == "nvfp4":
            self.scale = torch.ones((batch, self.pages_per_seq, num_kv_heads), dtype=dtype, device=self.device)
            self.open_page = torch.zeros((batch, PAGE, num_kv_heads, 128), dtype=dtype, device=self.device)
        self.seq_len = 0
        self._workspace: Optional[DecodeWorkspace] = None

    # ---- helpers -----------------------------------------------------------------------------------
    def _rows(self, start: int, count: int) -> torch.Tensor:
        t = torch.arange(start, start + count, device=self.device)
        page = self.block_table[:, (t // PAGE)].long()
        return (page * PAGE + (t % PAGE)[None, :]).reshape(-1)

    def _scatter(self, pool: torch.Tensor, rows: torch.Tensor, src: torch.Tensor) -> None:
        flat = pool.view(-1, *pool.shape[2:])
        flat.view(torch.uint8)[rows] = src.contiguous().view(torch.uint8).reshape(-1, *flat.view(torch.uint8).shape[1:])

    def _append_v(self, v: torch.Tensor, T_new: int) -> None:
        v = v.to(self.dtype).contiguous()
        _lib.check(_lib.lib().ffa_cache_append(_lib.VARIANT_CODE["fp8"], 0, v.data_ptr(), _lib.float_code(self.dtype),
                                               self.batch, T_new, self.num_kv_heads, _lib.fp8_code(self.fp8_dtype), 0, 0,
                                               self.value.data_ptr(), self.block_table.data_ptr(), self.block_table.shape[1],
                                               self.seq_len, _lib.current_stream(self.device)), "ffa_cache_append")

    def _check(self, k: torch.Tensor, v: torch.Tensor) -> int:
        B, T_new, HKV, D = k.shape
        if (B, HKV, D) != (self.batch, self.num_kv_heads, 128) or v.shape != k.shape:
            raise ValueError(f"expected [B={self.batch}, T, HKV={self.num_kv_heads}, 128] keys and values")
        if self.seq_len + T_new > self.max_seq_len:
            raise ValueError(f"cache capacity {self.max_seq_len} exceeded ({self.seq_len} + {T_new})")
        return T_new

    # ---- prompt ------------------------------------------------------------------------------------
    def prefill(self, k: torch.Tensor, v: torch.Tensor) -> None:
        """Quantise the prompt's post-RoPE keys ``[B, T, HKV, 128]`` as the reference does and place them."""
        if self.seq_len != 0:
            raise RuntimeError("prefill goes into an empty cache; use append afterwards")
        T = self._check(k, v)
        k = k.to(self.dtype).contiguous()
        if self.kind in ("q2", "nf4"):
            self.minmax = Q.minmax_scratch(self.batch, self.num_kv_heads, self.device)
        if self.kind == "q2":
            codes, self.scale, self.zero, res = Q.quantize_k_2bit_fp8_residual(k, self.fp8_dtype, scratch=self.minmax)
        elif self.kind == "nf4":
            codes, self.scale, res = Q.encode_k_nf4_fp8_residual(k, self.fp8_dtype, scratch=self.minmax)
        elif self.kind == "nvfp4":
            codes, sc, res = Q.encode_k_nvfp4_fp8_residual(k, self.fp8_dtype, PAGE)
            self.scale[:, :sc.shape[1]] = sc
            tail = T % PAGE
            if tail:
                self.open_page[:, :tail] = k[:, T - tail:]
        elif self.kind == "fp4":
            codes, res = Q.encode_k_fp4_fp8_residual(k, self.fp8_dtype)
        else:
            codes, res = Q.quantize_k_fp8_fp8_residual(k, self.fp8_dtype)
        rows = self._rows(0, T)
        self._scatter(self.codes, rows, codes)
        self._scatter(self.residual, rows, res)
        self._append_v(v, T)
        self.seq_len = T

    # ---- decode-time append ----------------------------------------------------------------------------
    def append(self, k_new: torch.Tensor, v_new: torch.Tensor) -> None:
        """Add ``k_new, v_new [B, T_new, HKV, 128]`` (post-RoPE keys) after the cached tokens."""
        T_new = self._check(k_new, v_new)
        k_new = k_new.to(self.dtype).contiguous()
        if self.kind in ("q2", "nf4") and self.scale is None:
            raise RuntimeError(f"{self.kind} scales come from the prompt: call prefill first")
        if self.kind == "nvfp4":
            self._append_nvfp4(k_new, T_new)
        else:
            Q.quantize_append(self.kind, k_new, self.codes, self.residual, self.block_table, self.seq_len,
                              fp8_dtype=self.fp8_dtype, scale=self.scale, zero=self.zero, running_minmax=self.minmax)
        self._append_v(v_new, T_new)
        self.seq_len += T_new

    def _append_nvfp4(self, k_new: torch.Tensor, T_new: int) -> None:
        done = 0
        while done < T_new:
            pos = self.seq_len + done
            page, off = divmod(pos, PAGE)
            n = min(PAGE - off, T_new - done)
            self.open_page[:, off:off + n] = k_new[:, done:done + n]
            filled = off + n
            codes, sc, res = Q.encode_k_nvfp4_fp8_residual(self.open_page[:, :filled].contiguous(), self.fp8_dtype, PAGE)
            rows = self._rows(page * PAGE, filled)
            self._scatter(self.codes, rows, codes)
            self._scatter(self.residual, rows, res)
            self.scale[:, page] = sc[:, 0]
            done += n

    def drift(self) -> float:
        """How far the running per-channel range has moved past the range the frozen scales were made
        from: the largest ratio over channels (1.0 = still inside; q2 and nf4 only)."""
        if self.minmax is None:
            return 1.0
        n = self.batch * self.num_kv_heads * 128
        u = self.minmax[:8 * n].view(torch.int32).view(self.batch, self.num_kv_heads, 128, 2).long() & 0xffffffff
        # ordered-integer decoding: values with the top bit set were non-negative floats
        bits = torch.where(u >= 0x80000000, u - 0x80000000, (~u) & 0xffffffff).to(torch.int32)
        lo, hi = bits[..., 0].contiguous().view(torch.float32), bits[..., 1].contiguous().view(torch.float32)
        if self.kind == "q2":
            frozen = (self.scale.float() * 3.0).clamp_min(1e-30)
            return float(((hi - lo) / frozen).max())
        return float((hi / self.scale.float().clamp_min(1e-30)).max())

    # ---- decode ------------------------------------------------------------------------------------
    def decode(self, q: torch.Tensor, **kwargs) -> torch.Tensor:
        if self.seq_len == 0:
            raise RuntimeError("the cache is empty")
        kwargs.setdefault("BS", PAGE)
        kwargs.setdefault("SBS", PAGE)
        if self.kind == "nvfp4" and kwargs["BS"] != PAGE:
            raise ValueError("the streaming nvfp4 cache keeps one scale per 64-token page: BS must be 64")
        if self._workspace is None:
            self._workspace = allocate_decode_workspace(q, self.value, BS=kwargs["BS"], SBS=kwargs["SBS"],
                                                        seq_len=self.max_seq_len)
        scale = self.scale
        if self.kind == "nvfp4":
            scale = self.scale[:, :-(-self.seq_len // PAGE)].contiguous()
        return decode_call(self.kind, q, self.codes, self.value, k_scale=scale, k_zero=self.zero,
                           k_residual=self.residual, block_table=self.block_table, seq_len=self.seq_len,
                           workspace=self._workspace, **kwargs)

    def get_seq_length(self) -> int:
        return self.seq_len
