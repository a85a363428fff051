"""A Llama-style decoder whose attention routes single-token steps to the pruned decode op.

The model-side half of the reference's end-to-end integration (ffa-fp8fp8/e2e/modeling_llama.py):
there a copy of the Hugging Face Llama model gets one change, in ``LlamaAttention.forward``
(:229-340) - with ``config.attn_settings["use_ffa_decode"]`` set and ``q_len == 1`` the layer calls
``attn_forward_decode_fp8fp8`` on the fp8 base / residual keys held by the ``FP8Fp8Cache``, otherwise
flash attention.  This file keeps that contract (``attn_settings`` keys ``use_ffa_decode``, ``BS``,
``SBS``, ``delta``, ``use_fp8_residual``, ``pattern_layers``; a cache object passed as
``past_key_values``; ``model(input_ids, past_key_values=cache, use_cache=True)``) on a compact
decoder written for this package: RMSNorm, rotary attention with grouped kv-heads, SwiGLU MLP,
random-initialised weights - what the tok/s driver needs around the hot path, not a model zoo.

What differs from the reference on purpose:
  * the cache is the paged ``PagedFP8Fp8Cache``; a decode step appends the new token with one fused
    kernel (K projection + RoPE + fp8 quantisation + scatter into the page, from the hidden state)
    and one copy kernel for V, then runs the decode op on the pools - no ``torch.cat``, no
    dequantised shadow copy of the keys;
  * RoPE pairs neighbouring channels (2i, 2i+1), the convention of the reference's fused K-projection
    (ffa-fp8fp8/fused_kproj_rope_fp8fp8.py:26-37), for q and k alike;
  * dense attention (prefill, and the baseline arm) is torch's scaled_dot_product_attention.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...kproj import apply_rope, build_rope_cache
from .fp8fp8_cache import PagedFP8Fp8Cache


@dataclass
class LlamaConfig:
    hidden_size: int = 4096
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    num_hidden_layers: int = 1
    intermediate_size: int = 0                 # 0: 4 x hidden
    max_position_embeddings: int = 4096
    vocab_size: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 500000.0
    attention_bias: bool = False
    mlp_bias: bool = False
    attn_settings: dict = field(default_factory=dict)

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


class DenseCache:
    """Unquantised K/V of every layer in preallocated ``[B, max, HKV, D]`` buffers: the baseline arm."""

    def __init__(self, batch: int, num_kv_heads: int, max_seq_len: int, head_dim: int, dtype, device):
        self._shape = (batch, max_seq_len, num_kv_heads, head_dim)
        self._dtype, self._device = dtype, device
        self.k: list[torch.Tensor] = []
        self.v: list[torch.Tensor] = []
        self.len: list[int] = []

    def update(self, k: torch.Tensor, v: torch.Tensor, layer_idx: int):
        while len(self.k) <= layer_idx:
            self.k.append(torch.empty(self._shape, dtype=self._dtype, device=self._device))
            self.v.append(torch.empty(self._shape, dtype=self._dtype, device=self._device))
            self.len.append(0)
        n, t = self.len[layer_idx], k.shape[1]
        if n + t > self._shape[1]:
            raise ValueError(f"cache capacity {self._shape[1]} exceeded ({n} + {t})")
        self.k[layer_idx][:, n:n + t] = k
        self.v[layer_idx][:, n:n + t] = v
        self.len[layer_idx] = n + t
        return self.k[layer_idx][:, :n + t], self.v[layer_idx][:, :n + t]

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.len[layer_idx] if len(self.len) > layer_idx else 0


class LlamaRMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return self.weight * xf.to(x.dtype)


class LlamaMLP(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        inter = cfg.intermediate_size or 4 * cfg.hidden_size
        self.gate_proj = nn.Linear(cfg.hidden_size, inter, bias=cfg.mlp_bias)
        self.up_proj = nn.Linear(cfg.hidden_size, inter, bias=cfg.mlp_bias)
        self.down_proj = nn.Linear(inter, cfg.hidden_size, bias=cfg.mlp_bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


def _dense_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool) -> torch.Tensor:
    """q ``[B, Tq, HQ, D]``, k / v ``[B, Tk, HKV, D]`` -> ``[B, Tq, HQ, D]``; with ``causal`` the Tq
    queries are the last Tq positions of the Tk keys."""
    B, Tq, HQ, D = q.shape
    Tk = k.shape[1]
    mask = None
    square = causal and Tq > 1 and Tq == Tk
    if causal and Tq > 1 and not square:
        pos_q = torch.arange(Tk - Tq, Tk, device=q.device)[:, None]
        mask = torch.arange(Tk, device=q.device)[None, :] <= pos_q
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask,
                                       is_causal=square, enable_gqa=k.shape[2] != HQ)
    return o.transpose(1, 2)


class LlamaAttention(nn.Module):
    def __init__(self, cfg: LlamaConfig, layer_idx: int):
        super().__init__()
        self.config, self.layer_idx = cfg, layer_idx
        self.head_dim = cfg.head_dim
        self.num_heads, self.num_kv_heads = cfg.num_attention_heads, cfg.num_key_value_heads
        self.q_proj = nn.Linear(cfg.hidden_size, self.num_heads * self.head_dim, bias=cfg.attention_bias)
        self.k_proj = nn.Linear(cfg.hidden_size, self.num_kv_heads * self.head_dim, bias=cfg.attention_bias)
        self.v_proj = nn.Linear(cfg.hidden_size, self.num_kv_heads * self.head_dim, bias=cfg.attention_bias)
        self.o_proj = nn.Linear(self.num_heads * self.head_dim, cfg.hidden_size, bias=cfg.attention_bias)

    def forward(self, hidden_states: torch.Tensor, position_embeddings, past_key_values=None) -> torch.Tensor:
        B, T, _ = hidden_states.shape
        cos, sin = position_embeddings                                   # rows of the new positions, [T, D]
        settings = dict(getattr(self.config, "attn_settings", {}) or {})
        use_ffa_decode = bool(settings.get("use_ffa_decode", False))
        pattern_layers = settings.get("pattern_layers", None)
        in_pattern = pattern_layers is None or self.layer_idx in pattern_layers

        q = apply_rope(self.q_proj(hidden_states).view(B, T, self.num_heads, self.head_dim), cos, sin)
        v = self.v_proj(hidden_states).view(B, T, self.num_kv_heads, self.head_dim)

        if isinstance(past_key_values, PagedFP8Fp8Cache):
            ffa_step = T == 1 and use_ffa_decode and in_pattern
            if ffa_step and settings.get("fused_append", True) and past_key_values.use_fp8_residual:
                # K projection + RoPE + quantisation + scatter in one kernel, straight from the hidden state
                past_key_values.update_from_hidden(hidden_states, self.k_proj.weight, cos, sin, v, self.layer_idx,
                                                   bias=self.k_proj.bias)
                k = None
            else:
                k = apply_rope(self.k_proj(hidden_states).view(B, T, self.num_kv_heads, self.head_dim), cos, sin)
                past_key_values.update(k, v, self.layer_idx)
            if ffa_step:
                kw = {name: settings[name] for name in ("BS", "SBS", "delta", "scale") if settings.get(name) is not None}
                kw["use_fp8_residual"] = settings.get("use_fp8_residual", past_key_values.use_fp8_residual)
                attn = past_key_values.decode(q, self.layer_idx, **kw)            # [B, HQ, D]
                attn = attn.view(B, 1, self.num_heads, self.head_dim)
            elif past_key_values.get_seq_length(self.layer_idx) == T:
                attn = _dense_attention(q, k, v, causal=True)                     # prefill from an empty cache
            else:
                raise RuntimeError("a PagedFP8Fp8Cache serves prefill from empty and single-token FFA decode steps; "
                                   "set attn_settings['use_ffa_decode'] or use a DenseCache for dense decode")
        else:
            k = apply_rope(self.k_proj(hidden_states).view(B, T, self.num_kv_heads, self.head_dim), cos, sin)
            if past_key_values is not None:
                k_all, v_all = past_key_values.update(k, v, self.layer_idx)
            else:
                k_all, v_all = k, v
            attn = _dense_attention(q, k_all, v_all, causal=True)
        return self.o_proj(attn.reshape(B, T, self.num_heads * self.head_dim))


class LlamaDecoderLayer(nn.Module):
    def __init__(self, cfg: LlamaConfig, layer_idx: int):
        super().__init__()
        self.self_attn = LlamaAttention(cfg, layer_idx)
        self.mlp = LlamaMLP(cfg)
        self.input_layernorm = LlamaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.post_attention_layernorm = LlamaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)

    def forward(self, x: torch.Tensor, position_embeddings, past_key_values=None) -> torch.Tensor:
        x = x + self.self_attn(self.input_layernorm(x), position_embeddings, past_key_values)
        return x + self.mlp(self.post_attention_layernorm(x))


class LlamaForCausalLM(nn.Module):
    """``model(input_ids, past_key_values=cache, use_cache=True)`` -> logits ``[B, T, vocab]``; the new
    tokens' positions continue from the cache's length."""

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.config = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList(LlamaDecoderLayer(cfg, i) for i in range(cfg.num_hidden_layers))
        self.norm = LlamaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        self._rope = None
        for prm in self.parameters():                       # small weights keep activations tame at any width
            if prm.dim() > 1:
                nn.init.normal_(prm, std=0.02)

    def _rope_rows(self, start: int, count: int, dtype, device):
        if self._rope is None or self._rope[0].device != device or self._rope[0].dtype != dtype:
            cos, sin = build_rope_cache(self.config.max_position_embeddings, self.config.head_dim,
                                        base=self.config.rope_theta, device=device)
            self._rope = (cos.to(dtype), sin.to(dtype))
        if start + count > self._rope[0].shape[0]:
            raise ValueError(f"position {start + count} exceeds max_position_embeddings {self._rope[0].shape[0]}")
        return self._rope[0][start:start + count], self._rope[1][start:start + count]

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, past_key_values=None, use_cache: bool = False) -> torch.Tensor:
        cache = past_key_values if use_cache else None
        start = cache.get_seq_length(0) if cache is not None else 0
        x = self.embed_tokens(input_ids)
        rope = self._rope_rows(start, input_ids.shape[1], x.dtype, x.device)
        for layer in self.layers:
            x = layer(x, rope, cache)
        return self.lm_head(self.norm(x))
