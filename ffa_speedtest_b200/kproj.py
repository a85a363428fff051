"""Host side of the fused K-projection + RoPE + quantise call.

Mirrors ``kproj_rope_quantize_{reference,triton,fused}`` and the fp4 / nf4 / nvfp4 siblings of the
reference (ffa-q2fp8/fused_kproj_rope_q2fp8.py:402-566 etc.): same arguments and return tuples.
The ``fused`` / ``triton`` names run one tcgen05 GEMM whose epilogue adds the bias, rounds to the
activation dtype and applies RoPE, followed by the variant's CUDA quantiser; ``reference`` keeps the
reference's own recipe (F.linear, eager RoPE) in front of the same quantiser, as a cross-check.

Additions (keyword-only): ``block_table`` + ``out`` scatter the codes straight into a paged cache;
``return_k=True`` appends the post-RoPE K to the returned tuple.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib, quantize as Q

PAGE = 64


def build_rope_cache(seq_len: int, head_dim: int, base: float = 10000.0, device=None,
                     dtype: torch.dtype = torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos / sin tables ``[seq_len, head_dim]``; entry i uses angle index ``i mod head_dim/2``
    (ffa-q2fp8/fused_kproj_rope_q2fp8.py:10-23)."""
    if head_dim % 2 != 0:
        raise ValueError(f"head_dim must be even for RoPE, got {head_dim}")
    expo = torch.arange(0, head_dim, 2, device=device, dtype=dtype) / head_dim
    inv_freq = 1.0 / (base ** expo)
    angles = torch.einsum("i,j->ij", torch.arange(seq_len, device=device, dtype=dtype), inv_freq)
    angles = torch.cat([angles, angles], dim=-1)
    return angles.cos(), angles.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """(x0, x1, x2, x3, ...) -> (-x1, x0, -x3, x2, ...)  (reference :26-30)."""
    return torch.stack((-x[..., 1::2], x[..., ::2]), dim=-1).flatten(-2)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    if cos.ndim == 2:
        cos, sin = cos[None, :, None, :], sin[None, :, None, :]
    return (x * cos) + (rotate_half(x) * sin)


def _normalize_k_weight(w_k: torch.Tensor, in_dim: int) -> torch.Tensor:
    """Return the weight as [out, in] (reference :71-78)."""
    if w_k.ndim != 2:
        raise ValueError(f"w_k must be 2D, got {w_k.shape}")
    if w_k.shape[1] == in_dim:
        return w_k
    if w_k.shape[0] == in_dim:
        return w_k.t().contiguous()
    raise ValueError(f"w_k shape {w_k.shape} is incompatible with in_dim={in_dim}")


def _resolve_fp8_dtype(device) -> torch.dtype:
    return torch.float8_e5m2


_QUANT = {
    "q2": lambda k, f8, page: Q.quantize_k_2bit_fp8_residual(k, f8),
    "fp8": lambda k, f8, page: Q.quantize_k_fp8_fp8_residual(k, f8),
    "fp4": lambda k, f8, page: Q.encode_k_fp4_fp8_residual(k, f8),
    "nf4": lambda k, f8, page: Q.encode_k_nf4_fp8_residual(k, f8),
    "nvfp4": lambda k, f8, page: Q.encode_k_nvfp4_fp8_residual(k, f8, page),
}


def kproj_reference(variant, h, w_k, cos, sin, num_kv_heads, head_dim, bias=None, fp8_dtype=None, page_size=PAGE):
    """The reference recipe on the GPU: F.linear -> eager RoPE -> quantiser."""
    if fp8_dtype is None:
        fp8_dtype = _resolve_fp8_dtype(h.device)
    w_k = _normalize_k_weight(w_k, h.shape[-1])
    lin = F.linear(h, w_k, bias)
    B, T, O = lin.shape
    if O != num_kv_heads * head_dim:
        raise ValueError(f"projection out_dim must be num_kv_heads*head_dim, got {O} vs {num_kv_heads}*{head_dim}")
    k = apply_rope(lin.view(B, T, num_kv_heads, head_dim), cos, sin)
    return _QUANT[variant](k.contiguous(), fp8_dtype, page_size)


_WORKSPACES: dict = {}


def _workspace(nbytes: int, device: torch.device) -> torch.Tensor:
    """Scratch of the fused call (post-RoPE K for the two-pass formats, split-K partials, status word in
    the last 256 bytes).  Few-token calls - a decode loop makes one per layer and token - keep theirs per
    (device, stream, size): an allocation plus a memset per call cost as much as the kernel itself, calls
    on one stream run in order, and the status word is only ever written by a kernel whose bounded wait
    gave up.  Larger (prompt-sized) workspaces are made per call."""
    if nbytes > (8 << 20):
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        ws[-256:].zero_()
        return ws
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream, nbytes)
    ws = _WORKSPACES.get(key)
    if ws is None:
        if len(_WORKSPACES) >= 64:
            _WORKSPACES.clear()
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        ws[-256:].zero_()
        _WORKSPACES[key] = ws
    return ws


def kproj_fused(variant: Optional[str], h, w_k, cos, sin, num_kv_heads, head_dim, bias=None, fp8_dtype=None,
                page_size: int = PAGE, *, block_table: Optional[torch.Tensor] = None, out=None,
                return_k: bool = False, position: int = 0):
    """tcgen05 GEMM + bias + RoPE epilogue, then the variant's quantiser (``variant=None``: K only).

    With ``block_table`` the codes and residual go straight into the pools ``out=(codes, residual)``;
    ``position`` is where token 0 of ``h`` sits in its sequence, so new tokens can be appended to a
    cache (fp8fp8 and fp4 only: the other formats take scales from the whole sequence or page)."""
    if not h.is_cuda:
        raise ValueError("h must be a CUDA tensor (this build has no CPU path)")
    if h.dim() != 3:
        raise ValueError(f"h must be [B, T, H], got {tuple(h.shape)}")
    if h.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError(f"h must be float16 or bfloat16, got {h.dtype}")
    if head_dim != 128:
        raise ValueError(f"this build supports head_dim 128, got {head_dim}")
    if fp8_dtype is None:
        fp8_dtype = _resolve_fp8_dtype(h.device)
    B, T, H = h.shape
    if H % 64 != 0:
        raise ValueError(f"hidden size must be a multiple of 64, got {H}")
    w_k = _normalize_k_weight(w_k, H).to(h.dtype).contiguous()
    if w_k.shape[0] != num_kv_heads * head_dim:
        raise ValueError(
            f"projection out_dim must be num_kv_heads*head_dim, got {w_k.shape[0]} vs {num_kv_heads}*{head_dim}")
    if cos.shape != (T, head_dim) or sin.shape != (T, head_dim):
        raise ValueError(f"cos/sin must be [T, head_dim] = [{T}, {head_dim}], got {tuple(cos.shape)}")
    if cos.dtype != h.dtype:
        cos, sin = cos.float(), sin.float()
    h, cos, sin = h.contiguous(), cos.contiguous(), sin.contiguous()
    if bias is not None:
        bias = bias.to(h.dtype).contiguous()
    k_dtype = torch.float32 if cos.dtype == torch.float32 else h.dtype
    dev = h.device
    HKV = num_kv_heads

    a = _lib.FfaKprojArgs()
    a.variant = -1 if variant is None else _lib.VARIANT_CODE[variant]
    a.B, a.T, a.H, a.HKV, a.head_dim = B, T, H, HKV, head_dim
    a.io_dtype, a.rope_dtype = _lib.float_code(h.dtype), _lib.float_code(cos.dtype)
    a.fp8_format, a.page_size = _lib.fp8_code(fp8_dtype), page_size
    a.h, a.w, a.bias, a.cos, a.sin = h.data_ptr(), w_k.data_ptr(), _lib.ptr(bias), cos.data_ptr(), sin.data_ptr()

    k_rope = torch.empty((B, T, HKV, head_dim), dtype=k_dtype, device=dev) if (return_k or variant is None) else None
    a.k_rope_out = _lib.ptr(k_rope)
    ws = _workspace(_lib.lib().ffa_kproj_workspace_bytes(B, T, HKV, a.rope_dtype), dev)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()

    outs = ()
    if variant is not None:
        if block_table is not None:
            if block_table.dtype != torch.int32 or block_table.dim() != 2 or block_table.shape[0] != B:
                raise ValueError("block_table must be an int32 tensor of shape [B, pages_per_sequence]")
            if position < 0 or block_table.shape[1] * PAGE < position + T:
                raise ValueError("block_table has too few pages for position + T")
            if position and variant not in ("fp8", "fp4"):
                raise ValueError("appending at a position needs an elementwise format (fp8fp8 or fp4)")
            if out is None:
                raise ValueError("with block_table, pass out=(codes_pool, residual_pool) to scatter into")
            codes, res = out
            a.slot_table, a.slot_stride = block_table.data_ptr(), block_table.shape[1]
            a.slot_pos0 = position
        else:
            code_w = {"q2": 32, "fp8": 128}.get(variant, 64)
            codes = torch.empty((B, T, HKV, code_w), dtype=fp8_dtype if variant == "fp8" else torch.uint8, device=dev)
            res = torch.empty((B, T, HKV, head_dim), dtype=fp8_dtype, device=dev)
        scale = zero = None
        if variant in ("q2", "nf4"):
            scale = torch.empty((B, HKV, head_dim), dtype=k_dtype, device=dev)
        if variant == "q2":
            zero = torch.empty_like(scale)
        if variant == "nvfp4":
            scale = torch.empty((B, -(-T // page_size), HKV), dtype=k_dtype, device=dev)
        a.codes, a.residual, a.scale, a.zero = codes.data_ptr(), res.data_ptr(), _lib.ptr(scale), _lib.ptr(zero)
        outs = {"q2": (codes, scale, zero, res), "fp8": (codes, res), "fp4": (codes, res), "nf4": (codes, scale, res),
                "nvfp4": (codes, scale, res)}[variant]

    _lib.check(_lib.lib().ffa_kproj_rope(a, _lib.current_stream(dev)), "ffa_kproj_rope")
    kproj_fused.last_workspace = ws     # lets tests read the status word
    if return_k or variant is None:
        return (*outs, k_rope)
    return outs
