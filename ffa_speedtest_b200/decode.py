"""Host side of the FFA decode call: the reference's validation, then one C-ABI call.

Mirrors the wrappers ``attn_forward_decode_*`` of the reference
(ffa-q2fp8/attn_kernel/attn_kernel_v1210_fused_bsz_q2fp8.py:191-309 and the fp8fp8 / fp4fp8 /
nf4fp8 / nvfp4fp8 siblings): same positional and keyword arguments, same exceptions for the
same mistakes, same return values.  Additions, all keyword-only and off by default:

* ``block_table`` ``[B, pages] int32`` (+ ``seq_len``): K/V tensors are then paged pools
  ``[n_pages, 64, HKV, D]``; ``None`` keeps the reference layout ``[B, T, HKV, D]``.
* ``workspace``: a :class:`DecodeWorkspace` to reuse scratch and output across calls.
* ``out``: preallocated output ``[B, HQ, V]``.
* ``partial_out``: ``[B, HQ, 129]`` fp32 buffer receiving (normalised output, base-2 LSE) for
  merging across sequence shards.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import _lib

PAGE = 64


MAX_SBS = 512      # largest prune granularity of this build (eight 64-token pages)


class DecodeWorkspace:
    """Reusable output, mask, threshold and scratch buffers of the decode call.

    Same constructor, attributes ``o`` / ``mask_buf`` / ``threshold_buf`` and ``matches`` as
    ``Q2FP8DecodeWorkspace`` of the reference
    (ffa-q2fp8-h100/attn_kernel/attn_kernel_v1210_fused_bsz_q2fp8.py:232-258), for all five
    variants.  The reference's ``m_buf`` / ``l_buf`` / ``o_buf`` (one partial per block) have no
    counterpart: partial results live in ``scratch``, one per page range of a CTA.

    ``NTBS`` is the number of prune blocks per sequence, ``ceil(T/BS) * (BS/SBS)``.  The scratch is
    sized for the longest sequence that many blocks can hold, so one workspace serves a cache
    that grows up to ``NTBS`` blocks (``fits``)."""

    def __init__(self, B: int, HQ: int, HKV: int, V: int, NTBS: int, device, dtype, *, pages_per_chunk: int = 0):
        self.B, self.HQ, self.HKV, self.V, self.NTBS = int(B), int(HQ), int(HKV), int(V), int(NTBS)
        self.device = torch.device(device)
        self.dtype = dtype
        self.pages_per_chunk = int(pages_per_chunk)
        nbytes = _lib.lib().ffa_decode_workspace_bytes(self.B, self.NTBS * MAX_SBS, self.HQ, self.HKV,
                                                       self.pages_per_chunk)
        self.scratch = torch.empty(max(nbytes, 65536), dtype=torch.uint8, device=self.device)
        self.scratch[:65536].zero_()     # arrival counters + status word: zero before first use
        self.o = torch.empty((self.B, self.HQ, self.V), dtype=dtype, device=self.device)
        self.mask_buf = torch.empty((self.B, self.HKV, self.NTBS), dtype=torch.int8, device=self.device)
        self.threshold_buf = torch.empty((self.B, self.HQ), dtype=torch.float32, device=self.device)

    @classmethod
    def for_shape(cls, B: int, T: int, HQ: int, HKV: int, V: int, *, BS: int, SBS: int, device, dtype,
                  pages_per_chunk: int = 0) -> "DecodeWorkspace":
        """Workspace for sequences of up to T tokens pruned in SBS-token blocks of BS-token blocks."""
        return cls(B, HQ, HKV, V, -(-T // BS) * (BS // SBS), device, dtype, pages_per_chunk=pages_per_chunk)

    # the names used before the reference's were adopted
    @property
    def mask(self) -> torch.Tensor:
        return self.mask_buf

    @property
    def threshold(self) -> torch.Tensor:
        return self.threshold_buf

    def matches(self, B: int, HQ: int, HKV: int, V: int, NTBS: int, device, dtype) -> bool:
        """Exactly the shape, device and dtype the workspace was made for (reference :248-258)."""
        return (self.B == int(B) and self.HQ == int(HQ) and self.HKV == int(HKV) and self.V == int(V)
                and self.NTBS == int(NTBS) and self.device == torch.device(device) and self.dtype == dtype)

    def fits(self, B: int, HQ: int, HKV: int, V: int, NTBS: int, device, dtype, pages_per_chunk: int = 0) -> bool:
        """True for the shape the workspace was made for and for shorter sequences of the same batch
        (a cache that grows towards the allocated length)."""
        return (self.matches(B, HQ, HKV, V, self.NTBS, device, dtype) and int(NTBS) <= self.NTBS
                and int(pages_per_chunk) == self.pages_per_chunk)

    def mask_view(self, B: int, HKV: int, ntbs: int) -> torch.Tensor:
        """The kept-page mask of a call over ``ntbs`` blocks per sequence (the buffer is sized for the
        longest sequence; a call writes the first B*HKV*ntbs entries)."""
        return self.mask_buf.view(-1)[:B * HKV * ntbs].view(B, HKV, ntbs)

    def status(self) -> int:
        """Device status word (synchronises): 0 = ok, 1 = a bounded wait inside a kernel gave up (the
        affected outputs are NaN)."""
        return int(self.scratch[65280:65284].view(torch.int32).item())


def allocate_decode_workspace(q, *kv, BS: int = 128, SBS: Optional[int] = None, seq_len: Optional[int] = None,
                              pages_per_chunk: int = 0) -> DecodeWorkspace:
    """``allocate_q2fp8_decode_workspace(q, k_q, v, BS=128, SBS=None)`` of the reference
    (ffa-q2fp8-h100/attn_kernel/attn_kernel_v1210_fused_bsz_q2fp8.py:261-277), for every variant.
    ``(q, v)`` without the K tensor is accepted too; BS and SBS may also be given positionally after
    the tensors as in the reference.  ``seq_len`` sizes a workspace for paged pools
    ``[n_pages, 64, HKV, D]``, whose second dimension is the page size and not the sequence length."""
    tensors = [t for t in kv if isinstance(t, torch.Tensor)]
    rest = [t for t in kv if not isinstance(t, torch.Tensor)]
    if len(tensors) not in (1, 2) or len(rest) > 2:
        raise TypeError("allocate_decode_workspace(q, [k,] v, BS=128, SBS=None)")
    if len(rest) >= 1:
        BS = rest[0]
    if len(rest) == 2:
        SBS = rest[1]
    v = tensors[-1]
    B, Tq, HQ, _ = q.shape
    Bv, Tv, HKV, V = v.shape
    if seq_len is None:
        if len(tensors) == 2:
            Bk, Tk, HKVk, _ = tensors[0].shape
            if B != Bk or Tk != Tv or HKVk != HKV:
                raise ValueError("K/V layouts must be [B, T, HKV, D]")
        if B != Bv or Tq != 1:
            raise ValueError("K/V layouts must be [B, T, HKV, D]")
    T = seq_len if seq_len is not None else Tv
    if SBS is None:
        SBS = BS
    return DecodeWorkspace.for_shape(B, T, HQ, HKV, V, BS=BS, SBS=SBS, device=q.device, dtype=q.dtype,
                                     pages_per_chunk=pages_per_chunk)


def _fp8_format(*tensors) -> int:
    """fp8 encoding shared by the fp8 tensors of a call (e5m2 if there is none)."""
    fmt = None
    for t in tensors:
        if t is None:
            continue
        if t.dtype not in (torch.float8_e5m2, torch.float8_e4m3fn):
            raise ValueError(
                f"this build reads fp8 (float8_e5m2 / float8_e4m3fn) K base tensors, got {t.dtype}")
        code = _lib.fp8_code(t.dtype)
        if fmt is not None and fmt != code:
            raise ValueError("fp8 K base and residual must use the same fp8 encoding")
        fmt = code
    return _lib.E5M2 if fmt is None else fmt


def _residual_as_fp8(k_residual: torch.Tensor, like: Optional[torch.dtype]) -> torch.Tensor:
    """The kernels read the residual as fp8.  The reference also takes float16 / bfloat16 / float32
    residuals (its kernel casts whatever it gets to float16, ...q2fp8.py:110-114; its quantisers fall back
    to float16 on a torch without fp8 types, fused_kproj_rope_q2fp8.py:81-88): those are rounded to fp8
    here, to the encoding of the fp8 base when there is one and to e5m2 (float16's exponent range)
    otherwise - a conversion pass per call, meant for compatibility and not for speed."""
    if k_residual.dtype in (torch.float8_e5m2, torch.float8_e4m3fn):
        return k_residual
    if k_residual.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise ValueError(f"k_residual must be fp8, float16, bfloat16 or float32, got {k_residual.dtype}")
    return k_residual.to(like if like is not None else torch.float8_e5m2)


def decode_call(
    variant: str,
    q: torch.Tensor,
    k_codes: torch.Tensor,
    v: torch.Tensor,
    *,
    k_scale: Optional[torch.Tensor] = None,
    k_zero: Optional[torch.Tensor] = None,
    k_residual: Optional[torch.Tensor] = None,
    scale: Optional[float] = None,
    BS: int = 128,
    SBS: Optional[int] = None,
    delta: float = 5.0,
    return_skip_ratio: bool = False,
    precomputed_threshold: Optional[torch.Tensor] = None,
    use_fp8_residual: bool = True,
    block_table: Optional[torch.Tensor] = None,
    seq_len: Optional[int] = None,
    workspace: Optional[DecodeWorkspace] = None,
    out: Optional[torch.Tensor] = None,
    partial_out: Optional[torch.Tensor] = None,
    pages_per_chunk: int = 0,
    kernel: str = "auto",
    mean_v: Optional[torch.Tensor] = None,
    peer=None,
):
    """Shape bookkeeping shared by the five entry points; tensors are already type-checked.

    ``mean_v [B, HKV, 128]`` (V's dtype) selects the mean-V variant of the 2-bit format: pruned pages
    are not dropped but contribute their coarse softmax mass times this vector.

    ``kernel``: "ws" is the warp-specialised TMA kernel (any q dtype, either V dtype, prune groups of
    up to eight pages); "pipe" the page-pipeline TMA kernel (bfloat16 q, or float16 q with float16 V;
    pages pruned one by one); "auto" takes "pipe" for fp8 coarse K below about a million cached tokens
    where it applies (it is the faster of the two there) and "ws" otherwise; "fp16" forces the fp16
    tensor-core kernel, which follows the reference's fp16 rounding of the refined K tile to the
    letter and prunes page by page only."""
    if kernel not in ("auto", "fp16", "pipe", "ws"):
        raise ValueError(f"kernel must be 'auto', 'ws', 'pipe' or 'fp16', got {kernel!r}")
    B, Tq, HQ, K = q.shape
    HKV, V = v.shape[2], v.shape[3]
    if block_table is None:
        T = v.shape[1]
    else:
        if block_table.dtype != torch.int32 or block_table.dim() != 2 or block_table.shape[0] != B:
            raise ValueError("block_table must be an int32 tensor of shape [B, pages_per_sequence]")
        if v.shape[1] != PAGE or k_codes.shape[1] != PAGE:
            raise ValueError("with block_table, K/V tensors are paged pools [n_pages, 64, HKV, D]")
        T = seq_len if seq_len is not None else block_table.shape[1] * PAGE
        if block_table.shape[1] * PAGE < T:
            raise ValueError("block_table has too few pages for seq_len")
        assert block_table.is_cuda and block_table.is_contiguous()
    if HQ % HKV != 0:
        raise ValueError(f"HQ ({HQ}) must be divisible by HKV ({HKV}) for GQA")
    G = HQ // HKV
    if K != 128 or V != 128:
        raise ValueError(f"this build supports head_dim 128 for K and V, got K={K}, V={V}")
    if G > 8:
        raise ValueError(f"this build supports GQA group sizes up to 8, got {G}")
    if scale is None:
        scale = 1.0 / math.sqrt(K)
    if SBS is None:
        SBS = BS
    if SBS in (16, 32):
        # prune blocks of a quarter / half of a page: BS stays in whole pages
        if BS % PAGE != 0:
            raise ValueError(f"with SBS below 64, BS must be a multiple of 64 (got BS={BS}, SBS={SBS})")
        if kernel not in ("auto", "ws"):
            raise ValueError("SBS below 64 needs kernel='auto' or 'ws': the other kernels prune page by page only")
        if mean_v is not None:
            raise ValueError("the mean-V variant prunes whole pages: SBS must be at least 64")
    else:
        if SBS % PAGE != 0 or SBS < PAGE or BS % SBS != 0:
            raise ValueError(f"SBS must be 16, 32 or a multiple of 64, and BS a multiple of SBS and of 64 "
                             f"(got BS={BS}, SBS={SBS})")
        if SBS > MAX_SBS or (SBS // PAGE) & (SBS // PAGE - 1):
            raise ValueError(f"this build prunes groups of 1, 2, 4 or 8 pages: SBS must be 64, 128, 256 or 512 (got {SBS})")
        if SBS != PAGE and kernel not in ("auto", "ws"):
            raise ValueError("SBS above 64 needs kernel='auto' or 'ws': the other kernels prune page by page only")
    NTB = -(-T // BS)
    NTBS = NTB * (BS // SBS)

    use_res = bool(use_fp8_residual and k_residual is not None)
    if use_res:
        k_residual = _residual_as_fp8(k_residual, k_codes.dtype if variant == "fp8" else None)
    fp8_fmt = _fp8_format(k_codes if variant == "fp8" else None, k_residual if use_res else None)

    if precomputed_threshold is not None:
        assert precomputed_threshold.is_cuda and precomputed_threshold.shape == (B, HQ)
        th_in = precomputed_threshold.contiguous()
        if th_in.dtype != torch.float32:
            th_in = th_in.float()
    else:
        th_in = None

    if workspace is None:
        workspace = DecodeWorkspace(B, HQ, HKV, V, NTBS, q.device, q.dtype, pages_per_chunk=pages_per_chunk)
    elif not isinstance(workspace, DecodeWorkspace):
        raise TypeError("workspace must be a Q2FP8DecodeWorkspace")
    elif not workspace.fits(B, HQ, HKV, V, NTBS, q.device, q.dtype, pages_per_chunk):
        raise ValueError("workspace shape/device/dtype mismatch")
    o = workspace.o if out is None else out
    if o.shape != (B, HQ, V) or o.dtype != q.dtype or not o.is_contiguous():
        raise ValueError("out must be a contiguous [B, HQ, V] tensor of q's dtype")
    if partial_out is not None:
        if partial_out.shape != (B, HQ, V + 1) or partial_out.dtype != torch.float32 or not partial_out.is_contiguous():
            raise ValueError("partial_out must be a contiguous fp32 [B, HQ, 129] tensor")

    a = _lib.FfaDecodeArgs()
    a.variant = _lib.VARIANT_CODE[variant]
    a.B, a.T, a.HQ, a.HKV, a.head_dim = B, T, HQ, HKV, K
    a.BS, a.SBS = BS, SBS
    a.sm_scale, a.delta = float(scale), float(delta)
    a.q_dtype = _lib.float_code(q.dtype)
    a.v_dtype = _lib.float_code(v.dtype)
    if a.v_dtype == _lib.F32:
        raise ValueError("v must be float16 or bfloat16")
    a.scale_dtype = _lib.float_code(k_scale.dtype) if k_scale is not None else _lib.F32
    a.fp8_format = fp8_fmt
    a.use_residual = int(use_res)
    a.q, a.k_codes, a.v = q.data_ptr(), k_codes.data_ptr(), v.data_ptr()
    a.k_scale, a.k_zero = _lib.ptr(k_scale), _lib.ptr(k_zero)
    a.k_residual = k_residual.data_ptr() if use_res else None
    a.block_table = _lib.ptr(block_table)
    a.bt_stride = block_table.shape[1] if block_table is not None else 0
    a.threshold_in = _lib.ptr(th_in)
    a.out = o.data_ptr()
    a.kept_mask = workspace.mask.data_ptr()
    a.threshold_out = workspace.threshold.data_ptr()
    a.partial_out = _lib.ptr(partial_out)
    if mean_v is not None:
        if variant != "q2":
            raise ValueError("the mean-V variant exists for the 2-bit format only")
        if mean_v.shape != (B, HKV, V) or mean_v.dtype != v.dtype or not mean_v.is_cuda:
            raise ValueError(f"mean_v must be a CUDA tensor [B, HKV, V] = [{B}, {HKV}, {V}] of v's dtype")
        if partial_out is not None or kernel == "fp16":
            raise ValueError("the mean-V variant has no partial output and runs on the TMA kernels only")
        mean_v = mean_v.contiguous()
    a.v_mean = _lib.ptr(mean_v)
    a.workspace = workspace.scratch.data_ptr()
    a.workspace_bytes = workspace.scratch.numel()
    a.pages_per_chunk = pages_per_chunk
    a.reserved = {"auto": 0, "fp16": 1, "pipe": 2, "ws": 4}[kernel]
    a.kv_rows = k_codes.shape[0] * k_codes.shape[1]
    if peer is not None:
        # sequence split over peer memory (sharded.PeerShardedDecode): the kernel's merge also stores every
        # partial row into this rank's slot on the peers and raises the step's flags when it is done
        _lib.check(_lib.lib().ffa_decode_peer(a, peer, _lib.current_stream(q.device)), "ffa_decode_peer")
    else:
        _lib.check(_lib.lib().ffa_decode(a, _lib.current_stream(q.device)), "ffa_decode")

    if return_skip_ratio:
        mask = workspace.mask_view(B, HKV, NTBS)
        kept = mask.to(torch.int32).sum()
        total = mask.numel()
        skip_ratio = float((1.0 - (kept.float() / float(total))).item())
        return o, skip_ratio
    return o


def check_common(q, k_codes, v, k_residual, what: str):
    """The checks every reference wrapper makes before launching (…q2fp8.py:211-262)."""
    assert q.is_cuda and k_codes.is_cuda and v.is_cuda
    if k_residual is not None and not k_residual.is_cuda:
        raise ValueError("k_residual must be a CUDA tensor when provided")
    if k_residual is not None and not k_residual.is_floating_point():
        raise ValueError("k_residual must be a floating point tensor (e.g., fp8/fp16/bf16)")
    if q.dim() != 4 or k_codes.dim() != 4 or v.dim() != 4:
        raise ValueError(f"{what}: q, K and v must be 4-D tensors")
    assert q.is_contiguous() and k_codes.is_contiguous() and v.is_contiguous()
    if k_residual is not None:
        assert k_residual.is_contiguous()


def check_layout(q, k_codes, v, k_residual, k_last: int, paged: bool):
    B, Tq, HQ, K = q.shape
    Bk, T, HKV, Kk = k_codes.shape
    Bv, Tv, HKVv, V = v.shape
    ok = Tq == 1 and Tv == T and HKVv == HKV and Kk == k_last and (paged or B == Bk == Bv) and Bk == Bv
    if k_residual is not None:
        Br, Tr, HKVr, Kr = k_residual.shape
        ok = ok and Br == Bk and Tr == T and HKVr == HKV and Kr == K
    assert ok, "K/V layouts must be [B, T, HKV, D]"
