"""CPU restatement of the FFA quantised, pruned decode-attention path.

TEST INFRASTRUCTURE ONLY.  This module is the checker for the CUDA kernels in
``ffa_speedtest_b200/csrc``; nothing in the product imports it.  It is used by
``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline legs of
``bench.py``.

Parity status: PINNED.  Every function below is checked against outputs of the
reference's own code (its torch quantisers, and its Triton stage-1/stage-2
kernels executed by the Triton interpreter on CPU tensors) on seeded inputs;
those outputs are committed under ``tests/golden/`` together with the script
that produced them (``tests/golden/make_golden.py``).  The reference holds no
golden vectors or known-answer tests of its own for this path.  On a GPU the
reference's unmodified Triton kernels, compiled by Triton's JIT, are a second
check of the CUDA kernels (``tests/test_reference_jit_gpu.py``).

All arithmetic follows the reference's sequence of roundings (reference paths
are relative to the root of qluoluo/ffa-speedtest):

* decode stage 1  : ffa-q2fp8/attn_kernel/attn_kernel_v1210_fused_bsz_q2fp8.py:30-139
  (fp8fp8 :42-136, fp4fp8 :45-147, nf4fp8 :60-167, nvfp4fp8 :60-169 of the
  sibling files; they differ only in how the coarse K tile is produced)
* decode stage 2  : same file :142-171
* quantisers      : ffa-q2fp8/fused_kproj_rope_q2fp8.py:40-68,
                    ffa-fp8fp8/fused_kproj_rope_fp8fp8.py:58-64,
                    ffa-fp4fp8/fused_kproj_rope_fp4fp8.py:40-73,
                    ffa-nf4fp8/fused_kproj_rope_nf4fp8.py:72-96,
                    ffa-nvfp4fp8/fused_kproj_rope_nvfp4fp8.py:62-114
* RoPE + K-proj   : ffa-q2fp8/fused_kproj_rope_q2fp8.py:10-37, 402-424
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch
import torch.nn.functional as F

LOG2E = 1.4426950408889634
THRESHOLD_SAMPLE = 16  # T_BS in the reference kernels

# e2m1 magnitudes indexed by the low three bits of a nibble (bit 3 is the sign).
E2M1_LEVELS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
E2M1_CUTS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)

# NormalFloat-4 code book (QLoRA), as used by ffa-nf4fp8/attn_kernel/...nf4fp8.py:10-27.
NF4_LEVELS = (
    -1.0, -0.6961928009986877, -0.5229921340942383, -0.39491748809814453,
    -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
    0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
    0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0,
)


# --------------------------------------------------------------------------------------
# bit packing helpers
# --------------------------------------------------------------------------------------
def pack_codes(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """Pack the last dim of a uint8 code tensor, first code in the low bits."""
    per = 8 // bits
    *lead, n = codes.shape
    n_bytes = (n + per - 1) // per
    if n_bytes * per != n:
        codes = F.pad(codes, (0, n_bytes * per - n))
    lanes = codes.reshape(*lead, n_bytes, per).to(torch.int32)
    out = torch.zeros(*lead, n_bytes, dtype=torch.int32)
    for i in range(per):
        out |= lanes[..., i] << (bits * i)
    return out.to(torch.uint8).contiguous()


def unpack_codes(packed: torch.Tensor, bits: int, n: int) -> torch.Tensor:
    per = 8 // bits
    shifts = torch.arange(per, dtype=torch.int32) * bits
    wide = (packed.to(torch.int32)[..., None] >> shifts) & ((1 << bits) - 1)
    return wide.reshape(*packed.shape[:-1], -1)[..., :n].to(torch.uint8)


# --------------------------------------------------------------------------------------
# quantisers (K [B, T, HKV, D] in the model dtype -> codes, scales, fp8 residual)
# --------------------------------------------------------------------------------------
def quantize_q2(k: torch.Tensor, fp8_dtype: torch.dtype):
    """2-bit asymmetric, one (scale, zero) per (b, kv-head, channel) over all tokens.

    Follows ffa-q2fp8/fused_kproj_rope_q2fp8.py:44-52: min/max, scale and the code
    are evaluated in K's own dtype (one rounding per torch op); dequantisation and the
    residual are evaluated in fp32.
    """
    lo = k.amin(dim=1)
    hi = k.amax(dim=1)
    step = ((hi - lo).clamp_min(1e-6) / 3.0).contiguous()
    zero = lo.contiguous()
    level = torch.round((k - zero.unsqueeze(1)) / step.unsqueeze(1)).clamp(0, 3).to(torch.uint8)
    recon = level.to(torch.float32) * step.unsqueeze(1).to(torch.float32) + zero.unsqueeze(1).to(torch.float32)
    resid = (k.to(torch.float32) - recon).to(fp8_dtype).contiguous()
    return pack_codes(level, 2), step, zero, resid


def quantize_fp8fp8(k: torch.Tensor, fp8_dtype: torch.dtype):
    """fp8 base = cast of K, fp8 residual = cast of the fp32 difference
    (ffa-fp8fp8/fused_kproj_rope_fp8fp8.py:58-64)."""
    base = k.to(fp8_dtype).contiguous()
    resid = (k.to(torch.float32) - base.to(torch.float32)).to(fp8_dtype).contiguous()
    return base, resid


def _e2m1_encode(x: torch.Tensor):
    """Nearest e2m1 magnitude by the seven cut points (ties go up), sign from ``x < 0``.
    The comparison is made in x's dtype (ffa-fp4fp8/fused_kproj_rope_fp4fp8.py:45-61)."""
    cuts = torch.tensor(E2M1_CUTS, dtype=x.dtype)
    levels = torch.tensor(E2M1_LEVELS, dtype=x.dtype)
    mag = torch.bucketize(x.abs(), cuts, right=True)
    neg = x < 0
    nib = mag.to(torch.uint8) | (neg.to(torch.uint8) << 3)
    val = levels[mag]
    val = torch.where(neg, -val, val)
    return nib, val


def quantize_fp4(k: torch.Tensor, fp8_dtype: torch.dtype):
    """Unscaled e2m1 nibbles; the residual is formed in K's dtype and then cast
    (ffa-fp4fp8/fused_kproj_rope_fp4fp8.py:40-73)."""
    nib, val = _e2m1_encode(k)
    resid = (k - val).to(fp8_dtype).contiguous()
    return pack_codes(nib, 4), resid


def quantize_nf4(k: torch.Tensor, fp8_dtype: torch.dtype):
    """NF4 code book with an fp32 absmax per (b, kv-head, channel) over all tokens
    (ffa-nf4fp8/fused_kproj_rope_nf4fp8.py:72-96)."""
    book = torch.tensor(NF4_LEVELS, dtype=torch.float32)
    mids = (book[:-1] + book[1:]) * 0.5
    kf = k.to(torch.float32)
    amax = kf.abs().amax(dim=1).clamp_min(1e-6)
    unit = (kf / amax.unsqueeze(1)).clamp(-1.0, 1.0)
    idx = torch.bucketize(unit, mids)
    recon = book[idx] * amax.unsqueeze(1)
    resid = (kf - recon).to(fp8_dtype).contiguous()
    return pack_codes(idx.to(torch.uint8), 4), amax.to(k.dtype).contiguous(), resid


def quantize_nvfp4(k: torch.Tensor, fp8_dtype: torch.dtype, page_size: int):
    """e2m1 nibbles with one scale per (b, page, kv-head) = absmax/6 held in K's dtype;
    everything is evaluated in K's dtype (ffa-nvfp4fp8/fused_kproj_rope_nvfp4fp8.py:62-114)."""
    if page_size <= 0:
        raise ValueError(f"page_size must be positive, got {page_size}")
    B, T, H, D = k.shape
    n_pages = (T + page_size - 1) // page_size
    kp = F.pad(k, (0, 0, 0, 0, 0, n_pages * page_size - T)) if n_pages * page_size != T else k
    blocks = kp.reshape(B, n_pages, page_size, H, D)
    top = torch.tensor(E2M1_LEVELS[-1], dtype=k.dtype)
    scale = (blocks.abs().amax(dim=(2, 4)) / top).clamp_min(1e-6).to(k.dtype).contiguous()
    sb = scale[:, :, None, :, None]
    nib, val = _e2m1_encode(blocks / sb)
    resid = (blocks - val * sb).to(fp8_dtype)
    nib = nib.reshape(B, n_pages * page_size, H, D)[:, :T]
    resid = resid.reshape(B, n_pages * page_size, H, D)[:, :T].contiguous()
    return pack_codes(nib, 4), scale, resid


# --------------------------------------------------------------------------------------
# coarse K tiles (what stage 1 feeds to its first dot): fp16 [B, n_tokens, HKV, K]
# --------------------------------------------------------------------------------------
def _e2m1_decode(nib: torch.Tensor) -> torch.Tensor:
    levels = torch.tensor(E2M1_LEVELS, dtype=torch.float32)
    mag = levels[(nib & 7).long()]
    return torch.where((nib >> 3) == 1, -mag, mag)


@dataclass
class CoarseK:
    """A coarse K cache in one of the five storage formats.

    ``tile(tokens, scale_block)`` returns the fp16 values the reference kernel builds
    for those token indices.  ``scale_block`` only matters for nvfp4, where the kernel
    picks the page scale by block index rather than by token (…nvfp4fp8.py:80,99,133).
    """
    kind: str
    codes: torch.Tensor
    scale: Optional[torch.Tensor] = None
    zero: Optional[torch.Tensor] = None
    head_dim: int = 128

    def tile(self, tokens: torch.Tensor, scale_block: Optional[torch.Tensor] = None) -> torch.Tensor:
        c = self.codes[:, tokens]
        D = self.head_dim
        if self.kind == "fp8":
            return c.to(torch.float16)
        if self.kind == "q2":
            lv = unpack_codes(c, 2, D).to(torch.float32)
            s = self.scale.to(torch.float32).unsqueeze(1)
            z = self.zero.to(torch.float32).unsqueeze(1)
            return (lv * s + z).to(torch.float16)
        if self.kind == "fp4":
            return _e2m1_decode(unpack_codes(c, 4, D)).to(torch.float16)
        if self.kind == "nf4":
            book = torch.tensor(NF4_LEVELS, dtype=torch.float32)
            val = book[unpack_codes(c, 4, D).long()]
            return (val * self.scale.to(torch.float32).unsqueeze(1)).to(torch.float16)
        if self.kind == "nvfp4":
            # scale [B, NTB, HKV]; one block index per token
            sc = self.scale.to(torch.float32)[:, scale_block]  # [B, n, HKV]
            return (_e2m1_decode(unpack_codes(c, 4, D)) * sc.unsqueeze(-1)).to(torch.float16)
        raise ValueError(self.kind)


# --------------------------------------------------------------------------------------
# decode attention
# --------------------------------------------------------------------------------------
def _scores(q16: torch.Tensor, k16: torch.Tensor, sm_scale: float) -> torch.Tensor:
    """q16 [B,HKV,G,K] fp16, k16 [B,n,HKV,K] fp16 -> [B,HKV,G,n] fp32 in log2 units.
    fp16 x fp16 products are exact in fp32; the dot accumulates in fp32 and is then
    multiplied by the softmax scale and by log2(e), in that order (…q2fp8.py:94)."""
    dots = torch.einsum("bhgk,bnhk->bhgn", q16.to(torch.float32), k16.to(torch.float32))
    return (dots * sm_scale) * LOG2E


def decode_threshold(q16, coarse: CoarseK, T: int, BS: int, sm_scale: float, delta: float) -> torch.Tensor:
    """Per-q-head prune threshold from two 16-token samples of the coarse K:
    tokens [0,16) and [(NTB-1)*16, (NTB-1)*16+16), NTB = ceil(T/BS)  (…q2fp8.py:58-82)."""
    NTB = (T + BS - 1) // BS
    best = None
    for blk in (0, NTB - 1):
        tok = blk * THRESHOLD_SAMPLE + torch.arange(THRESHOLD_SAMPLE)
        live = tok < T
        tok_c = tok.clamp_max(T - 1)
        sb = torch.full_like(tok_c, blk)
        s = _scores(q16, coarse.tile(tok_c, sb), sm_scale)
        s = torch.where(live, s, torch.tensor(float("-inf")))
        m = s.amax(dim=-1)
        best = m if best is None else torch.maximum(best, m)
    return best - delta  # [B,HKV,G]


def decode_attention(
    q: torch.Tensor,                # [B, 1, HQ, K] or [B, HQ, K]
    coarse: CoarseK,
    v: torch.Tensor,                # [B, T, HKV, V]
    k_residual: Optional[torch.Tensor] = None,
    *,
    sm_scale: Optional[float] = None,
    BS: int = 128,
    SBS: Optional[int] = None,
    delta: float = 5.0,
    precomputed_threshold: Optional[torch.Tensor] = None,   # [B, HQ] fp32
    use_fp8_residual: bool = True,
    out_dtype: Optional[torch.dtype] = None,
    return_parts: bool = False,
    mean_v: Optional[torch.Tensor] = None,                  # [B, HKV, V]: the mean-V variant
    keep_override: Optional[torch.Tensor] = None,           # [B, HKV, NTBS]: kept set imposed by the caller
):
    """Stage 1 + stage 2 of the reference decode path on CPU.

    ``keep_override`` replaces the prune decision (the coarse maxima and thresholds are still
    computed and returned): the tests use it to check an output whose kept set differs from the
    reference's on pages that sit within the allowed band around a threshold.

    Returns ``o [B,HQ,V]`` (and, with ``return_parts``, a dict holding the kept mask
    ``[B,HKV,NTBS]`` int8, the thresholds ``[B,HQ]`` and the per-block coarse maxima
    ``[B,HQ,NTBS]``).

    With ``mean_v`` the pruned sub-blocks are not dropped: each contributes its coarse softmax mass
    times the mean of V (ffa-q2fp8-meanv/attn_kernel/attn_kernel_v1210_meanv_bsz_q2fp8.py:107-119
    for the per-block (m, l), :169-200 for the separate scalar recurrence and the final fold)."""
    if q.dim() == 4:
        q = q[:, 0]
    B, HQ, K = q.shape
    T, HKV, V = v.shape[1], v.shape[2], v.shape[3]
    G = HQ // HKV
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(K)
    if SBS is None:
        SBS = BS
    NTB = (T + BS - 1) // BS
    NSB = (BS + SBS - 1) // SBS
    NTBS = NTB * NSB
    use_res = use_fp8_residual and k_residual is not None
    neg_inf = torch.tensor(float("-inf"))

    q16 = q.to(torch.float16).reshape(B, HKV, G, K)
    if precomputed_threshold is not None:
        th = precomputed_threshold.to(torch.float32).reshape(B, HKV, G)
    else:
        th = decode_threshold(q16, coarse, T, BS, sm_scale, delta)

    mask = torch.zeros(B, HKV, NTBS, dtype=torch.int8)
    blk_max = torch.full((B, HKV, G, NTBS), float("-inf"))
    run_m = torch.full((B, HKV, G), float("-inf"))
    run_l = torch.zeros(B, HKV, G)
    run_o = torch.zeros(B, HKV, G, V)
    apx_m = torch.full((B, HKV, G), float("-inf"))          # mean-V: running max / mass of pruned blocks
    apx_l = torch.zeros(B, HKV, G)

    for tb in range(NTB):
        for sb in range(NSB):
            t0 = tb * BS + sb * SBS
            idx = tb * NSB + sb
            tok = t0 + torch.arange(SBS)
            live = tok < T
            if not bool(live.any()):
                continue  # every score is -inf: pruned (…q2fp8.py:95-102)
            tok_c = tok.clamp_max(T - 1)
            k16 = coarse.tile(tok_c, torch.full_like(tok_c, tb))
            s_c = torch.where(live, _scores(q16, k16, sm_scale), neg_inf)
            m_c = s_c.amax(dim=-1)                       # [B,HKV,G]
            blk_max[..., idx] = m_c
            keep = ~((m_c < th).all(dim=-1))             # strict <, all heads of the group
            if keep_override is not None:
                keep = keep_override[..., idx].to(torch.bool)
            mask[..., idx] = keep.to(torch.int8)
            if mean_v is not None and not bool(keep.all()):
                p_c = torch.where(live, torch.exp2(s_c - m_c.unsqueeze(-1)), torch.tensor(0.0))
                l_c = p_c.sum(dim=-1)
                new_m = torch.maximum(apx_m, m_c)
                pr = ~keep.unsqueeze(-1)                                 # pruned (b, kv-head)s
                apx_l = torch.where(pr, apx_l * torch.exp2(apx_m - new_m) + l_c * torch.exp2(m_c - new_m), apx_l)
                apx_m = torch.where(pr, new_m, apx_m)
            if not bool(keep.any()):
                continue
            if use_res:
                k_ref = k16 + k_residual[:, tok_c].to(torch.float16)   # fp16 add (…q2fp8.py:115)
                s = torch.where(live, _scores(q16, k_ref, sm_scale), neg_inf)
                m = s.amax(dim=-1)
            else:
                s, m = s_c, m_c
            p = torch.where(live, torch.exp2(s - m.unsqueeze(-1)), torch.tensor(0.0))
            l = p.sum(dim=-1)
            v16 = v[:, tok_c].to(torch.float16).to(torch.float32)
            v16 = v16 * live.view(1, -1, 1, 1)
            o_b = torch.einsum("bhgn,bnhv->bhgv", p.to(torch.float16).to(torch.float32), v16)
            # stage 2: masked online merge in block order (…q2fp8.py:156-167)
            new_m = torch.maximum(run_m, m)
            r_prev = torch.exp2(run_m - new_m)
            r_blk = torch.exp2(m - new_m)
            kp = keep.unsqueeze(-1)
            run_l = torch.where(kp, run_l * r_prev + l * r_blk, run_l)
            run_o = torch.where(kp.unsqueeze(-1), run_o * r_prev.unsqueeze(-1) + o_b * r_blk.unsqueeze(-1), run_o)
            run_m = torch.where(kp, new_m, run_m)

    if mean_v is None:
        out = torch.where((run_l == 0).unsqueeze(-1), torch.zeros_like(run_o), run_o / run_l.unsqueeze(-1))
    else:
        have_any = (run_l > 0) | (apx_l > 0)
        new_m = torch.where(have_any, torch.maximum(run_m, apx_m), torch.zeros_like(run_m))
        r_b, r_p = torch.exp2(run_m - new_m), torch.exp2(apx_m - new_m)
        acc = run_l * r_b + apx_l * r_p
        mv = mean_v.to(torch.float32).unsqueeze(2)                       # [B,HKV,1,V]
        o_t = run_o * r_b.unsqueeze(-1) + mv * (apx_l * r_p).unsqueeze(-1)
        out = torch.where(have_any.unsqueeze(-1), o_t / acc.unsqueeze(-1), torch.zeros_like(o_t))
    out = out.reshape(B, HQ, V).to(out_dtype or q.dtype)
    if return_parts:
        return out, {
            "mask": mask,
            "threshold": th.reshape(B, HQ),
            "block_max": blk_max.reshape(B, HQ, NTBS),
        }
    return out


def decode_attention_fast(
    q, coarse: CoarseK, v, k_residual=None, *, sm_scale=None, BS=128, SBS=None, delta=5.0,
    precomputed_threshold=None, use_fp8_residual=True, out_dtype=None, keep_override=None, return_parts=False,
):
    """Same math as :func:`decode_attention`, batched over all sub-blocks at once
    (requires T % SBS == 0).  This is the torch-eager CPU baseline that ``bench.py``
    times; the merge uses one global maximum instead of the serial block order, which
    changes results only in the last fp32 bits.  ``keep_override [B,HKV,N]`` imposes a kept
    set; ``return_parts`` adds a dict with the thresholds ``[B,HQ]`` and the per-block coarse
    maxima ``[B,HQ,N]`` to the returned tuple."""
    if q.dim() == 4:
        q = q[:, 0]
    B, HQ, K = q.shape
    T, HKV, V = v.shape[1], v.shape[2], v.shape[3]
    G = HQ // HKV
    sm_scale = 1.0 / math.sqrt(K) if sm_scale is None else sm_scale
    SBS = BS if SBS is None else SBS
    assert T % SBS == 0 and T % BS == 0
    N = T // SBS
    q16 = q.to(torch.float16).reshape(B, HKV, G, K)
    if precomputed_threshold is not None:
        th = precomputed_threshold.to(torch.float32).reshape(B, HKV, G)
    else:
        th = decode_threshold(q16, coarse, T, BS, sm_scale, delta)
    tok = torch.arange(T)
    k16 = coarse.tile(tok, tok // BS)                                    # [B,T,HKV,K] fp16
    s_c = _scores(q16, k16, sm_scale).reshape(B, HKV, G, N, SBS)
    m_c = s_c.amax(dim=-1)                                               # [B,HKV,G,N]
    keep = ~((m_c < th.unsqueeze(-1)).all(dim=2))                        # [B,HKV,N]
    if keep_override is not None:
        keep = keep_override.to(torch.bool)
    bi, hi, ni = keep.nonzero(as_tuple=True)
    out = torch.zeros(B, HKV, G, V)
    if bi.numel():
        kb = k16.reshape(B, N, SBS, HKV, K)[bi, ni, :, hi]               # [n,SBS,K] fp16
        if use_fp8_residual and k_residual is not None:
            kb = kb + k_residual.reshape(B, N, SBS, HKV, K)[bi, ni, :, hi].to(torch.float16)
            qq = q16[bi, hi].to(torch.float32)                           # [n,G,K]
            s = (torch.bmm(qq, kb.to(torch.float32).transpose(1, 2)) * sm_scale) * LOG2E
        else:
            s = s_c[bi, hi, :, ni]
        m = s.amax(dim=-1)                                               # [n,G]
        p = torch.exp2(s - m.unsqueeze(-1))
        l = p.sum(dim=-1)
        vb = v.reshape(B, N, SBS, HKV, V)[bi, ni, :, hi].to(torch.float16).to(torch.float32)
        ob = torch.bmm(p.to(torch.float16).to(torch.float32), vb)        # [n,G,V]
        unit = bi * HKV + hi
        gmax = torch.full((B * HKV, G), float("-inf")).scatter_reduce(0, unit[:, None].expand(-1, G), m, "amax")
        w = torch.exp2(m - gmax[unit])
        acc = torch.zeros(B * HKV, G).index_add_(0, unit, l * w)
        osum = torch.zeros(B * HKV, G, V).index_add_(0, unit, ob * w.unsqueeze(-1))
        out = torch.where((acc == 0).unsqueeze(-1), torch.zeros_like(osum), osum / acc.unsqueeze(-1))
    out = out.reshape(B, HQ, V).to(out_dtype or q.dtype)
    if return_parts:
        return out, keep.to(torch.int8), {"threshold": th.reshape(B, HQ), "block_max": m_c.reshape(B, HQ, N)}
    return out, keep.to(torch.int8)


# --------------------------------------------------------------------------------------
# partial (O, LSE) merge used by split-KV and by the sequence-sharded multi-GPU path
# --------------------------------------------------------------------------------------
def merge_partials(o_parts: torch.Tensor, lse_parts: torch.Tensor) -> torch.Tensor:
    """o_parts [R,B,HQ,V] normalised partial outputs, lse_parts [R,B,HQ] base-2
    log-sum-exp (-inf for an empty part) -> merged [B,HQ,V] fp32."""
    top = lse_parts.amax(dim=0)
    w = torch.exp2(lse_parts - torch.where(torch.isinf(top), torch.zeros_like(top), top))
    w = torch.where(torch.isinf(lse_parts), torch.zeros_like(w), w)
    den = w.sum(dim=0)
    num = (o_parts * w.unsqueeze(-1)).sum(dim=0)
    return torch.where((den == 0).unsqueeze(-1), torch.zeros_like(num), num / den.unsqueeze(-1))


# --------------------------------------------------------------------------------------
# RoPE and the K projection (ffa-q2fp8/fused_kproj_rope_q2fp8.py:10-37, 402-424)
# --------------------------------------------------------------------------------------
def rope_tables(seq_len: int, head_dim: int, base: float = 10000.0, dtype=torch.float32):
    """cos/sin [seq_len, head_dim]; entry i uses angle index i mod head_dim/2."""
    if head_dim % 2:
        raise ValueError(f"head_dim must be even for RoPE, got {head_dim}")
    expo = torch.arange(0, head_dim, 2, dtype=dtype) / head_dim
    inv = 1.0 / (base ** expo)
    ang = torch.outer(torch.arange(seq_len, dtype=dtype), inv)
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos(), ang.sin()


def rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B,T,H,D].  Pairs are interleaved (2j, 2j+1) while the tables are laid out in
    halves, so the two members of a pair see different angles; out = x*cos + rot(x)*sin
    with rot(x)[2j] = -x[2j+1], rot(x)[2j+1] = x[2j]."""
    if cos.dim() == 2:
        cos = cos[None, :, None, :]
        sin = sin[None, :, None, :]
    ev, od = x[..., 0::2], x[..., 1::2]
    rot = torch.stack((-od, ev), dim=-1).flatten(-2)
    return x * cos + rot * sin


def kproj_rope(h, w_k, cos, sin, n_kv_heads, head_dim, bias=None):
    """h [B,T,H] x W_k ([out,in] or [in,out]) -> post-RoPE K [B,T,HKV,D] in h's dtype."""
    if w_k.shape[1] != h.shape[-1]:
        if w_k.shape[0] != h.shape[-1]:
            raise ValueError(f"w_k shape {tuple(w_k.shape)} is incompatible with in_dim={h.shape[-1]}")
        w_k = w_k.t()
    lin = F.linear(h, w_k, bias)
    B, T, O = lin.shape
    if O != n_kv_heads * head_dim:
        raise ValueError("projection out_dim must be num_kv_heads*head_dim")
    return rope_apply(lin.view(B, T, n_kv_heads, head_dim), cos, sin)


QUANTIZERS: dict[str, Callable] = {
    "q2": quantize_q2, "fp8": quantize_fp8fp8, "fp4": quantize_fp4, "nf4": quantize_nf4, "nvfp4": quantize_nvfp4,
}


def make_coarse(kind: str, k: torch.Tensor, fp8_dtype: torch.dtype, page_size: int = 64) -> Tuple[CoarseK, torch.Tensor]:
    """Quantise K with the variant's quantiser and wrap the result for the decode oracle."""
    D = k.shape[-1]
    if kind == "q2":
        c, s, z, r = quantize_q2(k, fp8_dtype)
        return CoarseK("q2", c, s, z, D), r
    if kind == "fp8":
        c, r = quantize_fp8fp8(k, fp8_dtype)
        return CoarseK("fp8", c, head_dim=D), r
    if kind == "fp4":
        c, r = quantize_fp4(k, fp8_dtype)
        return CoarseK("fp4", c, head_dim=D), r
    if kind == "nf4":
        c, s, r = quantize_nf4(k, fp8_dtype)
        return CoarseK("nf4", c, s, head_dim=D), r
    if kind == "nvfp4":
        c, s, r = quantize_nvfp4(k, fp8_dtype, page_size)
        return CoarseK("nvfp4", c, s, head_dim=D), r
    raise ValueError(kind)
