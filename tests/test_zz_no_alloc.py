"""ffa_decode_static_scratch: the decode entry point that brings its own scratch memory.

Collected last on purpose (pytest orders files by name): if it fails, a run that stops at the
first failure has already run everything else.  The check is against the regular entry point,
called through the same C ABI on the same inputs, twice in a row - the second call runs on top
of whatever the first one left in the shared array.
"""
import ctypes as C

import pytest
import torch

from oracle import ffa_oracle as fo
from ffa_speedtest_b200 import _lib
from ffa_speedtest_b200.synth import make_decode_inputs

pytestmark = pytest.mark.gpu


def _args(q, codes, res, v, out, mask, workspace, delta, *, variant=None, scale=None, zero=None, BS=64, SBS=64):
    """FfaDecodeArgs for a decode on contiguous [B, T, HKV, D] tensors (fp8 K + fp8 residual unless a
    variant with its scale / zero tensors is given)."""
    B, _, HQ, K = q.shape
    T, HKV = v.shape[1], v.shape[2]
    a = _lib.FfaDecodeArgs()
    a.variant = _lib.K_FP8 if variant is None else variant
    a.B, a.T, a.HQ, a.HKV, a.head_dim = B, T, HQ, HKV, K
    a.BS, a.SBS = BS, SBS
    if scale is not None:
        a.k_scale = scale.data_ptr()
    if zero is not None:
        a.k_zero = zero.data_ptr()
    a.sm_scale, a.delta = K ** -0.5, delta
    a.q_dtype = _lib.float_code(q.dtype)
    a.v_dtype = _lib.float_code(v.dtype)
    a.scale_dtype = _lib.F32 if scale is None else _lib.float_code(scale.dtype)
    a.fp8_format = _lib.fp8_code(res.dtype)
    a.use_residual = 1
    a.q, a.k_codes, a.k_residual, a.v = q.data_ptr(), codes.data_ptr(), res.data_ptr(), v.data_ptr()
    a.out, a.kept_mask = out.data_ptr(), mask.data_ptr()
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    a.kv_rows = B * T
    return a


def test_static_scratch_matches_regular_entry_point_twice():
    L = _lib.lib()
    L.ffa_decode_static_scratch.argtypes = [C.POINTER(_lib.FfaDecodeArgs), C.c_void_p]
    L.ffa_decode_static_scratch.restype = C.c_int
    L.ffa_static_scratch_bytes.restype = C.c_size_t
    dev = torch.device("cuda:0")
    stream = _lib.current_stream(dev)
    limit = L.ffa_static_scratch_bytes()
    assert limit == 4 << 20

    for seed, (B, T, delta) in enumerate([(2, 64 * 37 + 5, 5.0), (1, 4096, 8.0)]):
        q, k, v = make_decode_inputs(B, T, 32, 8, 128, seed=90 + seed, n_heavy=4)
        coarse, res = fo.make_coarse("fp8", k, torch.float8_e4m3fn, 64)
        q, codes, res, v = q.to(dev), coarse.codes.to(dev), res.to(dev), v.to(dev)
        ntbs = -(-T // 64)
        need = L.ffa_decode_workspace_bytes(B, T, 32, 8, 0)
        assert need <= limit
        ws = torch.zeros(need, dtype=torch.uint8, device=dev)
        want, want_mask = torch.empty(B, 32, 128, dtype=q.dtype, device=dev), torch.empty(B, 8, ntbs, dtype=torch.int8, device=dev)
        _lib.check(L.ffa_decode(_args(q, codes, res, v, want, want_mask, ws, delta), stream), "ffa_decode")
        for call in range(2):
            got = torch.full_like(want, float("nan"))
            got_mask = torch.full_like(want_mask, -1)
            rc = L.ffa_decode_static_scratch(_args(q, codes, res, v, got, got_mask, None, delta), stream)
            _lib.check(rc, "ffa_decode_static_scratch")
            torch.cuda.synchronize()
            assert torch.equal(got_mask, want_mask), f"call {call}: kept set differs"
            # same kernels on the same inputs: the tolerance of the other decode tests is far wider
            assert (got.float() - want.float()).abs().max().item() <= 2e-2, f"call {call}"
            assert torch.equal(got, want), f"call {call}: outputs are not bit-identical"


def test_static_scratch_prune_groups_and_status_word():
    """2-bit K pruned in groups of two pages (SBS = 128): the same comparison, twice in a row, plus the
    status block read back through ffa_static_scratch_status into pinned host memory."""
    L = _lib.lib()
    L.ffa_decode_static_scratch.argtypes = [C.POINTER(_lib.FfaDecodeArgs), C.c_void_p]
    L.ffa_decode_static_scratch.restype = C.c_int
    L.ffa_static_scratch_status.argtypes = [C.c_void_p, C.c_void_p]
    L.ffa_static_scratch_status.restype = C.c_int
    dev = torch.device("cuda:0")
    stream = _lib.current_stream(dev)
    B, T, delta = 2, 64 * 41 + 9, 4.0
    q, k, v = make_decode_inputs(B, T, 32, 8, 128, seed=95, n_heavy=4, dtype=torch.float16)
    coarse, res = fo.make_coarse("q2", k, torch.float8_e5m2, 128)
    q, codes, res, v = q.to(dev), coarse.codes.to(dev), res.to(dev), v.to(dev)
    scale, zero = coarse.scale.to(dev), coarse.zero.to(dev)
    ntbs = -(-T // 128)
    kw = dict(variant=_lib.K_Q2, scale=scale, zero=zero, BS=128, SBS=128)
    ws = torch.zeros(L.ffa_decode_workspace_bytes(B, T, 32, 8, 0), dtype=torch.uint8, device=dev)
    want, want_mask = torch.empty(B, 32, 128, dtype=q.dtype, device=dev), torch.empty(B, 8, ntbs, dtype=torch.int8, device=dev)
    _lib.check(L.ffa_decode(_args(q, codes, res, v, want, want_mask, ws, delta, **kw), stream), "ffa_decode")
    status = torch.full((7,), -1, dtype=torch.int32).pin_memory()
    for call in range(2):
        got, got_mask = torch.full_like(want, float("nan")), torch.full_like(want_mask, -1)
        _lib.check(L.ffa_decode_static_scratch(_args(q, codes, res, v, got, got_mask, None, delta, **kw), stream),
                   "ffa_decode_static_scratch")
        _lib.check(L.ffa_static_scratch_status(status.data_ptr(), stream), "ffa_static_scratch_status")
        torch.cuda.synchronize()
        assert status.tolist() == [0] * 7, f"call {call}: status block {status.tolist()}"
        assert torch.equal(got_mask, want_mask) and 0 < int(want_mask.sum()) < want_mask.numel()
        assert (got.float() - want.float()).abs().max().item() <= 2e-2, f"call {call}"
        assert torch.equal(got, want), f"call {call}: outputs are not bit-identical"
    assert L.ffa_static_scratch_status(None, stream) == -1        # FFA_E_NULL


def test_static_scratch_rejects_oversized_shapes():
    L = _lib.lib()
    L.ffa_decode_static_scratch.argtypes = [C.POINTER(_lib.FfaDecodeArgs), C.c_void_p]
    L.ffa_decode_static_scratch.restype = C.c_int
    dev = torch.device("cuda:0")
    # B=64 sequences of 64k tokens need more partial-result space than the built-in array holds;
    # the call must refuse before touching any tensor, so dummy one-element tensors are enough
    B, T = 64, 65536
    assert L.ffa_decode_workspace_bytes(B, T, 32, 8, 0) > (4 << 20)
    t = torch.zeros(16, dtype=torch.uint8, device=dev)
    a = _lib.FfaDecodeArgs()
    a.variant = _lib.K_FP8
    a.B, a.T, a.HQ, a.HKV, a.head_dim, a.BS, a.SBS = B, T, 32, 8, 128, 64, 64
    a.q = a.k_codes = a.k_residual = a.v = a.out = t.data_ptr()
    a.q_dtype, a.v_dtype, a.fp8_format, a.use_residual = _lib.BF16, _lib.BF16, _lib.E4M3, 1
    assert L.ffa_decode_static_scratch(a, _lib.current_stream(dev)) == -7      # FFA_E_LIMIT
    torch.cuda.synchronize()
