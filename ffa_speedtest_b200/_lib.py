"""ctypes binding of libffa_b200.so (the C ABI declared in include/ffa_b200.h).

There is no fallback: if the shared library is missing or a call fails, an exception is
raised.  Build it with ``python -m ffa_speedtest_b200.build`` (needs nvcc, no GPU).
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libffa_b200.so"

F16, BF16, F32 = 0, 1, 2
E5M2, E4M3 = 0, 1
K_FP8, K_Q2, K_FP4, K_NF4, K_NVFP4 = 0, 1, 2, 3, 4
VARIANT_CODE = {"fp8": K_FP8, "q2": K_Q2, "fp4": K_FP4, "nf4": K_NF4, "nvfp4": K_NVFP4}

_ERRORS = {
    -1: "FFA_E_NULL (a required pointer is NULL)",
    -2: "FFA_E_SHAPE (unsupported dimension)",
    -3: "FFA_E_DTYPE (unsupported element type)",
    -4: "FFA_E_WORKSPACE (workspace too small)",
    -5: "FFA_E_LAUNCH (CUDA runtime error)",
    -6: "FFA_E_VARIANT (unknown coarse-K format)",
    -7: "FFA_E_LIMIT (size beyond a compiled-in maximum)",
    -8: "FFA_E_ALIGN (a tensor pointer is not 16-byte aligned)",
}


class FfaDecodeArgs(C.Structure):
    _fields_ = [
        ("variant", C.c_int32),
        ("B", C.c_int32), ("T", C.c_int32), ("HQ", C.c_int32), ("HKV", C.c_int32),
        ("head_dim", C.c_int32),
        ("BS", C.c_int32), ("SBS", C.c_int32),
        ("sm_scale", C.c_float), ("delta", C.c_float),
        ("q_dtype", C.c_int32), ("v_dtype", C.c_int32), ("scale_dtype", C.c_int32),
        ("fp8_format", C.c_int32), ("use_residual", C.c_int32),
        ("q", C.c_void_p), ("k_codes", C.c_void_p), ("k_scale", C.c_void_p), ("k_zero", C.c_void_p),
        ("k_residual", C.c_void_p), ("v", C.c_void_p),
        ("block_table", C.c_void_p), ("bt_stride", C.c_int32),
        ("threshold_in", C.c_void_p),
        ("out", C.c_void_p), ("kept_mask", C.c_void_p), ("threshold_out", C.c_void_p), ("partial_out", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("pages_per_chunk", C.c_int32), ("reserved", C.c_int32),
        ("kv_rows", C.c_int64),
        ("v_mean", C.c_void_p),
    ]


class FfaPeerArgs(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("step", C.c_int32),
                ("peer_gathered", C.POINTER(C.c_void_p)), ("peer_flags", C.POINTER(C.c_void_p))]


class FfaKprojArgs(C.Structure):
    _fields_ = [
        ("variant", C.c_int32),
        ("B", C.c_int32), ("T", C.c_int32), ("H", C.c_int32), ("HKV", C.c_int32), ("head_dim", C.c_int32),
        ("io_dtype", C.c_int32), ("rope_dtype", C.c_int32), ("fp8_format", C.c_int32), ("page_size", C.c_int32),
        ("h", C.c_void_p), ("w", C.c_void_p), ("bias", C.c_void_p), ("cos", C.c_void_p), ("sin", C.c_void_p),
        ("slot_table", C.c_void_p), ("slot_stride", C.c_int32), ("slot_pos0", C.c_int32),
        ("codes", C.c_void_p), ("scale", C.c_void_p), ("zero", C.c_void_p), ("residual", C.c_void_p),
        ("k_rope_out", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


_lib = None


def lib() -> C.CDLL:
    """Load the shared library once; fail loudly if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: the CUDA library of ffa_speedtest_b200 has not been built. "
            "Run `python -m ffa_speedtest_b200.build` (needs nvcc). There is no fallback path."
        )
    L = C.CDLL(os.fspath(LIB_PATH))
    L.ffa_decode.argtypes = [C.POINTER(FfaDecodeArgs), C.c_void_p]
    L.ffa_decode.restype = C.c_int
    L.ffa_decode_workspace_bytes.argtypes = [C.c_int32] * 5
    L.ffa_decode_workspace_bytes.restype = C.c_size_t
    L.ffa_decode_plan.argtypes = [C.c_int32] * 4 + [C.POINTER(C.c_int32)] * 2
    L.ffa_decode_plan.restype = C.c_int
    L.ffa_merge_partials.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]
    L.ffa_merge_partials.restype = C.c_int
    L.ffa_quantize_scratch_bytes.argtypes = [C.c_int32, C.c_int32]
    L.ffa_quantize_scratch_bytes.restype = C.c_size_t
    vp, i32 = C.c_void_p, C.c_int32
    L.ffa_quantize_q2.argtypes = [vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp]
    L.ffa_quantize_fp8fp8.argtypes = [vp, i32, i32, i32, i32, i32, vp, vp, vp]
    L.ffa_quantize_fp4.argtypes = [vp, i32, i32, i32, i32, i32, vp, vp, vp]
    L.ffa_quantize_nf4.argtypes = [vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp]
    L.ffa_quantize_nvfp4.argtypes = [vp, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp]
    for name in ("ffa_quantize_q2", "ffa_quantize_fp8fp8", "ffa_quantize_fp4", "ffa_quantize_nf4",
                 "ffa_quantize_nvfp4"):
        getattr(L, name).restype = C.c_int
    L.ffa_cache_append.argtypes = [i32, vp, vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, i32, i32, vp]
    L.ffa_cache_append.restype = C.c_int
    L.ffa_peer_exchange_merge.argtypes = [vp, i32, i32, i32, C.POINTER(vp), C.POINTER(vp), i32, vp, i32, vp, vp]
    L.ffa_peer_exchange_merge.restype = C.c_int
    L.ffa_decode_peer.argtypes = [C.POINTER(FfaDecodeArgs), C.POINTER(FfaPeerArgs), C.c_void_p]
    L.ffa_decode_peer.restype = C.c_int
    L.ffa_peer_wait_merge.argtypes = [vp, vp, i32, i32, i32, vp, i32, vp, vp]
    L.ffa_peer_wait_merge.restype = C.c_int
    L.ffa_peer_alloc.argtypes = [C.c_size_t, C.POINTER(vp), C.c_char_p]
    L.ffa_peer_open.argtypes = [C.c_char_p, C.POINTER(vp)]
    L.ffa_peer_close.argtypes = [vp]
    L.ffa_peer_free.argtypes = [vp]
    for name in ("ffa_peer_alloc", "ffa_peer_open", "ffa_peer_close", "ffa_peer_free"):
        getattr(L, name).restype = C.c_int
    L.ffa_quantize_append.argtypes = [i32, vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, i32, i32, vp]
    L.ffa_quantize_append.restype = C.c_int
    L.ffa_kproj_rope.argtypes = [C.POINTER(FfaKprojArgs), C.c_void_p]
    L.ffa_kproj_rope.restype = C.c_int
    L.ffa_kproj_workspace_bytes.argtypes = [i32, i32, i32, i32]
    L.ffa_kproj_workspace_bytes.restype = C.c_size_t
    L.ffa_last_cuda_error.restype = C.c_char_p
    L.ffa_abi_version.restype = C.c_int
    _lib = L
    return L


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    msg = _ERRORS.get(rc, f"error {rc}")
    if rc == -5:
        msg += ": " + lib().ffa_last_cuda_error().decode()
    raise RuntimeError(f"{what} failed: {msg}")


def float_code(dt: torch.dtype) -> int:
    try:
        return {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}[dt]
    except KeyError:
        raise ValueError(f"unsupported floating dtype {dt}") from None


def fp8_code(dt: torch.dtype) -> int:
    try:
        return {torch.float8_e5m2: E5M2, torch.float8_e4m3fn: E4M3}[dt]
    except KeyError:
        raise ValueError(f"expected torch.float8_e5m2 or torch.float8_e4m3fn, got {dt}") from None


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def current_stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream
