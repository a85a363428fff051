"""The C-ABI library builds, loads and exports every symbol include/ffa_b200.h declares."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "ffa_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ffa_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_path():
    names = declared_symbols()
    for must in ("ffa_decode", "ffa_decode_workspace_bytes", "ffa_merge_partials", "ffa_quantize_q2",
                 "ffa_quantize_fp8fp8", "ffa_quantize_fp4", "ffa_quantize_nf4", "ffa_quantize_nvfp4"):
        assert must in names


def test_library_exports_every_declared_symbol(built_lib):
    lib = C.CDLL(str(built_lib))
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert not missing, missing
    lib.ffa_abi_version.restype = C.c_int
    assert lib.ffa_abi_version() >= 1


def test_plan_and_workspace_are_host_only(built_lib):
    from ffa_speedtest_b200 import _lib
    L = _lib.lib()
    ppc, nch = C.c_int32(), C.c_int32()
    assert L.ffa_decode_plan(8, 32768, 8, 0, C.byref(ppc), C.byref(nch)) == 0
    assert ppc.value >= 4 and nch.value * ppc.value >= 512 and (nch.value - 1) * ppc.value < 512
    assert L.ffa_decode_workspace_bytes(8, 32768, 32, 8, 0) >= 8 * 32 * nch.value * 130 * 4
    assert L.ffa_decode_plan(0, 10, 8, 0, None, None) < 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from ffa_speedtest_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.lib()
