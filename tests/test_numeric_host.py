"""The scalar quantiser code shared by the CUDA kernels (csrc/ffa_numeric.h), compiled for the
host, against torch casts and the oracle quantisers.  Bit-exact."""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import ffa_oracle as fo
from ffa_speedtest_b200.synth import make_decode_inputs

ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "ffa_speedtest_b200" / "csrc" / "ffa_numeric_host.cpp"
vp = C.c_void_p


@pytest.fixture(scope="module")
def host(tmp_path_factory):
    out = tmp_path_factory.mktemp("numeric") / "libffa_numeric_host.so"
    subprocess.run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", str(SRC), "-o", str(out)],
                   check=True)
    return C.CDLL(str(out))


def _probe_values():
    g = torch.Generator().manual_seed(0)
    x = torch.cat([torch.randn(100000, generator=g) * s for s in (1e-3, 0.1, 1, 30, 500, 70000)])
    every_bf16 = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).float()
    every_f16 = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.float16).float()
    edges = torch.tensor([464., 463.99, 464.01, 480., 479.9, 448., 61440., 61439., 65536., 65519., 65520.,
                          float("inf"), -float("inf"), 0.0, -0.0, 2.0 ** -9, 2.0 ** -10, 2.0 ** -17, 1.5 * 2.0 ** -10])
    x = torch.cat([x, every_bf16, every_f16, edges])
    return x[~torch.isnan(x)].contiguous()


@pytest.mark.parametrize("fmt,dt", [(0, torch.float8_e5m2), (1, torch.float8_e4m3fn)])
def test_fp8_casts(host, fmt, dt):
    x = _probe_values()
    out = np.zeros(x.numel(), dtype=np.uint8)
    host.ffa_host_f32_to_fp8(vp(x.data_ptr()), C.c_int64(x.numel()), fmt, vp(out.ctypes.data))
    assert np.array_equal(out, x.to(dt).view(torch.uint8).numpy())
    codes = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    back = np.zeros(256, dtype=np.float32)
    host.ffa_host_fp8_to_f32(vp(codes.data_ptr()), C.c_int64(256), fmt, vp(back.ctypes.data))
    ref = codes.view(dt).float().numpy()
    assert np.all((back == ref) | (np.isnan(back) & np.isnan(ref)))


@pytest.mark.parametrize("code,dt", [(0, torch.float16), (1, torch.bfloat16)])
def test_round_to_dtype(host, code, dt):
    x = _probe_values()
    out = np.zeros(x.numel(), dtype=np.float32)
    host.ffa_host_round_to(vp(x.data_ptr()), C.c_int64(x.numel()), code, vp(out.ctypes.data))
    assert np.array_equal(out, x.to(dt).float().numpy())


def _u16(t):
    if t.dtype == torch.float32:
        return t.view(torch.int32).numpy().view(np.uint32).ravel()
    return t.view(torch.int16).numpy().view(np.uint16).ravel()


@pytest.mark.parametrize("dtc,dt", [(1, torch.bfloat16), (0, torch.float16), (2, torch.float32)])
@pytest.mark.parametrize("fmt,f8", [(0, torch.float8_e5m2), (1, torch.float8_e4m3fn)])
def test_quantisers(host, dtc, dt, fmt, f8):
    B, T, HKV = 2, 203, 2
    _, k, _ = make_decode_inputs(B, T, 8, HKV, 128, seed=5, dtype=torch.bfloat16 if dt == torch.float32 else dt,
                                 n_heavy=2)
    if dt == torch.float32:
        k = k.float() * 1.0009765625      # values that need more than 16 bits
    k[:, :, 0, 5] = 0.75          # constant channel: exercises the scale floor
    k[:, :, 1, 9] = 0.0
    k = k.contiguous()
    n = k.numel()
    kp = vp(k.data_ptr())

    def buf(m, t=np.uint8):
        return np.zeros(m, dtype=t)

    c, s, z, r = fo.quantize_q2(k, f8)
    st = np.uint32 if dt == torch.float32 else np.uint16
    oc, os_, oz, orr = buf(n // 4), buf(B * HKV * 128, st), buf(B * HKV * 128, st), buf(n)
    host.ffa_host_quantize_q2(kp, dtc, B, T, HKV, fmt, vp(oc.ctypes.data), vp(os_.ctypes.data), vp(oz.ctypes.data),
                              vp(orr.ctypes.data))
    assert np.array_equal(oc, c.numpy().ravel()) and np.array_equal(os_, _u16(s)) and np.array_equal(oz, _u16(z))
    assert np.array_equal(orr, r.view(torch.uint8).numpy().ravel())

    c, r = fo.quantize_fp8fp8(k, f8)
    ob, orr = buf(n), buf(n)
    host.ffa_host_quantize_fp8fp8(kp, dtc, C.c_int64(n), fmt, vp(ob.ctypes.data), vp(orr.ctypes.data))
    assert np.array_equal(ob, c.view(torch.uint8).numpy().ravel())
    assert np.array_equal(orr, r.view(torch.uint8).numpy().ravel())

    c, r = fo.quantize_fp4(k, f8)
    oc, orr = buf(n // 2), buf(n)
    host.ffa_host_quantize_fp4(kp, dtc, C.c_int64(n), fmt, vp(oc.ctypes.data), vp(orr.ctypes.data))
    assert np.array_equal(oc, c.numpy().ravel()) and np.array_equal(orr, r.view(torch.uint8).numpy().ravel())

    c, s, r = fo.quantize_nf4(k, f8)
    oc, os_, orr = buf(n // 2), buf(B * HKV * 128, st), buf(n)
    host.ffa_host_quantize_nf4(kp, dtc, B, T, HKV, fmt, vp(oc.ctypes.data), vp(os_.ctypes.data), vp(orr.ctypes.data))
    assert np.array_equal(oc, c.numpy().ravel()) and np.array_equal(os_, _u16(s))
    assert np.array_equal(orr, r.view(torch.uint8).numpy().ravel())

    c, s, r = fo.quantize_nvfp4(k, f8, 64)
    npg = (T + 63) // 64
    oc, os_, orr = buf(n // 2), buf(B * npg * HKV, st), buf(n)
    host.ffa_host_quantize_nvfp4(kp, dtc, B, T, HKV, fmt, 64, vp(oc.ctypes.data), vp(os_.ctypes.data),
                                 vp(orr.ctypes.data))
    assert np.array_equal(oc, c.numpy().ravel()) and np.array_equal(os_, _u16(s))
    assert np.array_equal(orr, r.view(torch.uint8).numpy().ravel())
