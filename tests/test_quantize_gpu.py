"""CUDA quantisers against the oracle (itself bit-exact with the reference): bit-exact."""
import pytest
import torch

from oracle import ffa_oracle as fo
from ffa_speedtest_b200 import quantize as Q
from ffa_speedtest_b200.synth import make_decode_inputs

pytestmark = pytest.mark.gpu


def same(a: torch.Tensor, b: torch.Tensor) -> bool:
    a, b = a.cpu().contiguous(), b.cpu().contiguous()
    if a.dtype.itemsize == 1:
        return torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    if a.dtype.itemsize == 4:
        return torch.equal(a.view(torch.int32), b.view(torch.int32))
    return torch.equal(a.view(torch.int16), b.view(torch.int16))


def make_k(dt, T=203):
    _, k, _ = make_decode_inputs(2, T, 8, 2, 128, seed=5, dtype=dt, n_heavy=2)
    k[:, :, 0, 5] = 0.75
    k[:, :, 1, 9] = 0.0
    # large but inside e4m3's finite range: overflow makes NaN codes whose sign bit differs between
    # x86 and CUDA arithmetic (NaN propagation), which is not a property of the quantiser
    k[0, 3, 0, 0] = 440.0
    k[0, 4, 1, 1] = -300.0
    return k.contiguous()


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("f8", [torch.float8_e5m2, torch.float8_e4m3fn])
def test_all_quantisers_bit_exact(dt, f8):
    """float32 K is what the reference's kproj recipe produces when the RoPE tables are fp32."""
    k = make_k(torch.bfloat16).float() * 1.0009765625 if dt == torch.float32 else make_k(dt)
    kd = k.cuda()
    for got, ref in zip(Q.quantize_k_2bit_fp8_residual(kd, f8), fo.quantize_q2(k, f8)):
        assert same(got, ref)
    for got, ref in zip(Q.quantize_k_fp8_fp8_residual(kd, f8), fo.quantize_fp8fp8(k, f8)):
        assert same(got, ref)
    for got, ref in zip(Q.encode_k_fp4_fp8_residual(kd, f8), fo.quantize_fp4(k, f8)):
        assert same(got, ref)
    for got, ref in zip(Q.encode_k_nf4_fp8_residual(kd, f8), fo.quantize_nf4(k, f8)):
        assert same(got, ref)
    for page in (64, 128):
        for got, ref in zip(Q.encode_k_nvfp4_fp8_residual(kd, f8, page), fo.quantize_nvfp4(k, f8, page)):
            assert same(got, ref)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_q2_quotient_rounding_on_many_values(dt):
    """(k - zero) / scale rounded to K's dtype, then to the nearest code with ties to even: four million
    values, plus constructed ties at code + 0.5 and tiny / huge magnitudes, must give the oracle's bits."""
    _, k, _ = make_decode_inputs(1, 4096, 32, 8, 128, seed=17, dtype=dt)
    k = k.contiguous()
    # channels with an exact grid: min 0, max 3 -> scale 1, so values at n + 0.5 are exact ties
    k[0, :, 0, 0] = torch.tensor([0.0, 3.0, 0.5, 1.5, 2.5, 2.4921875, 2.5078125, 1.0], dtype=dt).repeat(512)
    k[0, :, 1, 1] = torch.tensor([-1e-4, 1e-4, 0.0, 6e-5], dtype=dt).repeat(1024)
    k[0, :, 2, 2] = torch.tensor([-30000.0, 30000.0, 1.0, -1.0], dtype=dt).repeat(1024)
    for f8 in (torch.float8_e4m3fn, torch.float8_e5m2):
        for got, ref in zip(Q.quantize_k_2bit_fp8_residual(k.cuda(), f8), fo.quantize_q2(k, f8)):
            assert same(got, ref)


def test_large_shape_properties():
    """Config-1-sized K (cut to B=2): idempotence of the fp8 base and residual bound."""
    _, k, _ = make_decode_inputs(2, 32768, 32, 8, 128, seed=1, device="cuda")
    base, res = Q.quantize_k_fp8_fp8_residual(k, torch.float8_e4m3fn)
    assert torch.equal(base.view(torch.uint8), k.to(torch.float8_e4m3fn).view(torch.uint8))
    recon = base.float() + res.float()
    assert (recon - k.float()).abs().max().item() <= 2.0 ** -4 * k.float().abs().max().item() / 8
    base2, res2 = Q.quantize_k_fp8_fp8_residual(base.to(k.dtype), torch.float8_e4m3fn)
    assert torch.equal(base2.view(torch.uint8), base.view(torch.uint8)) and bool((res2.view(torch.uint8) & 0x7f == 0).all())
    codes, scale, zero, r = Q.quantize_k_2bit_fp8_residual(k, torch.float8_e5m2)
    assert torch.equal(zero, k.amin(dim=1)) and int(codes.max()) <= 255
