"""The decode workspace: the reference's call shapes (ffa-q2fp8-h100/attn_kernel/
attn_kernel_v1210_fused_bsz_q2fp8.py:232-277) and the sizing rule behind them.  No GPU needed:
buffers are allocated on the CPU device, and the size function is plain host arithmetic."""
import pytest
import torch

from ffa_speedtest_b200 import _lib
from ffa_speedtest_b200.decode import DecodeWorkspace, allocate_decode_workspace


@pytest.mark.parametrize("B,HQ,HKV", [(1, 32, 8), (2, 32, 8), (1, 64, 8), (2, 64, 8), (1, 8, 8), (4, 16, 2),
                                      (8, 16, 2), (8, 32, 8), (32, 32, 8), (3, 6, 2)])
@pytest.mark.parametrize("ppc", [0, 1, 7, 64])
def test_workspace_bytes_never_shrink_with_length(built_lib, B, HQ, HKV, ppc):
    """A workspace sized for max_seq_len must serve every shorter sequence (a cache that grows during
    generation): bytes(T) is non-decreasing in T, page by page up to 128K tokens."""
    L = _lib.lib()
    prev = 0
    for T in range(64, 131072 + 1, 64):
        n = L.ffa_decode_workspace_bytes(B, T, HQ, HKV, ppc)
        assert n >= prev, f"T={T}: {n} < {prev}"
        prev = n
    assert L.ffa_decode_workspace_bytes(B, 131072 - 63, HQ, HKV, ppc) <= prev


def test_reference_constructor_and_matches(built_lib):
    q = torch.zeros(2, 1, 8, 128, dtype=torch.bfloat16)
    k_q = torch.zeros(2, 300, 2, 32, dtype=torch.uint8)
    v = torch.zeros(2, 300, 2, 128, dtype=torch.bfloat16)
    # allocate_q2fp8_decode_workspace(q, k_q, v, BS=128, SBS=None), positionally
    from ffa_speedtest_b200.q2fp8.attn_kernel.attn_kernel_v1210_fused_bsz_q2fp8 import (
        Q2FP8DecodeWorkspace, allocate_q2fp8_decode_workspace)
    ws = allocate_q2fp8_decode_workspace(q, k_q, v, 128, 64)
    assert isinstance(ws, Q2FP8DecodeWorkspace) and ws.NTBS == 3 * 2
    assert ws.o.shape == (2, 8, 128) and ws.o.dtype == torch.bfloat16
    assert ws.mask_buf.shape == (2, 2, 6) and ws.mask_buf.dtype == torch.int8
    assert ws.threshold_buf.shape == (2, 8) and ws.threshold_buf.dtype == torch.float32
    assert ws.matches(2, 8, 2, 128, 6, q.device, q.dtype)
    assert not ws.matches(2, 8, 2, 128, 5, q.device, q.dtype)
    assert not ws.matches(2, 8, 2, 128, 6, q.device, torch.float16)
    # defaults: BS = 128, SBS = BS
    assert allocate_q2fp8_decode_workspace(q, k_q, v).NTBS == 3
    # Q2FP8DecodeWorkspace(B, HQ, HKV, V, NTBS, device, dtype), positionally
    ws2 = Q2FP8DecodeWorkspace(2, 8, 2, 128, 6, q.device, q.dtype)
    assert ws2.matches(2, 8, 2, 128, 6, q.device, q.dtype) and ws2.scratch.numel() == ws.scratch.numel()
    with pytest.raises(ValueError, match=r"K/V layouts must be \[B, T, HKV, D\]"):
        allocate_q2fp8_decode_workspace(q, k_q[:, :200], v)
    # the keyword form used elsewhere in this package, and a growing cache
    ws3 = allocate_decode_workspace(q, v, BS=64, SBS=64, seq_len=4096)
    assert ws3.NTBS == 64 and ws3.fits(2, 8, 2, 128, 10, q.device, q.dtype) and not ws3.fits(2, 8, 2, 128, 65, q.device, q.dtype)
    assert isinstance(ws3, DecodeWorkspace)


def test_kproj_workspace_covers_its_regions(built_lib):
    """K-projection workspace = post-RoPE K + quantiser min/max + (k-split partial tiles for few tiles, or the
    epilogue's per-32-row min/max pairs when T is a multiple of the tile height) + 256 bytes of status."""
    L = _lib.lib()
    B, HKV, N = 1, 8, 1024
    bf16 = _lib.float_code(torch.bfloat16)

    def need(T):
        return L.ffa_kproj_workspace_bytes(B, T, HKV, bf16)

    k_and_mm = lambda T: T * N * 2 + B * N * 8
    # whole tiles, enough of them for an unsplit GEMM: one (min, max) pair per 32 rows and channel on top
    assert need(8192) >= k_and_mm(8192) + (8192 // 32) * N * 8 + 256
    # a ragged length keeps the separate min/max kernel: no such region
    assert need(8191) < k_and_mm(8191) + (8191 // 32) * N * 8
    # few tiles: fp32 partial tiles of the k split (up to 16 splits, capped at 16 MiB)
    assert need(64) >= k_and_mm(64) + 16 * 64 * N * 4 + 256
    assert need(1) >= k_and_mm(1) + 256
    assert L.ffa_kproj_workspace_bytes(0, 64, HKV, bf16) == 0
