"""Import shim for the fp8fp8 decode op, as the reference's model code expects it
(ffa-fp8fp8/e2e/ffa_fwd_decode_fp8fp8.py:12-25): ``attn_forward_decode_fp8fp8`` is the variant's entry
point; if the CUDA library cannot be loaded the name still imports and raises when called."""
from __future__ import annotations

from typing import Any

try:
    from ..attn_kernel.attn_kernel_v1210_fused_bsz_fp8fp8 import attn_forward_decode_fp8fp8 as _kernel
except Exception as exc:  # pragma: no cover - diagnostic path
    _IMPORT_ERROR = exc

    def attn_forward_decode_fp8fp8(*args: Any, **kwargs: Any):
        raise RuntimeError("Failed to import the fp8fp8 decode kernel: build the CUDA library first "
                           "(python -m ffa_speedtest_b200.build).") from _IMPORT_ERROR
else:

    def attn_forward_decode_fp8fp8(*args: Any, **kwargs: Any):
        return _kernel(*args, **kwargs)
