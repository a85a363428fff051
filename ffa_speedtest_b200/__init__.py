"""B200-native implementation of the FFA quantised, pruned decode-attention path.

Sub-packages mirror the variant directories of qluoluo/ffa-speedtest so that the reference's
``--kernel <module path>`` plug-in mechanism (ffa-q2fp8/run_attn_bench_q2.py:34-39,108-113) and
its direct imports keep working with only the package prefix changed, e.g.::

    ffa_speedtest_b200.q2fp8.attn_kernel.attn_kernel_v1210_fused_bsz_q2fp8
        -> attn_forward_decode_quantized

All compute runs in hand-written sm_100a CUDA kernels behind the C ABI in
``include/ffa_b200.h`` (``libffa_b200.so``).  There is no Triton path and no CPU fallback.
"""
__version__ = "0.1.0"
