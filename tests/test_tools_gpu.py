"""The command-line drivers: one tiny run each, checked for the result they promise."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def run(*args):
    return subprocess.run([sys.executable, *args], cwd=ROOT, capture_output=True, text=True, timeout=600)


def test_run_attn_bench_writes_the_reference_result_schema(tmp_path):
    r = run("-m", "ffa_speedtest_b200.run_attn_bench", "--variant", "fp4fp8", "--dtype", "bf16", "--BS", "128",
            "--SBS", "64", "--max-length", "2048", "--step", "1024", "--iters", "3", "--warmup", "1", "--bsz", "2",
            "--out-dir", str(tmp_path))
    assert r.returncode == 0, r.stderr[-2000:]
    files = list(tmp_path.rglob("*.json"))
    assert len(files) == 1 and "_BS128_SBS64_delta5_bf16_step1024_it3_wu1_bsz2" in files[0].name
    d = json.loads(files[0].read_text())
    assert set(d) == {"meta", "lengths", "fused_ms", "flash_ms", "skip_ratios"}
    assert d["lengths"] == [1024, 2048] and len(d["fused_ms"]) == 2 and all(x > 0 for x in d["fused_ms"])
    assert all(0.0 <= s <= 1.0 for s in d["skip_ratios"])
    assert d["meta"]["BS"] == 128 and d["meta"]["SBS"] == 64 and d["meta"]["bsz"] == 2


@pytest.mark.parametrize("what,variant", [("decode", "nvfp4fp8"), ("kproj", "fp4fp8")])
def test_run_case(what, variant):
    r = run("-m", "ffa_speedtest_b200.run_case", what, "--variant", variant, "--B", "1", "--T", "512", "--iters", "2")
    assert r.returncode == 0, r.stderr[-2000:]
    assert variant in r.stdout and ("status 0" in r.stdout or "outputs" in r.stdout)


def test_run_attn_bench_cudagraph_schema_and_kernel_option(tmp_path):
    """The second reference driver: eager and CUDA-graph columns under the variant's key prefix
    (ffa-q2fp8/run_attn_bench_q2_cudagraph.py:148-173), with the kernel given as a module path."""
    r = run("-m", "ffa_speedtest_b200.run_attn_bench", "--variant", "q2fp8", "--dtype", "fp16", "--BS", "128",
            "--kernel", "ffa_speedtest_b200.q2fp8.attn_kernel.attn_kernel_v1210_fused_bsz_q2fp8", "--cudagraph",
            "--cg-warmup", "1", "--no-flash", "--max-length", "4096", "--step", "2048", "--iters", "3", "--warmup", "1",
            "--out-dir", str(tmp_path))
    assert r.returncode == 0, r.stderr[-2000:]
    files = list(tmp_path.rglob("*.json"))
    assert len(files) == 1 and files[0].name.endswith("_bsz1_cudagraph_replay.json")
    d = json.loads(files[0].read_text())
    assert set(d) == {"meta", "lengths", "q2_ms", "q2_cg_ms", "flash_ms", "skip_ratios"}
    assert d["lengths"] == [2048, 4096] and all(x > 0 for x in d["q2_ms"] + d["q2_cg_ms"])
    assert d["flash_ms"] == [None, None] and d["meta"]["cudagraph_replay_only"] is True


def test_run_attn_bench_rejects_a_module_without_the_entry_point(tmp_path):
    r = run("-m", "ffa_speedtest_b200.run_attn_bench", "--variant", "fp8fp8", "--kernel", "ffa_speedtest_b200.synth",
            "--max-length", "1024", "--out-dir", str(tmp_path))
    assert r.returncode != 0 and "does not define 'attn_forward_decode_fp8fp8'" in r.stderr
