"""Copy the reference's decode kernels, unmodified, into baseline/_ref (git-ignored).

    python baseline/install_reference.py [--reference /path/to/ffa-speedtest]

The reference (qluoluo/ffa-speedtest) is a set of plain Python files holding Triton kernels; it has
no package metadata, so there is nothing to ``pip install``.  What the benchmark's Triton column and
the JIT parity test need is the ``attn_kernel/`` directory of each variant.  Those files are copied
byte for byte; the only additions are empty ``__init__.py`` files and directory names with ``-``
replaced by ``_`` so that the modules (whose CUDA-graph wrappers use relative imports) can be
imported as ``ffa_<variant>.attn_kernel.<module>`` with ``baseline/_ref`` on ``sys.path``.
Nothing under baseline/_ref is part of the product or of its history.
"""
from __future__ import annotations

import argparse
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
VARIANT_DIRS = ("ffa-q2fp8", "ffa-fp8fp8", "ffa-fp4fp8", "ffa-nf4fp8", "ffa-nvfp4fp8", "ffa-q2fp8-h100", "ffa-q2fp8-meanv")


def install(reference: Path) -> list[Path]:
    copied = []
    for d in VARIANT_DIRS:
        src = reference / d / "attn_kernel"
        if not src.is_dir():
            continue
        dst = DEST / d.replace("-", "_") / "attn_kernel"
        dst.mkdir(parents=True, exist_ok=True)
        (dst.parent / "__init__.py").touch()
        (dst / "__init__.py").touch()
        for f in sorted(src.glob("*.py")):
            shutil.copyfile(f, dst / f.name)
            copied.append(dst / f.name)
    return copied


def load(variant_dir: str, module: str):
    """Import ``module`` of an installed variant, e.g. ``load("ffa_fp8fp8",
    "attn_kernel_v1210_fused_bsz_fp8fp8_cudagraph")``.  Raises ImportError when the copy (or Triton) is missing."""
    import importlib
    if not (DEST / variant_dir / "attn_kernel" / (module + ".py")).exists():
        raise ImportError(f"{DEST / variant_dir / 'attn_kernel' / (module + '.py')} is not installed "
                          "(run baseline/install_reference.py where the reference checkout is available)")
    if str(DEST) not in sys.path:
        sys.path.insert(0, str(DEST))
    return importlib.import_module(f"{variant_dir}.attn_kernel.{module}")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    a = ap.parse_args()
    files = install(Path(a.reference))
    print(f"copied {len(files)} files into {DEST}")
