"""Stages the reference's own CPU implementation of the path under oracle/_ref/ (git-ignored).

TEST INFRASTRUCTURE ONLY.  The reference (Ther-LF/plaquant) is pure Python on this path, so "building" it means
making its quantiser importable where the checkout of the reference is not mounted: this script copies, from a
checkout given on the command line, exactly the modules the fake-quant path imports

    promix/quantize/quant_utils.py   ActQuantizer, fake_quantize_nvfp4 / mxfp8          (:182-224, :660-751)
    promix/quantize/hadamard.py      imported by quant_utils (its CUDA transform is never called on this path)
    promix/utils.py                  imported by both
    inference/rotation.py            get_hadamard_matrix                                  (:21-29)

into oracle/_ref/ with their package layout, and writes a stub module for `fast_hadamard_transform` (a CUDA
extension the reference imports at promix/utils.py:7 and only calls from matmul_hadU_cuda, which this path
replaces by the reference's own pure-torch Hadamard matrix).  Nothing under oracle/_ref/ is committed; the
benchmark's CPU-baseline leg imports it when present (cpu_baseline.kind = "reference") and falls back to the C
port otherwise.  The product package never imports it.

    python oracle/build_ref.py /path/to/plaquant
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
FILES = [
    "promix/__init__.py", "promix/utils.py", "promix/quantize/__init__.py", "promix/quantize/quant_utils.py",
    "promix/quantize/hadamard.py", "promix/quantize/hadamard_data.json", "inference/__init__.py",
    "inference/rotation.py",
]
STUB = '''"""Stand-in for the CUDA extension the reference imports but never calls on the FP fake-quant path."""


def hadamard_transform(*args, **kwargs):
    raise RuntimeError("fast_hadamard_transform is not available; the FP fake-quant path does not call it")
'''


def build_ref(ref_root: str) -> str:
    """Copies the modules listed above from `ref_root`; returns oracle/_ref.  Raises if one is missing."""
    for rel in FILES:
        src = os.path.join(ref_root, rel)
        if not os.path.exists(src):
            if rel.endswith(".json"):
                continue
            raise FileNotFoundError(src)
        dst = os.path.join(REF_DIR, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(src, dst)
    with open(os.path.join(REF_DIR, "fast_hadamard_transform.py"), "w") as f:
        f.write(STUB)
    return REF_DIR


def available() -> bool:
    return os.path.exists(os.path.join(REF_DIR, "promix", "quantize", "quant_utils.py"))


def load():
    """Imports the staged reference modules; returns (quant_utils module, get_hadamard_matrix)."""
    if not available():
        raise RuntimeError("oracle/_ref is empty: run `python oracle/build_ref.py <reference checkout>`")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
    import importlib
    qu = importlib.import_module("promix.quantize.quant_utils")
    rot = importlib.import_module("inference.rotation")
    return qu, rot.get_hadamard_matrix


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(build_ref(sys.argv[1]))
