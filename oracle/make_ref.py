"""Recipe that makes the reference's own CPU implementation of the path runnable next to the oracle.

Test infrastructure, not product code. The reference's implementation of the int8 path that runs on a CPU is its
PyTorch fake-quant module tree (lightseq/training/ops/pytorch/{quantization,torch_transformer_layers,util,
layer_base}.py and the vendored lightseq/training/pytorch_quantization package). It is pure Python, so "building" it
means placing those files, unmodified, under ``oracle/_ref/`` (git-ignored: it never enters this repository's
history) beside three EMPTY package files of our own: the reference's ``lightseq/training/__init__.py`` and the two
below it JIT-compile CUDA extensions at import and cannot run on a host without the matching toolkit.

    python oracle/make_ref.py <checkout of bytedance/lightseq>      (or $LIGHTSEQ_REF)

``available()`` tells whether the tree is in place; ``oracle/ref_torch.py`` imports it.
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"

FILES = [
    "lightseq/training/ops/pytorch/quantization.py",
    "lightseq/training/ops/pytorch/torch_transformer_layers.py",
    "lightseq/training/ops/pytorch/util.py",
    "lightseq/training/ops/pytorch/layer_base.py",
]
TREES = ["lightseq/training/pytorch_quantization"]
EMPTY_PACKAGES = ["lightseq", "lightseq/training", "lightseq/training/ops", "lightseq/training/ops/pytorch"]


def available() -> bool:
    return all((DEST / f).exists() for f in FILES) and (DEST / TREES[0] / "tensor_quant.py").exists()


def make(ref_root: str) -> Path:
    ref = Path(ref_root)
    missing = [f for f in FILES if not (ref / f).exists()]
    if missing:
        raise SystemExit(f"{ref}: not a checkout of bytedance/lightseq (missing {missing[0]})")
    if DEST.exists():
        shutil.rmtree(DEST)
    for f in FILES:
        (DEST / f).parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(ref / f, DEST / f)
    for t in TREES:
        shutil.copytree(ref / t, DEST / t, ignore=shutil.ignore_patterns("__pycache__", "*.pyc", "*.so", "*.cu", "*.cpp"))
    for p in EMPTY_PACKAGES:
        (DEST / p / "__init__.py").write_text("")
    (DEST / "README.txt").write_text(
        "Unmodified files of bytedance/lightseq placed here by oracle/make_ref.py so that the reference's own PyTorch\n"
        "fake-quant modules can be timed and compared on a host without the reference checkout. The four __init__.py\n"
        "files directly under lightseq/, training/, ops/ and ops/pytorch/ are empty stand-ins (the originals build CUDA\n"
        "extensions at import). Not part of this repository's history.\n")
    return DEST


if __name__ == "__main__":
    root = os.environ.get("LIGHTSEQ_REF") or (sys.argv[1] if len(sys.argv) > 1 else "")
    if not root:
        raise SystemExit("usage: python oracle/make_ref.py <checkout of bytedance/lightseq>")
    print("reference modules placed under", make(root))
