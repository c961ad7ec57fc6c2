"""Stages the reference's own tree-matmul kernel for GPU runs (TEST INFRASTRUCTURE ONLY).

    python -m oracle.build_ref [reference checkout]

The reference kernel (src/tbik/tree_based_matmul.py of nanomaoli/llm_reproducibility: a Triton kernel plus its
host wrapper `matmul_tp_persistent`) is JIT-compiled from its Python source at run time, so "building" it for a
machine that has no checkout of the reference means placing that one file, byte for byte, where the GPU tests
and the benchmark's comparator leg look for it: oracle/_ref/.  That folder is a build output: it is listed in
.gitignore, nothing in it is ever committed, and nothing of the product imports it.  The tests that use it skip
when it is absent.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
RELATIVE_SOURCE = os.path.join("src", "tbik", "tree_based_matmul.py")
DEFAULT_CHECKOUT = os.environ.get("TBIK_REFERENCE_CHECKOUT", "/root/reference")


def build(checkout: str = DEFAULT_CHECKOUT) -> str | None:
    """Copy the kernel file into oracle/_ref/ and return its path; None when there is no checkout."""
    src = os.path.join(checkout, RELATIVE_SOURCE)
    if not os.path.isfile(src):
        return None
    os.makedirs(OUT_DIR, exist_ok=True)
    dst = os.path.join(OUT_DIR, os.path.basename(src))
    shutil.copyfile(src, dst)
    with open(dst, "rb") as f:
        digest = hashlib.sha256(f.read()).hexdigest()
    with open(os.path.join(OUT_DIR, "SOURCE.txt"), "w") as f:
        f.write(f"{RELATIVE_SOURCE} of the reference checkout, unmodified\nsha256 {digest}\n")
    return dst


if __name__ == "__main__":
    out = build(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_CHECKOUT)
    print(out if out else "no reference checkout found; nothing staged")
