#!/usr/bin/env python
"""Stage the reference's own kernel_bench modules next to the oracle (TEST INFRASTRUCTURE ONLY).

The reference (PanZaifeng/FastTree-Artifact) is pure Python + Triton, so there
is nothing to compile: "building" the reference for this path means placing
its unmodified source files where the GPU tests and the benchmark's baseline
leg can import them.  This script copies

    kernel_bench/fasttree.py          planner + Triton stage-1 / stage-2 kernels
    kernel_bench/kv_tree_simple.py    tree node record and file reader
    kernel_bench/tree_generation.py   layered tree generator / writer
    kernel_bench/DeFT.py              the reference's Triton DeFT baseline (timed by the benchmark CLI's GPU test)

from a reference checkout into ``oracle/_ref/kernel_bench/``.  That directory
is git-ignored (the reference's sources are never committed here) and is not
imported by anything in the shipped package; ``oracle/ref_triton.py`` loads it
under a private module name for

  * the ``-m gpu`` parity tests that compare the engine's output with the
    reference kernels' output on the same tensors (bf16 included), and
  * the ``reference_triton`` leg of ``bench.py``, which times the reference's
    kernels on the same GPU beside the engine.

Usage:  python oracle/stage_ref.py --reference /path/to/FastTree-Artifact
        (or set FASTTREE_REFERENCE_DIR)
"""
import argparse
import hashlib
import json
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
FILES = ["kernel_bench/fasttree.py", "kernel_bench/kv_tree_simple.py", "kernel_bench/tree_generation.py",
         "kernel_bench/DeFT.py"]


def stage(reference_dir, dest=DEST, quiet=False):
    """Copy FILES from ``reference_dir`` to ``dest``; returns the manifest
    (relative path -> SHA-256) that is also written to ``dest/MANIFEST.json``."""
    manifest = {}
    for rel in FILES:
        src = os.path.join(reference_dir, rel)
        if not os.path.isfile(src):
            raise FileNotFoundError(f"{src}: not a reference checkout")
        dst = os.path.join(dest, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(src, dst)
        with open(dst, "rb") as fh:
            manifest[rel] = hashlib.sha256(fh.read()).hexdigest()
    with open(os.path.join(dest, "MANIFEST.json"), "w") as fh:
        json.dump({"source": "PanZaifeng/FastTree-Artifact (unmodified files)", "sha256": manifest}, fh, indent=1)
    if not quiet:
        for rel, digest in manifest.items():
            print(f"staged {rel}  sha256 {digest[:16]}")
    return manifest


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--reference", default=os.environ.get("FASTTREE_REFERENCE_DIR"),
                    help="reference checkout (default: $FASTTREE_REFERENCE_DIR)")
    args = ap.parse_args()
    if not args.reference:
        ap.error("give --reference DIR or set FASTTREE_REFERENCE_DIR")
    stage(args.reference)


if __name__ == "__main__":
    sys.exit(main())
