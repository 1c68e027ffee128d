"""Builds libfasttree_b200.so (sm_100a) in-tree with nvcc.

Usage:  python fasttree-artifact_b200/ft_b200/build.py [--force] [--verbose]
"""
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))   # fasttree-artifact_b200/
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(ROOT, "include")
LIB_PATH = os.path.join(PKG_DIR, "libfasttree_b200.so")

SOURCES = ["ft_api.cu", "ft_planner.cu"]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return exe


STAMP_PATH = LIB_PATH + ".srchash"


def _source_digest():
    """SHA-256 over the names and contents of every file the library is built from.  Content, not time stamps:
    a copy of the tree (another machine, a container snapshot) keeps no usable modification times."""
    import hashlib
    h = hashlib.sha256()
    for folder in (CSRC, INCLUDE):
        for name in sorted(os.listdir(folder)):
            if name.endswith((".cu", ".cuh", ".h")):
                h.update(name.encode())
                with open(os.path.join(folder, name), "rb") as fh:
                    h.update(fh.read())
    h.update(os.environ.get("FT_B200_NVCC_FLAGS", "").encode())
    return h.hexdigest()


def _stale():
    """True when the library is missing or was built from other sources than the ones in the tree."""
    if not os.path.exists(LIB_PATH) or not os.path.exists(STAMP_PATH):
        return True
    with open(STAMP_PATH) as fh:
        return fh.read().strip() != _source_digest()


def build_library(force=False, verbose=False):
    """Compile every CUDA source for sm_100a into one shared library."""
    if not force and not _stale():
        return LIB_PATH
    digest = _source_digest()
    cmd = [_nvcc(), "-shared", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo",
           "-gencode", "arch=compute_100a,code=sm_100a",
           "-I", INCLUDE, "-I", CSRC, "-o", LIB_PATH]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += os.environ.get("FT_B200_NVCC_FLAGS", "").split()
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    cmd += ["-lcuda"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or res.returncode != 0:
        print(res.stdout)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout)
    with open(STAMP_PATH, "w") as fh:
        fh.write(digest + "\n")
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
