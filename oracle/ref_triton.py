"""The reference's own Triton kernels as a GPU-side checker and timed baseline
(TEST INFRASTRUCTURE ONLY - nothing in the shipped package imports this).

``oracle/stage_ref.py`` places the unmodified ``kernel_bench/fasttree.py`` of
the reference under ``oracle/_ref/`` (git-ignored).  This module imports that
file under a private module name (the product ships a drop-in that is also
called ``fasttree``), plans a tree with the reference's planner and command-line
defaults, and runs the reference's ``fasttree_decode`` - Triton kernels JIT
compiled for the GPU at hand - on caller-supplied tensors.

Settings are the reference's own:
  * planner constants and thresholds       kernel_bench/benchmark.py:246-253
  * request tiles ``64 // G, 16 // G``      kernel_bench/run_benchmark.sh:46-53
  * KV tiles ``32, 32``                     kernel_bench/benchmark.py:250
  * call pattern                            kernel_bench/benchmark.py:88-128
"""
import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref", "kernel_bench")
_MODULE_NAME = "_fasttree_reference_triton"

ALPHA, BETA, GAMMA = 0.66, 0.33, 0.1
KV_TILES = [32, 32]
KV_SPLIT_SIZES = [1024, 128]
PARA_THRESHS1 = [132, 528]
PARA_THRESHS2 = [132, 132]


def q_tiles(group):
    """run_benchmark.sh:46-53 lists 64,16 / 16,4 / 4,1 for G = 1 / 4 / 16: 64 // G and 16 // G."""
    return [max(1, 64 // group), max(1, 16 // group)]


def availability():
    """(True, "") when the staged reference can be imported here, else (False, reason)."""
    path = os.path.join(REF_DIR, "fasttree.py")
    if not os.path.isfile(path):
        return False, "oracle/_ref is not staged (run oracle/stage_ref.py against a reference checkout)"
    try:
        import triton  # noqa: F401
    except Exception as exc:  # pragma: no cover - triton ships with the image
        return False, f"triton cannot be imported: {exc}"
    return True, ""


def load():
    """Import oracle/_ref/kernel_bench/fasttree.py under a private name."""
    if _MODULE_NAME in sys.modules:
        return sys.modules[_MODULE_NAME]
    ok, why = availability()
    if not ok:
        raise RuntimeError(why)
    spec = importlib.util.spec_from_file_location(_MODULE_NAME, os.path.join(REF_DIR, "fasttree.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[_MODULE_NAME] = mod          # triton's JIT looks the module up by name
    spec.loader.exec_module(mod)
    return mod


class _Node:
    """The five fields the reference planner reads (kernel_bench/kv_tree_simple.py:4-10)."""

    def __init__(self, src):
        self.parent, self.id, self.seqlen = int(src.parent), int(src.id), int(src.seqlen)
        self.num_children = int(src.num_children)
        self.requests = list(src.requests)


class ReferenceRun:
    """A tree planned by the reference planner for the current CUDA device, ready
    to decode with the reference kernels."""

    def __init__(self, nodes, ptrs, batch, hq, hkv, head_dim):
        import torch
        self.mod = load()
        self.hq, self.hkv, self.d, self.batch = hq, hkv, head_dim, batch
        group = hq // hkv
        self.params = self.mod.FastTreeParams()
        self.params.set_values(ALPHA, BETA, GAMMA)
        self.params.set_q_tile_sizes(q_tiles(group))
        self.params.set_kv_tile_sizes(list(KV_TILES))
        self.params.set_kv_group_num(group)
        tree = [_Node(n) for n in nodes]
        self.aux, self.assignments = self.mod.fasttree_preparation(
            tree, list(ptrs), batch, hq, hkv, head_dim, list(KV_SPLIT_SIZES), list(PARA_THRESHS1),
            list(PARA_THRESHS2), self.params)
        # The planner may settle on one tile size for both phases (kernel_bench/fasttree.py:180-186) and stores
        # that in ``params``; kernel_bench/benchmark.py:114-124 still hands the caller's original lists to the
        # decode call.  The planner's lists are used here: they always fit the plan (the caller's can truncate
        # a request tile) and are never the slower choice, so the baseline is not put at a disadvantage.
        self.caller_tsq, self.caller_tsk = q_tiles(group), list(KV_TILES)
        self.tsq, self.tsk = list(self.params.TSQs), list(self.params.TSKs)
        self.scale = 1.0 / head_dim ** 0.5
        self.vnodes = int(self.aux[1].numel())
        self.partial_rows = int(self.aux[3].numel())
        torch.cuda.synchronize()

    def decode(self, q, k, v, o):
        """One decode step with the reference's kernels, on torch's current stream."""
        self.mod.fasttree_decode(q, k, v, o, *self.aux, self.tsq, self.tsk, self.scale)
        return o
