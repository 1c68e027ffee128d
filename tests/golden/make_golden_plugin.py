#!/usr/bin/env python
"""Regenerate ``plugin_schedule_golden.npz`` from the reference's own SGLang-side
planner (sglang_v0.2.13_bench/fasttree_sglang_plugin_v0_2_13/schedule.py).

SGLang v0.2.13 is not installed, so the reference module is imported against the
stand-in host of tests/sglang_standin.py (registered under the ``sglang.*`` module
names it imports).  Only ``metadata.py`` and ``schedule.py`` of the reference
package are loaded - its ``__init__`` pulls in ``plugin.py``, which needs the
``nvtx`` package.  Everything runs on the CPU.

Usage:  python tests/golden/make_golden_plugin.py [--reference DIR]
"""
import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import sglang_standin  # noqa: E402

import plugin_cases  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("FASTTREE_REFERENCE_DIR"), required="FASTTREE_REFERENCE_DIR" not in os.environ,
                    help="checkout of PanZaifeng/FastTree-Artifact (or set FASTTREE_REFERENCE_DIR)")
    args = ap.parse_args()
    sglang_standin.install()
    ref_pkg = os.path.join(args.reference, "sglang_v0.2.13_bench", "fasttree_sglang_plugin_v0_2_13")
    pkg = types.ModuleType("fasttree_sglang_plugin_v0_2_13")
    pkg.__path__ = [ref_pkg]
    sys.modules["fasttree_sglang_plugin_v0_2_13"] = pkg
    import fasttree_sglang_plugin_v0_2_13.metadata as ref_md       # noqa
    import fasttree_sglang_plugin_v0_2_13.schedule as ref_sched    # noqa

    out = {}
    for name in plugin_cases.CASES:
        batch, _rows, hq, hkv = plugin_cases.build(name)
        md = ref_md.FastTreeMetadata(hq, hkv, 128, "cpu", max_vnodes=4096, max_vnode_to_q_entries=8192,
                                     max_batch_size=256)
        ref_sched.prepare_for_fasttree_meta(batch, md)
        nv = sum(md.phase_node_nums)
        bsz = len(batch.reqs)
        rows = int(md.req_to_vnode_lens[:bsz].sum())
        for key, n in (("vnode_to_kv_offs", nv), ("vnode_to_kv_lens", nv), ("vnode_to_q_offs", nv),
                       ("vnode_to_q_lens", nv), ("vnode_to_q_entries", rows), ("req_to_vnode_entries", rows),
                       ("req_to_vnode_offs", bsz), ("req_to_vnode_lens", bsz)):
            out[f"{name}/{key}"] = getattr(md, key)[:n].numpy().copy()
        out[f"{name}/phase_node_nums"] = np.asarray(md.phase_node_nums)
        out[f"{name}/phase_node_offsets"] = np.asarray(md.phase_node_offsets)
        out[f"{name}/phase_q_tile_sizes"] = np.asarray(md.phase_q_tile_sizes)
        out[f"{name}/phase_kv_tile_sizes"] = np.asarray(md.phase_kv_tile_sizes)
        out[f"{name}/req_last_vnodes"] = np.asarray(md.req_last_vnodes)
        print(name, "vnodes", nv, "rows", rows, "phases", md.phase_node_nums, md.phase_q_tile_sizes,
              md.phase_kv_tile_sizes)
    np.savez_compressed(os.path.join(HERE, "plugin_schedule_golden.npz"), **out)
    print("plugin_schedule_golden.npz written")


if __name__ == "__main__":
    main()
