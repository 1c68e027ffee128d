"""Shared builders for the tests: trees, seeded inputs and golden-fixture access.

Everything here is test infrastructure; inputs come from the oracle's
restatement of the reference's draw order so that they are bit-identical to
what the golden fixtures were generated from.
"""
import hashlib
import json
import os

import numpy as np
import torch

from oracle import ref_inputs, ref_planner

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def ints(s):
    return [int(x) for x in s.split(",")]


def q_tiles_for_group(g):
    return [max(1, 64 // g), max(1, 16 // g)]


def sha_np(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def sha_t(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def load_planner_golden():
    with open(os.path.join(GOLDEN, "planner_golden.json")) as fh:
        return json.load(fh)


def tree_for_planner_key(key):
    """Rebuild the tree a planner-golden record was produced from.
    Returns (nodes, hq, hkv, kwargs for the planner)."""
    parts = key.split("|")
    tag = parts[-1]
    if parts[0].startswith("cfg5_d4_seed"):
        nodes = ref_inputs.random_tree(4, int(parts[0][len("cfg5_d4_seed"):]))
        hq, hkv = (int(x) for x in parts[1][1:].split("/"))
    else:
        if not parts[0].startswith("n"):
            parts = parts[1:]
        nodes = ref_inputs.layered_tree(ints(parts[0][1:]), ints(parts[1][1:]))
        hq, hkv = (int(x) for x in parts[2][1:].split("/"))
    kw = {"default": dict(abg=(0.66, 0.33, 0.1), split=[1024, 128]),
          "gamma10": dict(abg=(0.0, 0.0, 10.0), split=[81920, 81920]),
          "gamma-10": dict(abg=(0.0, 0.0, -10.0), split=[1024, 128])}[tag]
    return nodes, hq, hkv, kw


DECODE_CASES = {
    # name: (level sizes | None, level lens | random-tree kwargs, hq, hkv, d, dtype, seed, tsq, q_scale)
    "cfg1_fp32": ("1,4", "512,64", 8, 2, 128, "fp32", 1234, [16, 4], 1.0),
    "mini3_fp32": ("1,3,7", "70,33,21", 8, 2, 128, "fp32", 7, [16, 4], 1.0),
    "mini3_fp16": ("1,3,7", "70,33,21", 8, 2, 128, "fp16", 7, [16, 4], 1.0),
    "mini3_bf16_as_fp32": ("1,3,7", "70,33,21", 8, 2, 128, "bf16", 7, [16, 4], 0.5),
    "merge_d64_fp16": ("1,2,16", "8,40,19", 8, 2, 64, "fp16", 11, [16, 4], 1.0),
    "rand3_fp16": (None, dict(levels=3, seed=5, max_children=6, lam=2.0, len_lo=3, len_hi=90),
                   16, 4, 128, "fp16", 21, [16, 4], 1.0),
    "cfg2_fp16": ("1,64", "4096,256", 32, 8, 128, "fp16", 2024, [16, 4], 1.0),
}


def build_decode_case(name):
    """Tree + seeded tensors of a golden decode case, and the fixture itself.
    Returns dict(nodes, q, k, v, ptrs, batch, hq, hkv, d, dtype, tsq, gold)."""
    sizes, lens, hq, hkv, d, dt, seed, tsq, q_scale = DECODE_CASES[name]
    if sizes is None:
        kw = dict(lens)
        nodes = ref_inputs.random_tree(kw.pop("levels"), kw.pop("seed"), **kw)
    else:
        nodes = ref_inputs.layered_tree(ints(sizes), ints(lens))
    q, k, v, ptrs, batch = ref_inputs.draw_qkv(nodes, hq, hkv, d, DTYPES[dt], seed, q_scale)
    gold = dict(np.load(os.path.join(GOLDEN, f"decode_{name}.npz")))
    return dict(nodes=nodes, q=q, k=k, v=v, ptrs=ptrs, batch=batch, hq=hq, hkv=hkv, d=d,
                dtype=DTYPES[dt], tsq=list(tsq), gold=gold, name=name)


def oracle_params(hq, hkv, tsq, tsk=(32, 32), abg=(0.66, 0.33, 0.1)):
    p = ref_planner.OracleParams()
    p.set_values(*abg)
    p.set_q_tile_sizes(list(tsq))
    p.set_kv_tile_sizes(list(tsk))
    p.set_kv_group_num(hq // hkv)
    return p


TABLES = ["kv_entries", "kv_offs", "kv_lens", "q_entries", "q_offs", "q_lens",
          "r2v_entries", "r2v_offs", "r2v_lens"]
