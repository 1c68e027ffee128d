#!/usr/bin/env python
"""Regenerate the golden fixtures in this directory from the reference's own code.

Needs a checkout of PanZaifeng/FastTree-Artifact (``--reference DIR`` or the
environment variable FASTTREE_REFERENCE_DIR); it is imported read-only and never copied.  The reference's
planner and Triton kernels (kernel_bench/fasttree.py) run on the CPU: Triton is
put in interpreter mode and the module's ``torch`` global is replaced by a
forwarding object whose ``device(...)`` always answers ``cpu`` (the planner
hard-codes ``with torch.device("cuda")`` at fasttree.py:265).

Outputs (all small, committed):
  planner_golden.json   node assignments, phase split, effective tile sizes and
                        SHA-256 of every int32 table, for the 15 tree shapes x 3
                        head configurations of kernel_bench/run_benchmark.sh:5-27,
                        their two ablations (:67-81), and the benchmark
                        configurations of this repository.
  decode_*.npz          plan tables + O / mid_o / mid_lse written by the
                        reference kernels on seeded inputs (inputs are
                        reproduced from the seed; their SHA-256 is stored).

Usage:  python tests/golden/make_golden.py --reference DIR [--with-cfg2]
"""
import argparse
import contextlib
import hashlib
import io
import json
import os
import sys
import tempfile
import time

os.environ["TRITON_INTERPRET"] = "1"          # must precede the first triton import

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import ref_inputs  # noqa: E402  (tree builders only; the arithmetic below is the reference's)


class _CpuTorch:
    """Forwards to torch, but every ``device(...)`` is the CPU."""

    def __getattr__(self, name):
        return getattr(torch, name)

    @staticmethod
    def device(*_a, **_k):
        return torch.device("cpu")


def load_reference(ref_dir):
    kb = os.path.join(ref_dir, "kernel_bench")
    sys.path.insert(0, kb)
    import fasttree as ref_ft            # noqa
    import kv_tree_simple as ref_tree    # noqa
    import flash_attn_wrap as ref_in     # noqa
    import tree_generation as ref_gen    # noqa
    ref_ft.torch = _CpuTorch()
    return ref_ft, ref_tree, ref_in, ref_gen


def sha(arr):
    return hashlib.sha256(np.ascontiguousarray(arr).tobytes()).hexdigest()


def tsha(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


SHAPES_15 = [  # kernel_bench/run_benchmark.sh:5-21
    ("1,2,64", "8,256,32"), ("1,4,256", "8,256,32"), ("1,4,8,256", "8,256,256,32"),
    ("1,256", "256,32"), ("1,1024", "2048,32"), ("1,16,64", "1024,256,32"),
    ("1,4,16,512", "1024,256,128,32"), ("1,4,16,64,256,1024", "256,8,256,64,32,256"),
    ("1,10", "4000,400"),
    ("1,2,4,8,16,32,64,128,1024", "16,16,16,16,16,16,16,16,16"),
    ("1,2,4,8,16,32,64,128,1024", "256,128,64,16,16,16,16,16,16"),
    ("1,8,16,32,64,128,1024", "256,128,64,16,16,16,16"),
    ("1,8,16,32,64,256,1024", "256,128,64,16,16,16,16"),
    ("1,16,32,64,128,1024", "256,128,64,16,16,16"),
    ("1,16,32,64,256,1024", "256,128,64,16,16,16"),
]
HEADS_3 = [(16, 1), (32, 8), (32, 32)]       # run_benchmark.sh:23-27
BENCH_CFGS = [                                # this repository's benchmark configurations
    ("cfg1", "1,4", "512,64", 8, 2), ("cfg2", "1,64", "4096,256", 32, 8),
    ("cfg3", "1,16,256", "2048,512,64", 32, 8), ("cfg3_tp8", "1,16,256", "2048,512,64", 4, 1),
    ("cfg4", "1,1024", "16384,32", 64, 8), ("cfg4_tp8", "1,1024", "16384,32", 8, 1),
]


def ints(s):
    return [int(x) for x in s.split(",")]


def ref_tree_from_spec(ref_tree, ref_gen, sizes, lens, tmpdir):
    """Tree through the reference's generator, writer and reader."""
    nodes = ref_gen.generate_tree(ints(sizes), ints(lens))
    path = os.path.join(tmpdir, "t.txt")
    ref_gen.save_tree(nodes, path)
    return ref_tree.retrive_from_file(path)


def ref_tree_from_oracle_nodes(ref_tree, onodes, tmpdir):
    path = os.path.join(tmpdir, "r.txt")
    ref_inputs.write_tree_file(onodes, path)
    return ref_tree.retrive_from_file(path)


def fill_requests(tree):
    """Request assignment without drawing tensors (flash_attn_wrap.py:24-33)."""
    n = 0
    for nd in tree:
        nd.requests = []
    for nd in tree:
        if nd.num_children == 0:
            cur = nd.id
            while cur != -1:
                tree[cur].requests.append(n)
                cur = tree[cur].parent
            n += 1
    ptrs = [0]
    for nd in tree:
        ptrs.append(ptrs[-1] + nd.seqlen)
    return n, ptrs


def run_ref_planner(ref_ft, tree, ptrs, batch, hq, hkv, tsq, tsk=(32, 32), abg=(0.66, 0.33, 0.1),
                    split=(1024, 128), th1=(132, 528), th2=(132, 132), head_dim=128):
    """Reference planner with the micro-benchmark's CLI defaults (benchmark.py:246-253)."""
    params = ref_ft.FastTreeParams()
    params.set_values(*abg)
    params.set_q_tile_sizes(list(tsq))
    params.set_kv_tile_sizes(list(tsk))
    params.set_kv_group_num(hq // hkv)
    with contextlib.redirect_stdout(io.StringIO()):
        aux, assign = ref_ft.fasttree_preparation(
            tree, ptrs, batch, hq, hkv, head_dim, list(split), list(th1), list(th2), params)
    return aux, assign, params


AUX_NAMES = ["kv_entries", "kv_offs", "kv_lens", "q_entries", "q_offs", "q_lens",
             "r2v_entries", "r2v_offs", "r2v_lens"]


def planner_record(aux, assign, params):
    rec = {"assign": "".join(str(a) for a in assign),
           "phase_node_nums": list(aux[11]), "phase_node_offsets": list(aux[12]),
           "tsq_after": list(params.TSQs), "tsk_after": list(params.TSKs)}
    for name, t in zip(AUX_NAMES, aux[:9]):
        a = t.numpy().astype(np.int32)
        rec[name] = {"n": int(a.size), "sha256": sha(a)}
    return rec


def q_tiles_for_group(g):
    # run_benchmark.sh:46-53 for ratios 1/4/16; the plugin rule 64//G,16//G elsewhere
    return [max(1, 64 // g), max(1, 16 // g)]


def make_planner_golden(ref_ft, ref_tree, ref_gen, tmpdir):
    out = {}
    for sizes, lens in SHAPES_15:
        for hq, hkv in HEADS_3:
            tsq = q_tiles_for_group(hq // hkv)
            for tag, kw in (("default", {}),
                            ("gamma10", dict(abg=(0.0, 0.0, 10.0), split=(81920, 81920))),
                            ("gamma-10", dict(abg=(0.0, 0.0, -10.0), split=(1024, 128)))):
                tree = ref_tree_from_spec(ref_tree, ref_gen, sizes, lens, tmpdir)
                batch, ptrs = fill_requests(tree)
                aux, assign, params = run_ref_planner(ref_ft, tree, ptrs, batch, hq, hkv, tsq, **kw)
                out[f"n{sizes}|c{lens}|h{hq}/{hkv}|{tag}"] = planner_record(aux, assign, params)
    for name, sizes, lens, hq, hkv in BENCH_CFGS:
        tree = ref_tree_from_spec(ref_tree, ref_gen, sizes, lens, tmpdir)
        batch, ptrs = fill_requests(tree)
        aux, assign, params = run_ref_planner(ref_ft, tree, ptrs, batch, hq, hkv,
                                              q_tiles_for_group(hq // hkv))
        out[f"{name}|n{sizes}|c{lens}|h{hq}/{hkv}|default"] = planner_record(aux, assign, params)
    for seed in (0, 1, 2):
        onodes = ref_inputs.random_tree(4, seed)
        tree = ref_tree_from_oracle_nodes(ref_tree, onodes, tmpdir)
        batch, ptrs = fill_requests(tree)
        aux, assign, params = run_ref_planner(ref_ft, tree, ptrs, batch, 32, 8, [16, 4])
        out[f"cfg5_d4_seed{seed}|h32/8|default"] = planner_record(aux, assign, params)
    with open(os.path.join(HERE, "planner_golden.json"), "w") as fh:
        json.dump(out, fh, indent=0, sort_keys=True)
    print("planner_golden.json:", len(out), "records")


def run_ref_decode(ref_ft, ref_in, tree, hq, hkv, d, dtype, seed, tsq, q_scale=1.0,
                   compute_dtype=None, **plan_kw):
    """Seeded inputs through the reference's qkv_preparation (CPU), plan through
    the reference planner, output through the reference kernels (interpreter).
    ``compute_dtype``: run the kernels on an exact up-cast of the drawn tensors
    (used for bf16, which the interpreter mishandles)."""
    for nd in tree:
        nd.requests = []
    torch.manual_seed(seed)
    q, _kc, _vc, _sl, k_tree, v_tree, ptrs = ref_in.qkv_preparation(tree, hq, hkv, d, "cpu", dtype)
    del _kc, _vc
    if q_scale != 1.0:
        q = (q.float() * q_scale).to(dtype)
    batch = q.shape[0]
    aux, assign, params = run_ref_planner(ref_ft, tree, ptrs, batch, hq, hkv, tsq, head_dim=d, **plan_kw)
    in_sha = {"q": tsha(q), "k": tsha(k_tree), "v": tsha(v_tree)}
    if compute_dtype is not None:
        q, k_tree, v_tree = q.to(compute_dtype), k_tree.to(compute_dtype), v_tree.to(compute_dtype)
    o = torch.empty_like(q)
    mid_o, mid_lse = aux[9], aux[10]
    mid_o.fill_(float("nan"))
    mid_lse.fill_(float("nan"))
    # The tile sizes the planner settled on (it may overwrite them, fasttree.py:181-186)
    ref_ft.fasttree_decode(q, k_tree, v_tree, o, *aux, list(params.TSQs), list(params.TSKs),
                           1.0 / d ** 0.5)
    rec = {name: t.numpy().astype(np.int32) for name, t in zip(AUX_NAMES, aux[:9])}
    rec.update(phase_node_nums=np.asarray(aux[11]), phase_node_offsets=np.asarray(aux[12]),
               tsq_after=np.asarray(params.TSQs), tsk_after=np.asarray(params.TSKs),
               assign=np.asarray(assign, dtype=np.int8),
               o=o.float().numpy(), mid_o=mid_o.numpy(), mid_lse=mid_lse.numpy(),
               in_sha=np.asarray(json.dumps(in_sha)), seed=np.asarray(seed),
               heads=np.asarray([hq, hkv, d]), q_scale=np.asarray(q_scale))
    return rec


def save_decode(name, rec, keep_mid=True):
    if not keep_mid:
        rec = {k: v for k, v in rec.items() if k not in ("mid_o",)}
    np.savez_compressed(os.path.join(HERE, f"decode_{name}.npz"), **rec)
    print(f"decode_{name}.npz written")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("FASTTREE_REFERENCE_DIR"), required="FASTTREE_REFERENCE_DIR" not in os.environ,
                    help="checkout of PanZaifeng/FastTree-Artifact (or set FASTTREE_REFERENCE_DIR)")
    ap.add_argument("--with-cfg2", action="store_true", help="also the full-size fp16 case (minutes)")
    ap.add_argument("--skip-planner", action="store_true")
    args = ap.parse_args()
    ref_ft, ref_tree, ref_in, ref_gen = load_reference(args.reference)
    with tempfile.TemporaryDirectory() as tmp:
        if not args.skip_planner:
            make_planner_golden(ref_ft, ref_tree, ref_gen, tmp)

        t0 = time.time()
        tree = ref_tree_from_spec(ref_tree, ref_gen, "1,4", "512,64", tmp)
        save_decode("cfg1_fp32", run_ref_decode(ref_ft, ref_in, tree, 8, 2, 128, torch.float32, 1234, [16, 4]))

        tree = ref_tree_from_spec(ref_tree, ref_gen, "1,3,7", "70,33,21", tmp)
        save_decode("mini3_fp32", run_ref_decode(ref_ft, ref_in, tree, 8, 2, 128, torch.float32, 7, [16, 4]))
        tree = ref_tree_from_spec(ref_tree, ref_gen, "1,3,7", "70,33,21", tmp)
        save_decode("mini3_fp16", run_ref_decode(ref_ft, ref_in, tree, 8, 2, 128, torch.float16, 7, [16, 4]))
        tree = ref_tree_from_spec(ref_tree, ref_gen, "1,3,7", "70,33,21", tmp)
        save_decode("mini3_bf16_as_fp32", run_ref_decode(ref_ft, ref_in, tree, 8, 2, 128, torch.bfloat16, 7,
                                                         [16, 4], q_scale=0.5, compute_dtype=torch.float32))
        # two children carry the short root's KV (assignment 1) on this one; head_dim 64
        tree = ref_tree_from_spec(ref_tree, ref_gen, "1,2,16", "8,40,19", tmp)
        save_decode("merge_d64_fp16", run_ref_decode(ref_ft, ref_in, tree, 8, 2, 64, torch.float16, 11, [16, 4]))
        # irregular tree, small contexts
        onodes = ref_inputs.random_tree(3, 5, max_children=6, lam=2.0, len_lo=3, len_hi=90)
        tree = ref_tree_from_oracle_nodes(ref_tree, onodes, tmp)
        save_decode("rand3_fp16", run_ref_decode(ref_ft, ref_in, tree, 16, 4, 128, torch.float16, 21, [16, 4]))
        print("small decode goldens: %.1f s" % (time.time() - t0))

        if args.with_cfg2:
            t0 = time.time()
            tree = ref_tree_from_spec(ref_tree, ref_gen, "1,64", "4096,256", tmp)
            rec = run_ref_decode(ref_ft, ref_in, tree, 32, 8, 128, torch.float16, 2024, [16, 4])
            rec["o"] = rec["o"].astype(np.float16)         # the reference wrote fp16; keep it exact and small
            rec["mid_lse"] = rec["mid_lse"].astype(np.float32)
            save_decode("cfg2_fp16", rec, keep_mid=False)
            print("cfg2: %.1f s" % (time.time() - t0))


if __name__ == "__main__":
    main()
