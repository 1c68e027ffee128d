"""Pins the CPU oracle to fixtures produced by the reference's own code
(tests/golden/make_golden.py).  No GPU needed."""
import json
import os

import numpy as np
import pytest
import torch

import cases
from oracle import ref_attention, ref_inputs, ref_planner

PLANNER_GOLD = cases.load_planner_golden()


@pytest.mark.parametrize("key", sorted(PLANNER_GOLD))
def test_oracle_planner_matches_reference_tables(key):
    """Bit-exact: every int32 table, the node assignments, the phase split and the
    tile sizes the planner leaves in the parameter bag."""
    gold = PLANNER_GOLD[key]
    nodes, hq, hkv, kw = cases.tree_for_planner_key(key)
    batch = ref_inputs.assign_requests(nodes)
    ptrs = ref_inputs.kv_prefix_sums(nodes)
    p = cases.oracle_params(hq, hkv, cases.q_tiles_for_group(hq // hkv), abg=kw["abg"])
    plan = ref_planner.plan_reference(nodes, ptrs, batch, hkv, kw["split"], [132, 528], [132, 132], p)
    assert "".join(str(a) for a in plan.node_assignments) == gold["assign"]
    assert plan.phase_node_nums == gold["phase_node_nums"]
    assert plan.phase_node_offsets == gold["phase_node_offsets"]
    assert list(p.TSQs) == gold["tsq_after"] and list(p.TSKs) == gold["tsk_after"]
    for name in cases.TABLES:
        arr = getattr(plan, name)
        assert arr.dtype == np.int32
        assert arr.size == gold[name]["n"], name
        assert cases.sha_np(arr) == gold[name]["sha256"], name


SMALL = [n for n in cases.DECODE_CASES if n != "cfg2_fp16"]


@pytest.mark.parametrize("name", SMALL)
def test_oracle_inputs_and_plan_match_reference(name):
    """The oracle's seeded draws are the very tensors the reference drew (SHA-256),
    and the oracle plan equals the reference plan table by table."""
    c = cases.build_decode_case(name)
    gold = c["gold"]
    in_sha = json.loads(str(gold["in_sha"]))
    assert cases.sha_t(c["q"]) == in_sha["q"]
    assert cases.sha_t(c["k"]) == in_sha["k"]
    assert cases.sha_t(c["v"]) == in_sha["v"]
    p = cases.oracle_params(c["hq"], c["hkv"], c["tsq"])
    plan = ref_planner.plan_reference(c["nodes"], c["ptrs"], c["batch"], c["hkv"], [1024, 128],
                                      [132, 528], [132, 132], p)
    for tname in cases.TABLES:
        np.testing.assert_array_equal(getattr(plan, tname), gold[tname], err_msg=tname)
    assert plan.phase_node_nums == list(gold["phase_node_nums"])
    assert list(p.TSQs) == list(gold["tsq_after"])
    assert list(plan.node_assignments) == list(gold["assign"])


def _tol(name):
    # fp32 end to end: rounding-order differences only.  fp16 storage: the reference rounds
    # the probabilities to fp16 before P*V (fasttree.py:391), the oracle keeps them in fp32.
    return (2e-6, 2e-6) if "fp32" in name else (1e-3, 1e-3)


@pytest.mark.parametrize("name", SMALL)
def test_oracle_arithmetic_matches_reference_kernels(name):
    """Stage-1 partials, their LSE, and the merged output against what the
    reference's Triton kernels wrote (CPU interpreter)."""
    c = cases.build_decode_case(name)
    gold = c["gold"]
    q, k, v = c["q"], c["k"], c["v"]
    scale = 1.0 / c["d"] ** 0.5
    mid_o, mid_lse = ref_attention.stage1_partials(
        q, k, v, gold["kv_entries"], gold["kv_offs"], gold["kv_lens"],
        gold["q_entries"], gold["q_offs"], gold["q_lens"], scale)
    atol, rtol = _tol(name)
    np.testing.assert_allclose(mid_lse.numpy(), gold["mid_lse"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(mid_o.numpy(), gold["mid_o"], rtol=rtol, atol=atol)
    o, _ = ref_attention.stage2_merge(mid_o, mid_lse, gold["r2v_entries"], gold["r2v_offs"], gold["r2v_lens"])
    np.testing.assert_allclose(o.numpy(), gold["o"], rtol=rtol, atol=atol)
    # and the tree decomposition agrees with plain per-request attention over the path
    truth, lse = ref_attention.per_leaf_attention(c["nodes"], c["ptrs"], q, k, v, scale)
    np.testing.assert_allclose(o.numpy(), truth.numpy(), rtol=1e-5, atol=2e-6)
    np.testing.assert_allclose(truth.numpy(), gold["o"], rtol=rtol, atol=atol)


def test_merged_lse_matches_path_lse():
    c = cases.build_decode_case("rand3_fp16")
    gold = c["gold"]
    scale = 1.0 / c["d"] ** 0.5
    mid_o, mid_lse = ref_attention.stage1_partials(
        c["q"], c["k"], c["v"], gold["kv_entries"], gold["kv_offs"], gold["kv_lens"],
        gold["q_entries"], gold["q_offs"], gold["q_lens"], scale)
    _, lse = ref_attention.stage2_merge(mid_o, mid_lse, gold["r2v_entries"], gold["r2v_offs"], gold["r2v_lens"])
    _, lse_path = ref_attention.per_leaf_attention(c["nodes"], c["ptrs"], c["q"], c["k"], c["v"], scale)
    np.testing.assert_allclose(lse.numpy(), lse_path.numpy(), rtol=1e-5, atol=1e-5)


@pytest.mark.skipif(not os.path.exists(os.path.join(cases.GOLDEN, "decode_cfg2_fp16.npz")),
                    reason="full-size fixture not generated")
def test_full_size_fp16_case_against_reference_output():
    """cfg2 at full size: the oracle's ground truth vs the reference kernels' fp16 output."""
    c = cases.build_decode_case("cfg2_fp16")
    gold = c["gold"]
    in_sha = json.loads(str(gold["in_sha"]))
    assert cases.sha_t(c["k"]) == in_sha["k"] and cases.sha_t(c["q"]) == in_sha["q"]
    truth, _ = ref_attention.per_leaf_attention(c["nodes"], c["ptrs"], c["q"], c["k"], c["v"],
                                                1.0 / 128 ** 0.5)
    err = (truth - torch.from_numpy(gold["o"].astype(np.float32))).abs().max().item()
    assert err <= 2e-3, err


def test_tree_file_round_trip(tmp_path):
    nodes = ref_inputs.layered_tree([1, 3, 7], [70, 33, 21])
    path = tmp_path / "t.txt"
    ref_inputs.write_tree_file(nodes, path)
    back = ref_inputs.read_tree_file(path)
    assert [(n.parent, n.id, n.seqlen, n.num_children) for n in back] == \
           [(n.parent, n.id, n.seqlen, n.num_children) for n in nodes]
    assert path.read_text().splitlines()[0] == "11"
