"""Host planner tests (CPU only): the reference-compatible splitter against the
reference's own tables, and structural properties of the B200 splitter."""
import numpy as np
import pytest

import cases
from oracle import ref_inputs

import fasttree                      # the drop-in module (fasttree-artifact_b200/kernel_bench)
from ft_b200 import planner
from kv_tree_simple import KVTreeNode, retrive_from_file, validate_tree
import tree_generation

PLANNER_GOLD = cases.load_planner_golden()


def product_tree(onodes):
    """Oracle tree -> the product's node type, with requests assigned by the
    reference rule (leaves in id order)."""
    out = [KVTreeNode(n.parent, n.id, n.seqlen, n.num_children) for n in onodes]
    nreq = 0
    for nd in out:
        if nd.num_children == 0:
            cur = nd.id
            while cur != -1:
                out[cur].requests.append(nreq)
                cur = out[cur].parent
            nreq += 1
    ptrs = [0]
    for nd in out:
        ptrs.append(ptrs[-1] + nd.seqlen)
    return out, nreq, ptrs


def make_params(hq, hkv, tsq, abg=(0.66, 0.33, 0.1), planner_name="reference"):
    p = fasttree.FastTreeParams()
    p.set_values(*abg)
    p.set_q_tile_sizes(list(tsq))
    p.set_kv_tile_sizes([32, 32])
    p.set_kv_group_num(hq // hkv)
    p.set_planner(planner_name)
    return p


@pytest.mark.parametrize("key", sorted(PLANNER_GOLD))
def test_reference_mode_is_bit_identical_to_reference_planner(key):
    gold = PLANNER_GOLD[key]
    onodes, hq, hkv, kw = cases.tree_for_planner_key(key)
    tree, batch, ptrs = product_tree(onodes)
    p = make_params(hq, hkv, cases.q_tiles_for_group(hq // hkv), abg=kw["abg"])
    plan = fasttree.build_plan(tree, ptrs, batch, hq, hkv, 128, kw["split"], [132, 528], [132, 132], p)
    assert "".join(map(str, plan.node_assignments)) == gold["assign"]
    assert plan.phase_node_nums == gold["phase_node_nums"]
    assert plan.phase_node_offsets == gold["phase_node_offsets"]
    assert list(p.TSQs) == gold["tsq_after"] and list(p.TSKs) == gold["tsk_after"]
    names = ["kv_entries", "kv_offs", "kv_lens", "q_entries", "q_offs", "q_lens",
             "r2v_entries", "r2v_offs", "r2v_lens"]
    for name, arr in zip(names, plan.tables()):
        assert arr.dtype == np.int32, name
        assert arr.size == gold[name]["n"], name
        assert cases.sha_np(arr) == gold[name]["sha256"], name


def check_plan_covers_every_path_once(tree, ptrs, batch, plan):
    """Every request must see each token of its root->leaf path in exactly one
    of its partial rows, and nothing else."""
    kv_entries = plan.vnode_to_kv_entries
    ranges = plan.vnode_q_kv_ranges          # groups of short nodes: a row sees only [begin, end) of its chunk
    n_big = plan.phase_node_nums[0]
    row_tokens = {}
    for vn in range(plan.num_vnodes):
        ko, kl = int(plan.vnode_to_kv_offs[vn]), int(plan.vnode_to_kv_lens[vn])
        qo, ql = int(plan.vnode_to_q_offs[vn]), int(plan.vnode_to_q_lens[vn])
        assert kl > 0 and ql > 0
        toks = kv_entries[ko:ko + kl]
        assert toks.min() >= 0
        for row in range(qo, qo + ql):
            assert row not in row_tokens, "two vnodes write the same partial row"
            if ranges is None:
                row_tokens[row] = toks
            else:
                b, e = int(ranges[row, 0]), int(ranges[row, 1])
                assert 0 <= b < e <= kl
                if vn >= n_big:                  # the few-row kernels do not look at the ranges
                    assert (b, e) == (0, kl)
                row_tokens[row] = toks[b:e]
    assert len(row_tokens) == plan.num_partial_rows
    paths = {}
    for nd in tree:
        if nd.num_children == 0:
            chain, cur = [], nd.id
            while cur != -1:
                chain.append(cur)
                cur = tree[cur].parent
            paths[nd.requests[0]] = chain
    for r in range(batch):
        off, n = int(plan.req_to_vnode_offs[r]), int(plan.req_to_vnode_lens[r])
        rows = plan.req_to_vnode_entries[off:off + n]
        assert all(plan.vnode_to_q_entries[row] == r for row in rows)
        seen = np.sort(np.concatenate([row_tokens[int(row)] for row in rows]))
        want = np.sort(np.concatenate([np.arange(ptrs[n_], ptrs[n_ + 1]) for n_ in paths[r]]))
        np.testing.assert_array_equal(seen, want)
    # phases: a stable split on the small request tile, contiguous ranges
    n0, n1 = plan.phase_node_nums
    assert plan.phase_node_offsets == [0, n0] and n0 + n1 == plan.num_vnodes


B200_TREES = {
    "cfg1": ([1, 4], [512, 64], 8, 2),
    "cfg2": ([1, 64], [4096, 256], 32, 8),
    "cfg3": ([1, 16, 256], [2048, 512, 64], 32, 8),
    "cfg3_one_kv_head": ([1, 16, 256], [2048, 512, 64], 4, 1),
    "deep_short": ([1, 2, 4, 8, 16, 32, 64], [16, 16, 16, 16, 16, 16, 16], 32, 32),
    "single_node": ([1], [300], 8, 8),
    "one_token_nodes": ([1, 3, 9], [1, 1, 1], 16, 4),
}


@pytest.mark.parametrize("name", sorted(B200_TREES))
def test_b200_plan_is_valid_and_deterministic(name):
    sizes, lens, hq, hkv = B200_TREES[name]
    plans = []
    for _ in range(2):
        tree, batch, ptrs = product_tree(ref_inputs.layered_tree(sizes, lens))
        p = make_params(hq, hkv, [16, 4], planner_name="b200")
        plan = fasttree.build_plan(tree, ptrs, batch, hq, hkv, 128, [1024, 128], [132, 528], [132, 132], p)
        check_plan_covers_every_path_once(tree, ptrs, batch, plan)
        plans.append(plan)
    for a, b in zip(plans[0].tables(), plans[1].tables()):
        np.testing.assert_array_equal(a, b)
    assert plans[0].node_assignments == plans[1].node_assignments
    group = hq // hkv
    assert int(plans[0].vnode_to_q_lens.max()) * group <= max(128, group)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_b200_plan_on_random_trees(seed):
    tree, batch, ptrs = product_tree(ref_inputs.random_tree(4, seed, len_lo=1, len_hi=300))
    p = make_params(32, 8, [16, 4], planner_name="b200")
    plan = fasttree.build_plan(tree, ptrs, batch, 32, 8, 128, [1024, 128], [132, 528], [132, 132], p)
    check_plan_covers_every_path_once(tree, ptrs, batch, plan)


def _same_plan(a, b):
    for x, y, name in zip(a.tables(), b.tables(), cases.TABLES):
        np.testing.assert_array_equal(x, y, err_msg=name)
    assert (a.vnode_q_kv_ranges is None) == (b.vnode_q_kv_ranges is None)
    if a.vnode_q_kv_ranges is not None:
        np.testing.assert_array_equal(a.vnode_q_kv_ranges, b.vnode_q_kv_ranges)
    assert list(a.node_assignments) == list(b.node_assignments)
    assert list(a.phase_node_nums) == list(b.phase_node_nums)
    assert list(a.phase_node_offsets) == list(b.phase_node_offsets)
    assert list(a.phase_q_tile_sizes) == list(b.phase_q_tile_sizes)
    assert a.info["target_bytes"] == b.info["target_bytes"] and a.info["vnodes"] == b.info["vnodes"]


NATIVE_TREES = dict(B200_TREES)
NATIVE_TREES.update({
    "cfg4": ([1, 1024], [16384, 32], 64, 8),
    "mha_chain": ([1, 1, 1, 4], [100, 7, 300, 20], 8, 8),
    "gqa16": ([1, 2, 64], [8, 256, 32], 16, 1),
})


@pytest.mark.parametrize("name", sorted(NATIVE_TREES))
@pytest.mark.parametrize("head_dim", [64, 128])
def test_native_splitter_matches_the_python_specification(name, head_dim):
    """ft_plan_b200_build (C++, in the shared library; host code only) against ft_b200.planner.plan_b200."""
    sizes, lens, hq, hkv = NATIVE_TREES[name]
    tree, batch, ptrs = product_tree(ref_inputs.layered_tree(sizes, lens))
    pa, pb = make_params(hq, hkv, [16, 4], planner_name="b200"), make_params(hq, hkv, [16, 4], planner_name="b200")
    spec = planner.plan_b200(tree, ptrs, batch, hq, hkv, head_dim, pa)
    native = planner.plan_b200_native(tree, ptrs, batch, hq, hkv, head_dim, pb)
    _same_plan(spec, native)
    assert list(pa.TSQs) == list(pb.TSQs) and list(pa.TSKs) == list(pb.TSKs)


@pytest.mark.parametrize("seed", range(8))
def test_native_splitter_matches_on_random_trees_and_models(seed):
    from dataclasses import replace
    rng = np.random.default_rng(seed)
    tree, batch, ptrs = product_tree(ref_inputs.random_tree(3 + seed % 3, seed, max_children=6 + seed, lam=2.0 + seed % 3,
                                                            len_lo=1, len_hi=40 * (1 + seed)))
    hq, hkv = [(32, 8), (8, 8), (16, 1), (64, 8)][seed % 4]
    model = replace(planner.B200Model(), waves=float(rng.choice([0.5, 1.0, 2.0, 3.0])), min_chunk=int(rng.choice([64, 128, 256])),
                    rows_per_cta=int(rng.choice([64, 128])), ridge_flop_per_byte=float(rng.choice([90.0, 360.0])),
                    group_member_tokens=int(rng.choice([0, 48, 128, 256])), group_min_members=int(rng.choice([2, 6, 10])))
    pa, pb = make_params(hq, hkv, [16, 4], planner_name="b200"), make_params(hq, hkv, [16, 4], planner_name="b200")
    spec = planner.plan_b200(tree, ptrs, batch, hq, hkv, 128, pa, model=model)
    native = planner.plan_b200_native(tree, ptrs, batch, hq, hkv, 128, pb, model=model)
    _same_plan(spec, native)
    check_plan_covers_every_path_once(tree, ptrs, batch, native)


@pytest.mark.parametrize("name", ["cfg2", "cfg3"])
def test_last_round_of_the_schedule_is_halved(name):
    """planner.b200_split_tail: the benchmark trees whose CTAs fill 2.05 / 1.3 rounds of the GPU get the chunks that end
    their last round halved (simulated makespan 24 -> 22 and 34 -> 30 tile times), identically in the native splitter."""
    sizes, lens, makespans, halved = {"cfg2": ([1, 64], [4096, 256], (24, 22), 14),
                                      "cfg3": ([1, 16, 256], [2048, 512, 64], (34, 30), 6)}[name]
    tree, batch, ptrs = product_tree(ref_inputs.layered_tree(sizes, lens))
    p = make_params(32, 8, [16, 4], planner_name="b200")
    m = planner.b200_model_for(p, 128)
    vnodes, _, q_tile, small_tile, target = planner.b200_virtual_nodes(
        tree, 32, 8, 128, m, lambda a, i: planner._chain_ranges(tree, ptrs, a, i))
    vnodes = planner.b200_group_short_nodes(vnodes, q_tile, small_tile, m, int(target // (2 * 128 * m.elem_bytes)))
    slots = 2 * 148 // 8
    before = planner.b200_simulated_schedule(vnodes, q_tile, small_tile, m, slots)
    cut = planner.b200_split_tail(vnodes, q_tile, small_tile, m, 8)
    after = planner.b200_simulated_schedule(cut, q_tile, small_tile, m, slots)
    assert (before[0], after[0]) == makespans
    changed = [(a.kv_split, b.kv_split) for a, b in zip(vnodes, cut) if a.kv_split != b.kv_split]
    assert len(changed) == halved and all(new * 2 == old for old, new in changed)
    assert all(a.row_ranges is None for a, b in zip(vnodes, cut) if a.kv_split != b.kv_split)   # groups stay whole
    pa, pb = make_params(32, 8, [16, 4], planner_name="b200"), make_params(32, 8, [16, 4], planner_name="b200")
    spec = planner.plan_b200(tree, ptrs, batch, 32, 8, 128, pa)
    native = planner.plan_b200_native(tree, ptrs, batch, 32, 8, 128, pb)
    _same_plan(spec, native)
    check_plan_covers_every_path_once(tree, ptrs, batch, native)
    # on a GPU with room for every task at once the step lasts as long as its longest task: the short ones stay whole
    from dataclasses import replace
    roomy = planner.b200_split_tail(vnodes, q_tile, small_tile, replace(m, num_sms=4 * 148), 8)
    longest = max(v.kv_split for v in vnodes)
    assert all(a.kv_split == b.kv_split for a, b in zip(vnodes, roomy) if a.kv_split < longest)


def test_groups_grow_to_keep_the_step_in_one_round():
    """cfg3 on a 4-KV-head shard: at the default token target the step is 32 + 16 plain tasks and 32 groups of 8 leaves,
    80 tasks on 74 slots; the target grows so that 26 groups of 10 leaves fill the round exactly."""
    tree, batch, ptrs = product_tree(ref_inputs.layered_tree([1, 16, 256], [2048, 512, 64]))
    plans = []
    for native in (False, True):
        p = make_params(16, 4, [16, 4], planner_name="b200")
        p.native_planner = native
        plans.append(fasttree.build_plan(tree, ptrs, batch, 16, 4, 128, [1024, 128], [132, 528], [132, 132], p))
    _same_plan(*plans)
    plan = plans[0]
    check_plan_covers_every_path_once(tree, ptrs, batch, plan)
    assert plan.num_vnodes == 2 * 148 // 4
    group = plan.vnode_to_q_lens == 10                        # ten single-request leaves, 64 tokens each
    assert group.sum() == 25 and (plan.vnode_to_kv_lens[group] == 640).all()


@pytest.mark.parametrize("seed", range(6))
def test_native_splitter_matches_on_small_gpus(seed):
    """Few task slots put most random trees into several rounds, which is where the last-round pass acts."""
    from dataclasses import replace
    rng = np.random.default_rng(100 + seed)
    tree, batch, ptrs = product_tree(ref_inputs.random_tree(3 + seed % 3, 100 + seed, max_children=5 + 2 * seed, lam=3.0,
                                                            len_lo=1, len_hi=int(rng.choice([300, 2048]))))
    hq, hkv = [(32, 8), (8, 8), (16, 1)][seed % 3]
    model = replace(planner.B200Model(), num_sms=int(rng.choice([2, 4, 16])), rows_per_cta=128,
                    group_member_tokens=int(rng.choice([0, 128])))
    pa, pb = make_params(hq, hkv, [16, 4], planner_name="b200"), make_params(hq, hkv, [16, 4], planner_name="b200")
    spec = planner.plan_b200(tree, ptrs, batch, hq, hkv, 128, pa, model=model)
    native = planner.plan_b200_native(tree, ptrs, batch, hq, hkv, 128, pb, model=model)
    _same_plan(spec, native)
    check_plan_covers_every_path_once(tree, ptrs, batch, native)


@pytest.mark.parametrize("block", range(4))
def test_native_splitter_matches_on_many_shapes(block):
    """Sweep of tree depths, fan-outs, node lengths, head counts and slot counts (ten trees per block): the two
    splitters agree table for table, every plan covers every path once, and the schedule-aware passes act on some."""
    from dataclasses import replace
    acted = 0
    for seed in range(1000 + 10 * block, 1010 + 10 * block):
        rng = np.random.default_rng(seed)
        tree, batch, ptrs = product_tree(ref_inputs.random_tree(
            int(rng.integers(2, 6)), seed, max_children=int(rng.integers(3, 20)), lam=float(rng.uniform(1.5, 6)),
            len_lo=1, len_hi=int(rng.choice([40, 300, 2048]))))
        hq, hkv = [(32, 8), (8, 8), (16, 1), (64, 8), (4, 1)][seed % 5]
        model = replace(planner.B200Model(), num_sms=int(rng.choice([4, 16, 148])), waves=float(rng.choice([0.5, 1.0, 2.0])),
                        min_chunk=int(rng.choice([64, 128])), rows_per_cta=int(rng.choice([64, 128])),
                        group_member_tokens=int(rng.choice([0, 128])))
        pa, pb = make_params(hq, hkv, [16, 4], planner_name="b200"), make_params(hq, hkv, [16, 4], planner_name="b200")
        spec = planner.plan_b200(tree, ptrs, batch, hq, hkv, 128, pa, model=model)
        native = planner.plan_b200_native(tree, ptrs, batch, hq, hkv, 128, pb, model=model)
        _same_plan(spec, native)
        check_plan_covers_every_path_once(tree, ptrs, batch, native)
        m = planner.b200_model_for(pa, 128, model)
        vnodes, _, q_tile, small_tile, target = planner.b200_virtual_nodes(
            tree, hq, hkv, 128, m, lambda a, i: planner._chain_ranges(tree, ptrs, a, i))
        if m.elem_bytes == 2:
            vnodes = planner.b200_group_short_nodes(vnodes, q_tile, small_tile, m, int(target // (2 * 128 * m.elem_bytes)),
                                                    num_kv_heads=hkv)
        cut = planner.b200_split_tail(vnodes, q_tile, small_tile, m, hkv)
        slots = max(m.num_sms * m.ctas_per_sm // hkv, 1)
        before = planner.b200_simulated_schedule(vnodes, q_tile, small_tile, m, slots)[0]
        after = planner.b200_simulated_schedule(cut, q_tile, small_tile, m, slots)[0]
        changed = any(a.kv_split != b.kv_split for a, b in zip(vnodes, cut))
        assert after < before if changed else after == before      # a cut is kept only if the makespan drops
        acted += changed
    assert acted >= 1                                              # these seeds include plans the last-round pass cuts


def test_native_splitter_rejects_bad_trees():
    from ft_b200 import lib
    tree, batch, ptrs = product_tree(ref_inputs.layered_tree([1, 2], [5, 5]))
    p = make_params(8, 8, [16, 4], planner_name="b200")
    with pytest.raises(ValueError):
        planner.plan_b200_native(tree, ptrs[:-1], batch, 8, 8, 128, p)
    with pytest.raises(lib.FastTreeError):                      # a request id outside the batch
        planner.plan_b200_native(tree, ptrs, batch - 1, 8, 8, 128, p)
    import ctypes
    L, handle = lib.load(), ctypes.c_void_p()                  # a plan without groups has no row-range table to give
    parent, seqlen, req_offs, req_ids = planner._tree_arrays(tree)
    i32p, i64p = ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int64)
    kv = np.asarray(ptrs, dtype=np.int64)
    assert L.ft_plan_b200_build(parent.ctypes.data_as(i32p), seqlen.ctypes.data_as(i32p), len(tree),
                                req_offs.ctypes.data_as(i64p), req_ids.ctypes.data_as(i32p), kv.ctypes.data_as(i64p),
                                batch, 8, 8, 128, None, ctypes.byref(handle)) == 0
    info = lib.PlanInfo()
    assert L.ft_plan_get_info(handle, ctypes.byref(info)) == 0 and info.has_row_ranges == 0
    out = np.zeros(2 * max(int(info.partial_rows), 1), dtype=np.int32)
    assert L.ft_plan_copy_row_ranges(handle, out.ctypes.data_as(i32p)) == -1
    L.ft_plan_free(handle)
    tree[1].parent = 2                                         # parent after child
    with pytest.raises(lib.FastTreeError):
        planner.plan_b200_native(tree, ptrs, batch, 8, 8, 128, p)


def test_b200_plan_splits_long_prefix_and_keeps_leaves_whole():
    tree, batch, ptrs = product_tree(ref_inputs.layered_tree([1, 64], [4096, 256]))
    p = make_params(32, 8, [16, 4], planner_name="b200")
    plan = fasttree.build_plan(tree, ptrs, batch, 32, 8, 128, [1024, 128], [132, 528], [132, 132], p)
    lens = plan.vnode_to_kv_lens
    leaf = lens[plan.vnode_to_q_lens == 1]
    # leaves: one task each, except the 14 whose CTAs would form the step's last, partly filled round - those are halved
    assert (leaf == 256).sum() == 50 and (leaf == 128).sum() == 28 and leaf.size == 78
    assert lens.max() < 4096 and lens.max() % 64 == 0              # the shared prefix is cut on tile boundaries
    # long tasks first inside each phase
    n0 = plan.phase_node_nums[0]
    assert (np.diff(lens[:n0]) <= 0).all() and (np.diff(lens[n0:]) <= 0).all()
    # far fewer partial rows than the reference plan for the same tree (2176)
    assert plan.num_partial_rows < 1000


@pytest.mark.parametrize("native", [True, False], ids=["native", "spec"])
def test_fp32_hint_cuts_a_small_problem_into_single_tiles(native):
    """With the splitter told that K/V are fp32 (FastTreeParams.set_kv_dtype), a problem too small to fill the
    machine is cut into 32-token chunks (one tile of the CUDA-core kernel each) instead of 128-token ones."""
    import torch
    tree, batch, ptrs = product_tree(ref_inputs.layered_tree([1, 4], [512, 64]))
    plans = []
    for told in (False, True):
        p = make_params(8, 2, [16, 4], planner_name="b200")
        p.native_planner = native
        if told:
            p.set_kv_dtype(torch.float32)
        plans.append(fasttree.build_plan(tree, ptrs, batch, 8, 2, 128, [1024, 128], [132, 528], [132, 132], p))
        check_plan_covers_every_path_once(tree, ptrs, batch, plans[-1])
    assert sorted(set(plans[0].vnode_to_kv_lens.tolist())) == [64, 128]
    assert set(plans[1].vnode_to_kv_lens.tolist()) == {32}
    with pytest.raises(ValueError):
        make_params(8, 2, [16, 4], planner_name="b200").set_kv_dtype(torch.float64)


def test_reference_mode_covers_every_path_once():
    tree, batch, ptrs = product_tree(ref_inputs.layered_tree([1, 2, 16], [8, 40, 19]))
    p = make_params(8, 2, [16, 4])
    plan = fasttree.build_plan(tree, ptrs, batch, 8, 2, 64, [1024, 128], [132, 528], [132, 132], p)
    assert sum(plan.node_assignments) > 0          # this tree triggers KV-carrying children
    check_plan_covers_every_path_once(tree, ptrs, batch, plan)


def test_tree_file_tools_match_reference_format(tmp_path):
    rows = tree_generation.generate_tree([1, 3, 7], [70, 33, 21])
    path = tmp_path / "tree.txt"
    tree_generation.save_tree(rows, str(path))
    onodes = ref_inputs.layered_tree([1, 3, 7], [70, 33, 21])
    ref_path = tmp_path / "ref.txt"
    ref_inputs.write_tree_file(onodes, ref_path)
    assert path.read_text() == ref_path.read_text()
    nodes = retrive_from_file(str(path))
    validate_tree(nodes)
    assert [(n.parent, n.id, n.seqlen, n.num_children) for n in nodes] == [tuple(r) for r in rows]
    tree_generation.main(["-n", "1,2", "-l", "5,6", "-o", str(tmp_path / "cli.txt")])
    assert (tmp_path / "cli.txt").read_text() == "3\n-1 0 5 2\n0 1 6 0\n0 2 6 0\n"
    with pytest.raises(ValueError):
        tree_generation.generate_tree([1, 2], [3])


def test_validate_tree_rejects_bad_trees():
    nodes = [KVTreeNode(-1, 0, 4, 1), KVTreeNode(0, 1, 4, 0)]
    validate_tree(nodes)
    nodes[1].parent = 1
    with pytest.raises(ValueError):
        validate_tree(nodes)
    nodes[1].parent = 0
    nodes[0].num_children = 2
    with pytest.raises(ValueError):
        validate_tree(nodes)


GROUP_TREES = {
    # tree                                                         heads      groups expected
    "cfg3": (([1, 16, 256], [2048, 512, 64]), (32, 8), True),
    "deep_short": (([1, 2, 4, 8, 16, 32, 64], [16] * 7), (32, 32), True),
    "ragged_members": (([1, 3, 24], [30, 129, 31]), (16, 4), True),
    "long_leaves": (([1, 64], [4096, 256]), (32, 8), False),          # members longer than the limit
    "too_few": (([1, 5], [300, 20]), (8, 8), False),                  # fewer members than a group needs
}


@pytest.mark.parametrize("name", sorted(GROUP_TREES))
@pytest.mark.parametrize("native", [False, True], ids=["python", "native"])
def test_groups_of_short_nodes(name, native):
    """Short nodes with disjoint requests are packed into many-row tasks whose rows carry token ranges; the
    grouped plan still covers every path once, the few-row tasks keep whole-chunk ranges, and the oracle's
    two-stage evaluation of the grouped plan reproduces path-concatenated attention."""
    import torch
    from oracle import ref_attention
    (sizes, lens), (hq, hkv), expect = GROUP_TREES[name]
    onodes = ref_inputs.layered_tree(sizes, lens)
    tree, batch, ptrs = product_tree(onodes)
    p = make_params(hq, hkv, [16, 4], planner_name="b200")
    p.native_planner = native
    plan = fasttree.build_plan(tree, ptrs, batch, hq, hkv, 128, [1024, 128], [132, 528], [132, 132], p)
    assert (plan.vnode_q_kv_ranges is not None) == expect
    check_plan_covers_every_path_once(tree, ptrs, batch, plan)
    if not expect:
        return
    assert plan.vnode_q_kv_ranges.shape == (plan.num_partial_rows, 2) and plan.vnode_q_kv_ranges.dtype == np.int32
    # the same tree with grouping switched off has more tasks (partial rows: equal up to the chunks either plan halves
    # in its last round, planner.b200_split_tail)
    q = make_params(hq, hkv, [16, 4], planner_name="b200")
    q.native_planner = native
    from dataclasses import replace
    q.b200_model = replace(planner.b200_model_for(q, 128), group_member_tokens=0)
    flat = fasttree.build_plan(tree, ptrs, batch, hq, hkv, 128, [1024, 128], [132, 528], [132, 132], q)
    assert flat.vnode_q_kv_ranges is None
    assert flat.num_vnodes > plan.num_vnodes
    check_plan_covers_every_path_once(tree, ptrs, batch, flat)
    if sum(s * l for s, l in zip(sizes, lens)) > 20000:
        return                                     # the arithmetic check below is for the small trees
    qq, k, v, _, _ = ref_inputs.draw_qkv(onodes, hq, hkv, 128, torch.float32, 5, 0.5)
    scale = 1.0 / 128 ** 0.5
    mid_o, mid_lse = ref_attention.stage1_partials(qq, k, v, *plan.tables()[:6], scale, q_ranges=plan.vnode_q_kv_ranges)
    out, lse = ref_attention.stage2_merge(mid_o, mid_lse, *plan.tables()[6:9])
    truth, truth_lse = ref_attention.per_leaf_attention(onodes, ptrs, qq, k, v, scale)
    np.testing.assert_allclose(out.numpy(), truth.numpy(), rtol=1e-5, atol=2e-6)
    np.testing.assert_allclose(lse.numpy(), truth_lse.numpy(), rtol=1e-5, atol=1e-5)


def test_no_groups_outside_head_dim_128():
    tree, batch, ptrs = product_tree(ref_inputs.layered_tree([1, 16, 256], [64, 32, 16]))
    for native in (False, True):
        p = make_params(32, 8, [16, 4], planner_name="b200")
        p.native_planner = native
        plan = fasttree.build_plan(tree, ptrs, batch, 32, 8, 64, [1024, 128], [132, 528], [132, 132], p)
        assert plan.vnode_q_kv_ranges is None


def test_product_tree_builders_match_the_oracle():
    """The benchmark builds its trees with the shipped generator; the oracle's restatement must describe the
    same trees (layered and seeded irregular), request assignment and row ranges."""
    import kv_tree_simple
    import tree_generation
    for levels, seed in ((3, 0), (4, 0), (4, 2), (5, 1)):
        mine = kv_tree_simple.tree_from_rows(tree_generation.generate_random_tree(levels, seed))
        theirs = ref_inputs.random_tree(levels, seed)
        batch, ptrs = kv_tree_simple.assign_requests(mine)
        assert batch == ref_inputs.assign_requests(theirs) and ptrs == ref_inputs.kv_prefix_sums(theirs)
        assert [(n.parent, n.id, n.seqlen, n.num_children, n.requests) for n in mine] == \
               [(n.parent, n.id, n.seqlen, n.num_children, n.requests) for n in theirs]
    mine = kv_tree_simple.tree_from_rows(tree_generation.generate_tree([1, 16, 256], [2048, 512, 64]))
    theirs = ref_inputs.layered_tree([1, 16, 256], [2048, 512, 64])
    kv_tree_simple.assign_requests(mine)
    ref_inputs.assign_requests(theirs)
    assert [(n.parent, n.seqlen, n.num_children, n.requests) for n in mine] == \
           [(n.parent, n.seqlen, n.num_children, n.requests) for n in theirs]


def test_cascade_levels_describe_the_tree():
    """The multi-level cascade adapter's page lists: per depth every node's rows once, the requests split into
    consecutive ranges."""
    import flashinfer_wrap
    import kv_tree_simple
    for rows in (tree_generation.generate_tree([1, 4, 16], [256, 64, 32]), tree_generation.generate_random_tree(4, 1)):
        tree = kv_tree_simple.tree_from_rows(rows)
        batch, ptrs = kv_tree_simple.assign_requests(tree)
        qo, kv, idx = flashinfer_wrap.cascade_levels(tree, ptrs, batch)
        assert sorted(x for lv in idx for x in lv) == list(range(ptrs[-1]))
        for q, k in zip(qo, kv):
            assert q[0] == 0 and q[-1] == batch and len(q) == len(k) and all(b > a for a, b in zip(q, q[1:]))
