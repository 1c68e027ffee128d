"""SGLang-plugin tests that need no GPU: the SGLang-side planner against tables
produced by the reference's own schedule.py (run against the same stand-in
host), structural checks of the B200 planner, and the monkey-patch plumbing."""
import os

import numpy as np
import pytest
import torch

import sglang_standin

sglang_standin.install()

import plugin_cases  # noqa: E402
from fasttree_sglang_plugin_v0_2_13 import load_fasttree_plugin, metadata, plugin, schedule  # noqa: E402

GOLD = dict(np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "plugin_schedule_golden.npz")))
KEYS = ["vnode_to_kv_offs", "vnode_to_kv_lens", "vnode_to_q_offs", "vnode_to_q_lens", "vnode_to_q_entries",
        "req_to_vnode_entries", "req_to_vnode_offs", "req_to_vnode_lens"]


def make_md(hq, hkv, planner, group_load=0.0):
    # group_load 0: every burst with enough short tails is planned with groups, whatever its size
    return metadata.FastTreeMetadata(hq, hkv, 128, "cpu", max_vnodes=4096, max_vnode_to_q_entries=8192,
                                     max_batch_size=512, planner=planner, group_tails_min_load=group_load)


ALL_BURSTS = sorted(plugin_cases.CASES) + sorted(plugin_cases.TRAFFIC_SHAPES)


@pytest.mark.parametrize("name", sorted(plugin_cases.CASES))
def test_reference_mode_matches_reference_schedule_tables(name):
    batch, _rows, hq, hkv = plugin_cases.build(name)
    md = make_md(hq, hkv, "reference")
    schedule.prepare_for_fasttree_meta(batch, md)
    assert batch.fasttree_metadata is md
    nv, bsz = md.num_vnodes, len(batch.reqs)
    sizes = {"vnode_to_q_entries": md.num_partial_rows, "req_to_vnode_entries": md.num_partial_rows,
             "req_to_vnode_offs": bsz, "req_to_vnode_lens": bsz}
    for key in KEYS:
        want = GOLD[f"{name}/{key}"]
        got = getattr(md, key)[:sizes.get(key, nv)].numpy()
        np.testing.assert_array_equal(got, want, err_msg=key)
    for key in ("phase_node_nums", "phase_node_offsets", "phase_q_tile_sizes", "phase_kv_tile_sizes",
                "req_last_vnodes"):
        assert list(getattr(md, key)) == list(GOLD[f"{name}/{key}"]), key


AUX_BIT = 1 << 30


def check_cover(batch, rows, md, extra_prompt, steps_done=0):
    """Every request's partial rows together cover exactly its KV positions
    0 .. P + n (inclusive of the token being decoded), each once.  A vnode whose offset carries the
    auxiliary bit takes its row ids from the gathered table, and its rows see only their token ranges."""
    stride = batch.req_to_token_pool.req_to_token.stride(0)
    nv = md.num_vnodes
    kv_offs, kv_lens = md.vnode_to_kv_offs[:nv].numpy(), md.vnode_to_kv_lens[:nv].numpy()
    q_offs, q_lens = md.vnode_to_q_offs[:nv].numpy(), md.vnode_to_q_lens[:nv].numpy()
    q_entries = md.vnode_to_q_entries[:md.num_partial_rows].numpy()
    table = batch.req_to_token_pool.req_to_token.cpu().numpy().reshape(-1)
    grouped = getattr(md, "group_tails", False)
    aux = md.kv_entries_aux.numpy() if grouped else None
    ranges = md.vnode_q_kv_ranges[:md.num_partial_rows].numpy() if grouped else None
    seen = {r: [] for r in range(len(batch.reqs))}
    for v in range(nv):
        if kv_offs[v] & AUX_BIT:
            assert grouped and q_lens[v] * md.kv_group_num > 16        # only many-row kernels honour row ranges
            off = kv_offs[v] - AUX_BIT
            slots = aux[off:off + kv_lens[v]]
        else:
            slots = table[kv_offs[v]:kv_offs[v] + kv_lens[v]]
        for row in range(q_offs[v], q_offs[v] + q_lens[v]):
            lo, hi = (0, kv_lens[v]) if ranges is None else (max(ranges[row, 0], 0), min(ranges[row, 1], kv_lens[v]))
            if not (kv_offs[v] & AUX_BIT):
                assert (lo, hi) == (0, kv_lens[v])                      # rows of plain vnodes see the whole chunk
            seen[int(q_entries[row])].append(slots[lo:hi])
    for r, req in enumerate(batch.reqs):
        total = len(req.origin_input_ids) + len(req.output_ids) + 1
        want = np.sort(rows[r][:total].numpy())
        got = np.sort(np.concatenate(seen[r]))
        np.testing.assert_array_equal(got, want)
    assert sum(md.phase_node_nums) == nv and md.phase_node_offsets == [0, md.phase_node_nums[0]]
    # the task that ends at the request's last position, and what the per-step bump will advance
    state = md.tail_state[:len(batch.reqs)].numpy()
    for r, req in enumerate(batch.reqs):
        v = md.req_last_vnodes[r]
        end = stride * int(batch.req_pool_indices[r]) + len(req.origin_input_ids) + len(req.output_ids) + 1
        if state[r, 0] < 0:
            assert state[r, 2] == v
            assert kv_offs[v] + kv_lens[v] == end and q_lens[v] == 1 and q_entries[q_offs[v]] == r
        else:
            aux_pos, src_pos, row, room = state[r]
            assert src_pos == end and room == md.tail_room - steps_done and q_entries[row] == r
            assert q_offs[v] <= row < q_offs[v] + q_lens[v] and (kv_offs[v] & AUX_BIT)
            assert aux_pos == kv_offs[v] - AUX_BIT + ranges[row, 1]
            assert aux_pos + room <= kv_offs[v] - AUX_BIT + kv_lens[v]


@pytest.mark.parametrize("name", ALL_BURSTS)
@pytest.mark.parametrize("planner,extra,group_load", [("reference", 0, 0.0), ("b200", 0, 0.0), ("b200", 5, 0.0),
                                                      ("b200", 5, 4.0)])
def test_plans_cover_every_position_once(name, planner, extra, group_load):
    batch, rows, hq, hkv = plugin_cases.build(name, extra_prompt=extra)
    md = make_md(hq, hkv, planner, group_load)
    schedule.prepare_for_fasttree_meta(batch, md)
    check_cover(batch, rows, md, extra)
    if group_load > 0:          # the default threshold: few-row tasks x KV heads against four rounds of 2 x 148 resident CTAs
        plain = make_md(hq, hkv, planner, 1e9)
        again, _rows, _, _ = plugin_cases.build(name, extra_prompt=extra)
        schedule.prepare_for_fasttree_meta(again, plain)
        assert (md.num_grouped_tails > 0) == (plain.phase_node_nums[1] * hkv >= group_load * 296)


def test_a_burst_step_moves_every_tail():
    """prepare_for_fasttree_step on host-resident tables: a grouped tail's partial row sees one token more, a
    tail with a vnode of its own grows by one; a burst longer than the reserved room is refused."""
    batch, rows, hq, hkv = plugin_cases.build("long_tail", extra_prompt=2, steps=3)
    md = make_md(hq, hkv, "b200")
    md.tail_room = 2
    schedule.prepare_for_fasttree_meta(batch, md)
    assert 0 < md.num_grouped_tails < len(batch.reqs) or md.num_grouped_tails == len(batch.reqs)
    for step in range(2):
        for req in batch.reqs:
            req.output_ids.append(9_000_000 + step)
        schedule.prepare_for_fasttree_step(batch, md)
        # the row ids of the new tokens reach the auxiliary table in the step's first attention call: emulate it
        state = md.tail_state[:len(batch.reqs)].numpy()
        flat = batch.req_to_token_pool.req_to_token.reshape(-1)
        for aux_pos, src_pos, _row, _room in state.tolist():
            if aux_pos >= 0:
                md.kv_entries_aux[aux_pos - 1] = flat[src_pos - 1]
        check_cover(batch, rows, md, 2, steps_done=step + 1)
    with pytest.raises(RuntimeError):
        schedule.prepare_for_fasttree_step(batch, md)


@pytest.mark.parametrize("name", ALL_BURSTS)
@pytest.mark.parametrize("extra", [0, 5])
def test_native_schedule_matches_the_python_specification(name, extra):
    """ft_plan_b200_build_direct against b200_virtual_nodes + emit_tables on the same burst."""
    got = []
    for native in (True, False):
        batch, _rows, hq, hkv = plugin_cases.build(name, extra_prompt=extra)
        md = make_md(hq, hkv, "b200")
        md.native_planner = native
        schedule.prepare_for_fasttree_meta(batch, md)
        nv, rows = md.num_vnodes, md.num_partial_rows
        got.append(dict(
            kv_offs=md.vnode_to_kv_offs[:nv].clone(), kv_lens=md.vnode_to_kv_lens[:nv].clone(),
            q_entries=md.vnode_to_q_entries[:rows].clone(), q_offs=md.vnode_to_q_offs[:nv].clone(),
            q_lens=md.vnode_to_q_lens[:nv].clone(), r2v=md.req_to_vnode_entries[:rows].clone(),
            r2v_offs=md.req_to_vnode_offs[:len(batch.reqs)].clone(), r2v_lens=md.req_to_vnode_lens[:len(batch.reqs)].clone(),
            nums=list(md.phase_node_nums), offs=list(md.phase_node_offsets), last=list(md.req_last_vnodes),
            tiles=(list(md.phase_q_tile_sizes), list(md.phase_kv_tile_sizes)),
            ranges=md.vnode_q_kv_ranges[:rows].clone(), tails=md.tail_state[:len(batch.reqs)].clone(),
            grouped=md.num_grouped_tails))
    for k in got[0]:
        a, b = got[0][k], got[1][k]
        assert torch.equal(a, b) if torch.is_tensor(a) else a == b, k
    if name in plugin_cases.TRAFFIC_SHAPES:        # every traffic shape has enough short tails to form groups
        assert got[0]["grouped"] > 0


def test_b200_plan_is_deterministic():
    tabs = []
    for _ in range(2):
        batch, _rows, hq, hkv = plugin_cases.build("long_tail")
        md = make_md(hq, hkv, "b200")
        schedule.prepare_for_fasttree_meta(batch, md)
        tabs.append([getattr(md, k)[:md.num_vnodes if "vnode_to_kv" in k or k.endswith(("q_offs", "q_lens")) else
                                    md.num_partial_rows].clone() for k in KEYS[:5]])
    for a, b in zip(*tabs):
        assert torch.equal(a, b)


def test_capacity_overflow_is_reported():
    batch, _rows, hq, hkv = plugin_cases.build("long_tail")
    md = metadata.FastTreeMetadata(hq, hkv, 128, "cpu", max_vnodes=8, max_vnode_to_q_entries=64, max_batch_size=256)
    with pytest.raises(ValueError):
        schedule.prepare_for_fasttree_meta(batch, md)


def test_monkey_patches_and_burst_loop(monkeypatch):
    """load_fasttree_plugin wires the worker: metadata per worker, CUDA graphs off,
    one plan per burst, a bump between steps, stale-plan break when the batch shrinks."""
    from sglang.srt.managers.tp_worker import ModelTpServer, ServerArgs, global_config
    from sglang.srt.layers.radix_attention import RadixAttention
    from sglang.srt.model_executor.forward_batch_info import InputMetadata

    created = {}

    class FakeMd:
        def __init__(self, hq, hkv, d, device, graph_safe=False):
            created["args"] = (hq, hkv, d, device)
            created["graph_safe"] = graph_safe

    calls = []
    monkeypatch.setattr(plugin, "FastTreeMetadata", FakeMd)
    monkeypatch.setattr(schedule, "prepare_for_fasttree_meta", lambda b, m: calls.append("meta"))
    monkeypatch.setattr(schedule, "prepare_for_fasttree_step", lambda b, m: calls.append("step"))
    monkeypatch.setattr(ModelTpServer, "__init__", ModelTpServer.__init__)      # restored after the test
    monkeypatch.setattr(ModelTpServer, "forward_step", ModelTpServer.forward_step)
    monkeypatch.setattr(RadixAttention, "__init__", RadixAttention.__init__)
    monkeypatch.setattr(InputMetadata, "from_schedule_batch", InputMetadata.from_schedule_batch)
    monkeypatch.setattr(torch.cuda, "device", torch.cuda.device)

    load_fasttree_plugin(enable_fasttree=False, annotate_breakdown=False)      # prints a warning, patches nothing
    load_fasttree_plugin(enable_fasttree=True)
    args = ServerArgs()
    args.tp_size = 2
    server = ModelTpServer(0, 0, args, 1234, {"num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128})
    assert args.disable_cuda_graph is True
    assert created["args"][:3] == (16, 4, 128)                                  # local head counts at TP=2
    attn = RadixAttention(16, 128, 0.088, 4, 0)
    assert attn.decode_forward is not None and attn.decode_forward.__func__.__name__ == "decode_forward_fasttree"

    batch, _rows, _, _ = plugin_cases.build("small_g4")
    server.running_batch = batch
    server.forward_step()                                                       # a full burst
    assert calls == ["meta"] + ["step"] * (global_config.num_continue_decode_steps - 1)
    assert server.decode_forward_ct == global_config.num_continue_decode_steps

    calls.clear()
    server.decode_fn = lambda b: b.reqs.pop()                                   # a request finishes in step 1
    server.forward_step()
    assert calls == ["meta"]                                                    # plan is stale: burst aborted
    meta = InputMetadata.from_schedule_batch(None, batch, "decode")
    assert hasattr(meta, "fasttree")

    server.running_batch = None
    server.forward_step()
    assert server.memory_checks == 1
