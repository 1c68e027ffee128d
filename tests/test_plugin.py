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


def make_md(hq, hkv, planner):
    return metadata.FastTreeMetadata(hq, hkv, 128, "cpu", max_vnodes=4096, max_vnode_to_q_entries=8192,
                                     max_batch_size=512, planner=planner)


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


def check_cover(batch, rows, md, extra_prompt):
    """Every request's partial rows together cover exactly its KV positions
    0 .. P + n (inclusive of the token being decoded), each once."""
    stride = batch.req_to_token_pool.req_to_token.stride(0)
    nv = md.num_vnodes
    kv_offs, kv_lens = md.vnode_to_kv_offs[:nv].numpy(), md.vnode_to_kv_lens[:nv].numpy()
    q_offs, q_lens = md.vnode_to_q_offs[:nv].numpy(), md.vnode_to_q_lens[:nv].numpy()
    q_entries = md.vnode_to_q_entries[:md.num_partial_rows].numpy()
    table = batch.req_to_token_pool.req_to_token.cpu().numpy().reshape(-1)
    seen = {r: [] for r in range(len(batch.reqs))}
    for v in range(nv):
        slots = table[kv_offs[v]:kv_offs[v] + kv_lens[v]]
        for row in range(q_offs[v], q_offs[v] + q_lens[v]):
            seen[int(q_entries[row])].append(slots)
    for r, req in enumerate(batch.reqs):
        total = len(req.origin_input_ids) + len(req.output_ids) + 1
        want = np.sort(rows[r][:total].numpy())
        got = np.sort(np.concatenate(seen[r]))
        np.testing.assert_array_equal(got, want)
    assert sum(md.phase_node_nums) == nv and md.phase_node_offsets == [0, md.phase_node_nums[0]]
    # req_last_vnodes: the task that ends at the request's last position
    for r, req in enumerate(batch.reqs):
        v = md.req_last_vnodes[r]
        end = stride * int(batch.req_pool_indices[r]) + len(req.origin_input_ids) + len(req.output_ids) + 1
        assert kv_offs[v] + kv_lens[v] == end and q_lens[v] == 1 and q_entries[q_offs[v]] == r


@pytest.mark.parametrize("name", ALL_BURSTS)
@pytest.mark.parametrize("planner,extra", [("reference", 0), ("b200", 0), ("b200", 5)])
def test_plans_cover_every_position_once(name, planner, extra):
    batch, rows, hq, hkv = plugin_cases.build(name, extra_prompt=extra)
    md = make_md(hq, hkv, planner)
    schedule.prepare_for_fasttree_meta(batch, md)
    check_cover(batch, rows, md, extra)


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
            tiles=(list(md.phase_q_tile_sizes), list(md.phase_kv_tile_sizes))))
    for k in got[0]:
        a, b = got[0][k], got[1][k]
        assert torch.equal(a, b) if torch.is_tensor(a) else a == b, k


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
