"""The SGLang hook on a GPU, against the stand-in host: a burst of decode steps
through the patched ``RadixAttention.decode_forward`` (store the new token's K/V,
tree attention through ``req_to_token``), each step checked against fp32
attention over every request's own token list."""
import pytest
import torch

import sglang_standin

sglang_standin.install()

import plugin_cases  # noqa: E402
from fasttree_sglang_plugin_v0_2_13 import metadata, plugin, schedule  # noqa: E402
from ft_b200 import engine, lib  # noqa: E402

pytestmark = pytest.mark.gpu


def reference_attention(batch, rows, q, layer, step, scale):
    kv = batch.token_to_kv_pool
    k_pool, v_pool = kv.get_key_buffer(layer).float().cpu(), kv.get_value_buffer(layer).float().cpu()
    hq, hkv = q.shape[1], k_pool.shape[1]
    out = []
    for r, req in enumerate(batch.reqs):
        total = len(req.origin_input_ids) + len(req.output_ids) + 1
        slots = rows[r][:total].long()
        k, v = k_pool[slots], v_pool[slots]                          # [L, hkv, d]
        qq = q[r].float().cpu().view(hkv, hq // hkv, -1)
        s = torch.einsum("hgd,lhd->hgl", qq, k) * scale
        p = torch.softmax(s, dim=-1)
        out.append(torch.einsum("hgl,lhd->hgd", p, v).reshape(hq, -1))
    return torch.stack(out)


@pytest.mark.parametrize("name", ["small_g4", "three_level", "wide_mha", "long_tail"])
@pytest.mark.parametrize("planner,extra", [("reference", 0), ("b200", 0), ("b200", 3)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_decode_burst_through_the_hook(name, planner, extra, dtype):
    run_burst(name, planner, extra, dtype, steps=3)


@pytest.mark.parametrize("name", sorted(plugin_cases.TRAFFIC_SHAPES))
@pytest.mark.parametrize("slot_layout", ["scattered", "prefill"])
def test_serving_traffic_shapes_through_the_hook(name, slot_layout):
    """The tree shapes of the reference's four serving benchmarks (synthetic token counts), two decode steps, on
    a pool whose slots are a random permutation (every row gathered) and on one laid out as a serving process
    leaves it (radix nodes in consecutive slots: tiled copies; generated tokens interleaved across requests)."""
    run_burst(name, "b200", 2, torch.float16, steps=2, slot_layout=slot_layout)


@pytest.mark.parametrize("name", ["system_4x128", "few_shot_8x16", "long_tail"])
@pytest.mark.parametrize("grouped", [True, False], ids=["grouped", "one_task_per_tail"])
def test_grouped_private_tails_through_the_hook(name, grouped):
    """The plan packs the requests' private tails into many-row vnodes whose row ids are gathered into the
    auxiliary table once per burst; every step extends each member by the token just decoded (its row id arrives
    in the step's first attention call, its partial row's range grows in the bump).  Four steps against fp32
    attention, with and without grouping; the grouped plan has far fewer tasks."""
    md = run_burst(name, "b200", 2, torch.float16, steps=4, group_tails=grouped)
    assert (md.num_grouped_tails > 0) == grouped
    if grouped:
        plain = metadata.FastTreeMetadata(md.num_qo_heads, md.num_kv_heads, 128, "cpu", max_vnodes=4096,
                                          max_vnode_to_q_entries=8192, max_batch_size=512, group_tails=False)
        batch, _rows, _, _ = plugin_cases.build(name, extra_prompt=2, steps=4)
        schedule.prepare_for_fasttree_meta(batch, plain)
        assert md.num_vnodes < plain.num_vnodes


@pytest.mark.parametrize("name", ["long_tail", "system_4x128", "small_g4"])
def test_decode_burst_in_graph_safe_mode(name):
    """The same bursts with the phase split read on the device and the persistent stage-1 kernel behind the hook."""
    run_burst(name, "b200", 2, torch.float16, steps=3, graph_safe=True)


def run_burst(name, planner, extra, dtype, steps, graph_safe=False, group_tails=True, slot_layout="scattered"):
    from sglang.srt.layers.radix_attention import RadixAttention
    from sglang.srt.model_executor.forward_batch_info import InputMetadata

    batch, rows, hq, hkv = plugin_cases.build(name, device="cuda", dtype=dtype, extra_prompt=extra, steps=steps,
                                              slot_layout=slot_layout)
    d = 128
    md = metadata.FastTreeMetadata(hq, hkv, d, "cuda", max_vnodes=4096, max_vnode_to_q_entries=8192,
                                   max_batch_size=512, planner=planner, graph_safe=graph_safe, group_tails=group_tails,
                                   group_tails_min_load=0.0)     # groups whenever the tails allow, whatever the burst's size
    plugin._replace_fwd_batch_info()
    plugin._replace_radix_attn()
    attn = RadixAttention(hq, d, 1.0 / d ** 0.5, hkv, 0)
    g = torch.Generator(device="cuda").manual_seed(11)
    # As in SGLang, a token's KV-pool slot enters req_to_token only when its step's batch is prepared - after the
    # plan, and after the bump between steps: entries of tokens not yet decoded hold -1 until then.
    r2t = batch.req_to_token_pool.req_to_token
    pool_rows = batch.req_pool_indices.tolist()
    first_new = [len(req.origin_input_ids) + len(req.output_ids) for req in batch.reqs]
    for r, row in enumerate(pool_rows):
        r2t[row, first_new[r]:] = -1
    schedule.prepare_for_fasttree_meta(batch, md)
    bsz = len(batch.reqs)
    for step in range(steps):
        for r, row in enumerate(pool_rows):
            r2t[row, first_new[r] + step] = rows[r][first_new[r] + step]
        q = (torch.randn(bsz, hq * d, generator=g, device="cuda") * 0.5).to(dtype)
        k_new = torch.randn(bsz, hkv * d, generator=g, device="cuda").to(dtype)
        v_new = torch.randn(bsz, hkv * d, generator=g, device="cuda").to(dtype)
        meta = InputMetadata.from_schedule_batch(None, batch, "decode")
        assert meta.fasttree is md
        o = attn.decode_forward(q, k_new, v_new, meta)
        torch.cuda.synchronize()
        assert lib.read_device_status() == 0
        want = reference_attention(batch, rows, q.view(bsz, hq, d), 0, step, attn.scaling)
        tol = 2e-3 + (float(want.abs().max()) * 2 ** -8 if dtype == torch.bfloat16 else 0.0)
        err = (o.view(bsz, hq, d).float().cpu() - want).abs().max().item()
        assert err <= tol, (step, err)
        # the host appends the sampled token and reserves the next slot, the plugin bumps its plan
        for r, req in enumerate(batch.reqs):
            req.output_ids.append(9_000_000 + step)
        if step < steps - 1:
            batch.out_cache_loc = torch.stack([rows[r][len(req.origin_input_ids) + len(req.output_ids)]
                                               for r, req in enumerate(batch.reqs)]).cuda()
            schedule.prepare_for_fasttree_step(batch, md)
    return md


def test_captured_decode_step_survives_a_replan():
    """``FastTreeMetadata(graph_safe=True)``: the decode call takes its phase split from device memory and runs
    the persistent stage-1 kernel, whose launch does not depend on the plan.  A step captured ONCE in a CUDA graph
    is replayed after the plan tables (fixed-capacity device buffers) have been rewritten for other bursts -
    other trees, other vnode counts, same batch size and pools - and must give the bits of an eager call on the
    new plan, and the right attention."""
    from fasttree_sglang_plugin_v0_2_13 import attn_kernels
    from oracle import ref_inputs
    hq, hkv, d, dtype = 32, 8, 128, torch.float16
    shapes = [([1, 3, 9], [100, 30, 7]), ([1, 9], [300, 11]), ([1, 9], [5, 70]), ([1, 1, 9], [700, 64, 1])]
    pool, width, gen = 8192, 1024, [3, 0, 5, 1]
    bursts = []
    for i, (sizes, lens) in enumerate(shapes):
        nodes = ref_inputs.layered_tree(sizes, lens)
        generated = [gen[(r + i) % len(gen)] for r in range(9)]
        bursts.append(sglang_standin.build_batch(nodes, 2, generated, pool, hkv, d, dtype, "cuda", seed=50 + i,
                                                 max_context_len=width, steps=1))
    base = bursts[0][0]
    r2t = base.req_to_token_pool.req_to_token
    k_buf, v_buf = base.token_to_kv_pool.get_key_buffer(0), base.token_to_kv_pool.get_value_buffer(0)
    md = metadata.FastTreeMetadata(hq, hkv, d, "cuda", max_vnodes=1024, max_vnode_to_q_entries=4096,
                                   max_batch_size=64, graph_safe=True)
    q = torch.zeros(9, hq, d, dtype=dtype, device="cuda")
    o = torch.zeros_like(q)
    scale = 1.0 / d ** 0.5

    def call():
        # what the attention hook does for the first layer of a step: the grouped tails take their newest row id,
        # then the decode call with the range table and the auxiliary row-id table of the plan
        engine.refresh_tails(md.tail_state, md.max_batch_size, r2t, md.kv_entries_aux)
        attn_kernels.fasttree_decode(q, k_buf, v_buf, o, r2t, md.vnode_to_kv_offs, md.vnode_to_kv_lens,
                                     md.vnode_to_q_entries, md.vnode_to_q_offs, md.vnode_to_q_lens,
                                     md.req_to_vnode_entries, md.req_to_vnode_offs, md.req_to_vnode_lens,
                                     md.mid_o, md.mid_lse, md.phase_node_nums, md.phase_node_offsets,
                                     md.phase_q_tile_sizes, md.phase_kv_tile_sizes, scale, phase_info=md.phase_info_dev,
                                     row_ranges=md.vnode_q_kv_ranges, kv_entries_aux=md.kv_entries_aux)

    schedule.prepare_for_fasttree_meta(base, md)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        call()
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            call()
    torch.cuda.current_stream().wait_stream(side)
    plans = set()
    g = torch.Generator(device="cuda").manual_seed(3)
    contents = [(b.req_to_token_pool.req_to_token.clone(), b.token_to_kv_pool.get_key_buffer(0).clone(),
                 b.token_to_kv_pool.get_value_buffer(0).clone()) for b, _ in bursts]
    for idx in (1, 2, 3, 0):
        batch, rows = bursts[idx]
        # the pools are persistent in a serving process: bring this burst's contents into the captured tensors
        r2t.copy_(contents[idx][0])
        k_buf.copy_(contents[idx][1])
        v_buf.copy_(contents[idx][2])
        batch.req_to_token_pool.req_to_token = r2t
        batch.token_to_kv_pool.k_buffer[0], batch.token_to_kv_pool.v_buffer[0] = k_buf, v_buf
        schedule.prepare_for_fasttree_meta(batch, md)
        plans.add((tuple(md.phase_node_nums), md.num_vnodes, md.num_partial_rows))
        q.copy_((torch.randn(9, hq, d, generator=g, device="cuda") * 0.5).to(dtype))
        o.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        replayed = o.clone()
        assert lib.read_device_status() == 0
        o.fill_(float("nan"))
        call()
        torch.cuda.synchronize()
        assert torch.equal(replayed, o)
        want = reference_attention(batch, rows, q, 0, 0, scale)
        assert (replayed.float().cpu() - want).abs().max().item() <= 2e-3
    assert len(plans) >= 3          # the replays really ran on different plans
