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
from ft_b200 import lib  # noqa: E402

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
def test_serving_traffic_shapes_through_the_hook(name):
    """The tree shapes of the reference's four serving benchmarks (synthetic token counts), two decode steps."""
    run_burst(name, "b200", 2, torch.float16, steps=2)


def run_burst(name, planner, extra, dtype, steps):
    from sglang.srt.layers.radix_attention import RadixAttention
    from sglang.srt.model_executor.forward_batch_info import InputMetadata

    batch, rows, hq, hkv = plugin_cases.build(name, device="cuda", dtype=dtype, extra_prompt=extra, steps=steps)
    d = 128
    md = metadata.FastTreeMetadata(hq, hkv, d, "cuda", max_vnodes=4096, max_vnode_to_q_entries=8192,
                                   max_batch_size=512, planner=planner)
    plugin._replace_fwd_batch_info()
    plugin._replace_radix_attn()
    attn = RadixAttention(hq, d, 1.0 / d ** 0.5, hkv, 0)
    g = torch.Generator(device="cuda").manual_seed(11)
    schedule.prepare_for_fasttree_meta(batch, md)
    bsz = len(batch.reqs)
    for step in range(steps):
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
