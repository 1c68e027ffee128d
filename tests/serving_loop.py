#!/usr/bin/env python
"""Timed decode loop of a random-init Llama-3-8B-shaped model on the stand-in SGLang host.

SGLang v0.2.13, model weights and the reference's datasets are not available here,
so the reference's end-to-end serving benchmarks
(sglang_v0.2.13_bench/benchmarks/bench_multi_*.py driven by run_benchmark.sh)
are stood in for by:

  * the stand-in host of tests/sglang_standin.py (radix cache, token pools,
    ``RadixAttention`` with the plugin's ``decode_forward`` hook installed by the
    plugin's own patch functions),
  * a decoder of Llama-3-8B shape with random weights (32 layers, hidden 4096,
    32 query / 8 KV heads of 128, MLP 14336; RMSNorm, fused QKV projection,
    attention hook, row-parallel output projection + all-reduce, SwiGLU MLP +
    all-reduce), tensor-parallel over the ranks of ``torchrun``,
  * the tree shapes of the four serving benchmarks with synthetic token counts
    (tests/plugin_cases.py::TRAFFIC_SHAPES).

One burst = one ``prepare_for_fasttree_meta`` followed by ``--steps`` decode
steps with ``prepare_for_fasttree_step`` in between - the burst loop of
fasttree_sglang_plugin_v0_2_13/plugin.py:111-135.  A decode step is timed with
CUDA events on the launching stream (max over ranks), in two launch modes:
``eager`` (Python launches every layer, as SGLang does with CUDA graphs off - the
only mode the reference supports, plugin.py:209-211) and ``graph`` (the whole
32-layer step captured ONCE in a CUDA graph and replayed, across bursts too,
which the plan-independent launch of ``FastTreeMetadata(graph_safe=True)``
makes possible).  On the first and last step of the run the attention output of
the first and last layer is compared with fp32 attention over each sampled
request's own token list.

    python tests/serving_loop.py --shape all
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 tests/serving_loop.py --shape all

Prints one JSON line per shape on rank 0.
"""
import argparse
import json
import os
import statistics
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for _p in (HERE, ROOT, os.path.join(ROOT, "fasttree-artifact_b200"), os.path.join(ROOT, "fasttree-artifact_b200", "kernel_bench")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import sglang_standin  # noqa: E402

sglang_standin.install()

import plugin_cases  # noqa: E402
from fasttree_sglang_plugin_v0_2_13 import metadata, plugin, schedule  # noqa: E402
from oracle import ref_inputs  # noqa: E402

HIDDEN, HQ, HKV, HEAD_DIM, INTER = 4096, 32, 8, 128, 14336


class Block:
    """One decoder layer, this rank's shard."""

    def __init__(self, layer_id, hq_l, hkv_l, inter_l, dtype, dev, gen, world):
        from sglang.srt.layers.radix_attention import RadixAttention

        def w(rows, cols):
            return (torch.randn(rows, cols, generator=gen, device=dev, dtype=torch.float32) * 0.02).to(dtype)

        self.hq_l, self.hkv_l, self.world = hq_l, hkv_l, world
        self.wqkv = w(HIDDEN, (hq_l + 2 * hkv_l) * HEAD_DIM)
        self.wo = w(hq_l * HEAD_DIM, HIDDEN)
        self.w13 = w(HIDDEN, 2 * inter_l)
        self.w2 = w(inter_l, HIDDEN)
        self.attn = RadixAttention(hq_l, HEAD_DIM, HEAD_DIM ** -0.5, hkv_l, layer_id)   # the plugin's hook is installed by its patch
        self.probe = None       # (q, o) of the last call when probing is on

    @staticmethod
    def norm(x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)).to(x.dtype)

    def forward(self, h, meta, probing=False):
        qkv = self.norm(h) @ self.wqkv
        nq, nk = self.hq_l * HEAD_DIM, self.hkv_l * HEAD_DIM
        q, k, v = qkv[:, :nq].contiguous(), qkv[:, nq:nq + nk].contiguous(), qkv[:, nq + nk:].contiguous()
        a = self.attn.decode_forward(q, k, v, meta)
        if probing:
            self.probe = (q.clone(), a.clone())
        part = a @ self.wo
        if self.world > 1:
            dist.all_reduce(part)
        h = h + part
        gu = self.norm(h) @ self.w13
        g, u = gu.chunk(2, dim=-1)
        part = (torch.nn.functional.silu(g) * u) @ self.w2
        if self.world > 1:
            dist.all_reduce(part)
        return h + part


def truth_for(batch, rows, layer, q, sample, scale, step_total):
    """fp32 attention of the sampled requests over their own token lists (this rank's heads)."""
    kv = batch.token_to_kv_pool
    k_pool, v_pool = kv.get_key_buffer(layer), kv.get_value_buffer(layer)
    hq, hkv = q.shape[1], k_pool.shape[1]
    out = []
    for r in sample:
        req = batch.reqs[r]
        total = len(req.origin_input_ids) + len(req.output_ids) + 1
        slots = rows[r][:total].long().to(k_pool.device)
        k, v = k_pool[slots].float(), v_pool[slots].float()
        qq = q[r].float().view(hkv, hq // hkv, -1)
        s = torch.einsum("hgd,lhd->hgl", qq, k) * scale
        out.append(torch.einsum("hgl,lhd->hgd", torch.softmax(s, dim=-1), v).reshape(hq, -1))
    return torch.stack(out)


def run_shape(name, args, rank, world, dev):
    dtype = torch.float16 if args.dtype == "fp16" else torch.bfloat16
    sizes, lens, gen_cycle, hq, hkv = plugin_cases.TRAFFIC_SHAPES.get(name) or plugin_cases.CASES[name]
    hq, hkv = HQ, HKV                     # the model's heads, whatever the case lists
    hq_l, hkv_l, inter_l = hq // world, hkv // world, INTER // world
    nodes = ref_inputs.layered_tree(sizes, lens)
    bsz = sum(1 for n in nodes if n.num_children == 0)
    generated = [gen_cycle[i % len(gen_cycle)] for i in range(bsz)]
    total_steps = args.steps * args.bursts * (2 if args.mode == "both" else 1) + 2
    pool = sum(n.seqlen for n in nodes) + sum(g + total_steps + args.extra_prompt for g in generated) + 64
    batch, rows = sglang_standin.build_batch(nodes, args.extra_prompt, generated, pool, hkv_l, HEAD_DIM, dtype, dev,
                                             seed=len(name) * 7, num_layers=1, steps=total_steps,
                                             slot_layout=args.pool_layout)
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    kv = batch.token_to_kv_pool
    for _ in range(1, args.layers):      # the remaining layers' pools, drawn on the device
        kv.k_buffer.append(torch.randn(pool, hkv_l, HEAD_DIM, generator=g, device=dev, dtype=torch.float32).to(dtype))
        kv.v_buffer.append(torch.randn(pool, hkv_l, HEAD_DIM, generator=g, device=dev, dtype=torch.float32).to(dtype))
    context_tokens = sum(len(r.origin_input_ids) + len(r.output_ids) for r in batch.reqs)

    plugin._replace_fwd_batch_info()
    plugin._replace_radix_attn()
    from sglang.srt.model_executor.forward_batch_info import InputMetadata
    blocks = [Block(i, hq_l, hkv_l, inter_l, dtype, dev, g, world) for i in range(args.layers)]
    out = {"shape": name, "tp": world, "pool_layout": args.pool_layout, "requests": bsz, "context_tokens": context_tokens,
           "layers": args.layers,
           "dtype": args.dtype, "steps_per_burst": args.steps, "bursts": args.bursts}
    modes = ["eager", "graph"] if args.mode == "both" else [args.mode]
    out_loc = batch.out_cache_loc.clone()             # static: the graph reads it, the loop rewrites it
    batch.out_cache_loc = out_loc
    hidden_in = torch.zeros(bsz, HIDDEN, dtype=dtype, device=dev)
    sample = sorted(set(int(round(i * (bsz - 1) / 7)) for i in range(8))) if bsz > 1 else [0]
    parity = 0.0
    scale = HEAD_DIM ** -0.5

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for mode in modes:
        md = metadata.FastTreeMetadata(hq_l, hkv_l, HEAD_DIM, dev, max_vnodes=16384, max_vnode_to_q_entries=32768,
                                       max_batch_size=max(64, bsz), planner="b200", graph_safe=(mode == "graph"))
        graph, hidden_out = None, None
        step_us, plan_ms = [], []
        for burst in range(args.bursts):
            t0 = time.perf_counter()
            schedule.prepare_for_fasttree_meta(batch, md)
            torch.cuda.synchronize()
            plan_ms.append((time.perf_counter() - t0) * 1e3)
            meta = InputMetadata.from_schedule_batch(None, batch, "decode")

            def step_fn(probing=False):
                h = hidden_in
                for blk in blocks:
                    h = blk.forward(h, meta, probing)
                return h

            for step in range(args.steps):
                hidden_in.copy_(torch.randn(bsz, HIDDEN, generator=g, device=dev, dtype=torch.float32).to(dtype))
                first, last = burst == 0 and step == 0, burst == args.bursts - 1 and step == args.steps - 1
                if mode == "graph" and graph is None:
                    step_fn()                                     # first-use costs outside the capture
                    torch.cuda.synchronize()
                    side = torch.cuda.Stream(device=dev)
                    side.wait_stream(torch.cuda.current_stream())
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.stream(side):
                        with torch.cuda.graph(graph, stream=side):
                            hidden_out = step_fn()
                    torch.cuda.current_stream().wait_stream(side)
                fence()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                if mode == "graph":
                    graph.replay()
                else:
                    hidden_out = step_fn()
                e1.record()
                fence()
                us = torch.tensor([e0.elapsed_time(e1) * 1e3], device=dev, dtype=torch.float64)
                if world > 1:
                    dist.all_reduce(us, op=dist.ReduceOp.MAX)
                step_us.append(us.item())
                if first or last:
                    # the same step once more, eagerly, with the first and last layer's q / o recorded; their
                    # attention is checked against fp32 attention over the sampled requests' token lists
                    step_fn(probing=True)
                    torch.cuda.synchronize()
                    for li in sorted({0, args.layers - 1}):
                        q, a = blocks[li].probe
                        want = truth_for(batch, rows, li, q.view(bsz, hq_l, HEAD_DIM), sample, scale, None)
                        got = a.view(bsz, hq_l, HEAD_DIM)[sample].float()
                        parity = max(parity, (got - want).abs().max().item())
                        blocks[li].probe = None
                # the host appends the sampled token and reserves the next slot; the plugin bumps its plan
                for r, req in enumerate(batch.reqs):
                    req.output_ids.append(9_000_000 + len(req.output_ids))
                out_loc.copy_(torch.stack([rows[r][len(req.origin_input_ids) + len(req.output_ids)]
                                           for r, req in enumerate(batch.reqs)]).to(dev))
                if step < args.steps - 1:
                    schedule.prepare_for_fasttree_step(batch, md)
        # attention alone: the 32 hook calls of one step on fixed projections (eager launches)
        if mode == "eager":
            qs = (torch.randn(bsz, hq_l * HEAD_DIM, generator=g, device=dev, dtype=torch.float32) * 0.5).to(dtype)
            kn = torch.randn(bsz, hkv_l * HEAD_DIM, generator=g, device=dev, dtype=torch.float32).to(dtype)
            schedule.prepare_for_fasttree_meta(batch, md)
            meta = InputMetadata.from_schedule_batch(None, batch, "decode")
            for rep in range(2):
                fence()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for blk in blocks:
                    blk.attn.decode_forward(qs, kn, kn, meta)
                e1.record()
                fence()
            out["attention_us_per_step_eager"] = e0.elapsed_time(e1) * 1e3
        out[f"step_us_{mode}"] = statistics.median(step_us)
        out[f"step_us_{mode}_min"] = min(step_us)
        out[f"plan_ms_{mode}"] = statistics.median(plan_ms)
        out[f"vnodes_{mode}"] = md.num_vnodes
        del graph
    from ft_b200 import lib
    status = lib.read_device_status()
    t = torch.tensor([parity, float(status)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out["parity_max_abs"], out["device_status"] = t[0].item(), int(t[1].item())
    tol = 2e-3 + (2 ** -8 * 4 if dtype == torch.bfloat16 else 0.0)
    out["parity_ok"] = bool(out["parity_max_abs"] <= tol and out["device_status"] == 0)
    del blocks, batch, kv
    torch.cuda.empty_cache()
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="all", help="a traffic shape of tests/plugin_cases.py, or 'all'")
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--steps", type=int, default=8, help="decode steps per burst")
    ap.add_argument("--bursts", type=int, default=2)
    ap.add_argument("--extra-prompt", type=int, default=2, help="private prompt tokens per request (not in the radix cache)")
    ap.add_argument("--mode", default="both", choices=["eager", "graph", "both"])
    ap.add_argument("--pool-layout", default="scattered", choices=["scattered", "prefill"],
                    help="KV-pool slots: a random permutation (every row gathered on its own), or what a serving process "
                         "leaves behind (radix nodes in consecutive slots, generated tokens interleaved across requests)")
    ap.add_argument("--dtype", default="fp16", choices=["fp16", "bf16"])
    args = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if HKV % world:
        raise SystemExit(f"{HKV} kv heads cannot be sharded over {world} ranks")
    shapes = sorted(plugin_cases.TRAFFIC_SHAPES) if args.shape == "all" else args.shape.split(",")
    results = []
    with torch.inference_mode():
        for name in shapes:
            res = run_shape(name, args, rank, world, dev)
            results.append(res)
            if rank == 0:
                print(json.dumps(res), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return results


if __name__ == "__main__":
    main()
