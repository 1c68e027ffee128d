#!/usr/bin/env python
"""Decode-step benchmark of the B200 tree-attention engine.

    python bench.py --gpus N --steps K --warmup W            # this engine
    python bench.py --impl reference --steps K --warmup W    # CPU baseline arm

A step is one tree-attention decode call (one layer) over a synthetic radix
tree.  Default workload: N=[1,64] nodes per level, C=[4096,256] tokens per
node, 32 query / 8 KV heads, head_dim 128, fp16 - 64 decode requests sharing a
4096-token prefix.  Under torchrun the KV heads are sharded across ranks
(tensor parallel); the output stays head-sharded on its rank, as it does in
tensor-parallel serving where it feeds a row-parallel projection, so the step
has no collective (``--gather-output`` adds an NCCL all-gather of the heads).

Prints ONE JSON line on rank 0.  ``value`` is microseconds per step with
everything resident in HBM; ``e2e`` is the same call fed from pinned host
memory (query copied in, output copied out, every step); ``roofline`` relates
the stage-1 kernel to the measured HBM copy bandwidth; ``cpu_baseline`` is the
oracle's per-request path-concatenated attention on the host cores.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "fasttree-artifact_b200")
for _p in (ROOT, PKG, os.path.join(PKG, "kernel_bench")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

_JSON_FD = os.dup(1)      # keep the real stdout for the result line ...
os.dup2(2, 1)             # ... and send every other write to fd 1 to stderr

import torch  # noqa: E402

WORKLOADS = {
    # name: level sizes, level lengths, query heads, kv heads, dtype, q scale
    "cfg1": ([1, 4], [512, 64], 8, 2, "fp32", 1.0),
    "cfg2": ([1, 64], [4096, 256], 32, 8, "fp16", 1.0),
    "cfg3": ([1, 16, 256], [2048, 512, 64], 32, 8, "bf16", 0.5),
    "cfg4": ([1, 1024], [16384, 32], 64, 8, "bf16", 1.0),
}
RANDOM_WORKLOADS = {"cfg5-d4": 4, "cfg5-d5": 5, "cfg5-d6": 6}      # random trees: node levels
DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}
HEAD_DIM = 128
L2_BYTES = 126 * 2 ** 20
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0


def build_tree(workload, seed):
    from oracle import ref_inputs
    if workload in RANDOM_WORKLOADS:
        nodes = ref_inputs.random_tree(RANDOM_WORKLOADS[workload], seed)
        hq, hkv, dt, qs = 32, 8, "fp16", 1.0
        desc = f"random tree, {RANDOM_WORKLOADS[workload]} node levels, seed {seed}"
    else:
        sizes, lens, hq, hkv, dt, qs = WORKLOADS[workload]
        nodes = ref_inputs.layered_tree(sizes, lens)
        desc = "N=%s C=%s" % (sizes, lens)
    batch = ref_inputs.assign_requests(nodes)
    ptrs = ref_inputs.kv_prefix_sums(nodes)
    return nodes, ptrs, batch, hq, hkv, dt, qs, desc


def to_product_tree(onodes):
    from kv_tree_simple import KVTreeNode
    tree = [KVTreeNode(n.parent, n.id, n.seqlen, n.num_children) for n in onodes]
    for nd, src in zip(tree, onodes):
        nd.requests = list(src.requests)
    return tree


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def measured_tensor_peak():
    """Dense bf16 TFLOP/s: the burst figure (the kernel is timed alone)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            return float(json.load(fh)["bf16_tflops"]), "measured"
    except Exception:
        return FALLBACK_BF16_TFLOPS, "fallback"


def recorded_traffic(workload, n_gpus):
    """DRAM bytes per stage-1 launch from the committed ncu capture, if one
    exists for this workload (profiles/ncu_traffic.json)."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as fh:
            rec = json.load(fh).get(f"{workload}@{n_gpus}gpu")
        return rec["dram_bytes_per_launch"] if rec else None
    except Exception:
        return None


class ClockSampler(threading.Thread):
    """Reads SM clock and throttle reasons through NVML while the GPU works
    (read-only queries)."""

    def __init__(self, index, period=0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def _once(self):
        nv = self.nv
        self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
        try:
            mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
        except Exception:
            mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
        names = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
                 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}
        for bit, name in names.items():
            if mask & bit:
                self.reasons.add(name)

    def run(self):
        if not self.ok:
            return
        while not self._stop_evt.is_set():
            try:
                self._once()
            except Exception:
                break
            self._stop_evt.wait(self.period)

    def finish(self):
        self._stop_evt.set()
        self.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        # idle samples (clock not yet ramped) are dropped: keep the upper half
        s = sorted(self.samples)
        load = s[len(s) // 2:]
        return {"sm_mhz": statistics.median(load), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def cpu_baseline_sample(nodes, ptrs, q, k, v, batch, budget_s=12.0, max_requests=None):
    """Oracle per-request attention on the host cores over a bounded sample of
    requests; returns (us per full step, description, cores)."""
    from oracle import ref_attention
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    scale = 1.0 / HEAD_DIM ** 0.5
    n = batch if max_requests is None else min(batch, max_requests)
    sample = [int(round(i * (batch - 1) / max(1, n - 1))) for i in range(n)] if n > 1 else [0]
    sample = sorted(set(sample))
    ref_attention.per_leaf_attention(nodes, ptrs, q, k, v, scale, requests=sample[:1])   # warm the allocator
    times = []
    t_all = time.perf_counter()
    while True:
        t0 = time.perf_counter()
        ref_attention.per_leaf_attention(nodes, ptrs, q, k, v, scale, requests=sample)
        times.append(time.perf_counter() - t0)
        if len(times) >= 3 and time.perf_counter() - t_all > budget_s or len(times) >= 50:
            break
    per_step_us = statistics.median(times) * batch / len(sample) * 1e6
    what = (f"{len(sample)} of {batch} requests (evenly spaced), median of {len(times)} runs, "
            f"scaled to the full step")
    return per_step_us, what, cores


def run_reference_arm(args):
    """--impl reference: the reference has no CPU implementation of this path and
    its Triton kernels cannot travel without the reference checkout, so the arm
    times the oracle's restatement of the reference's per-request PyTorch attention
    (path-concatenated K/V, fp32) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    nodes, ptrs, batch, hq, hkv, dt, qs, desc = build_tree(args.workload, args.seed)
    g = torch.Generator().manual_seed(args.seed)
    dtype = DTYPES[dt]
    k = torch.randn(ptrs[-1], hkv, HEAD_DIM, generator=g).to(dtype)
    v = torch.randn(ptrs[-1], hkv, HEAD_DIM, generator=g).to(dtype)
    q = (torch.randn(batch, hq, HEAD_DIM, generator=g) * qs).to(dtype)
    from oracle import ref_attention
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n = min(batch, args.ref_requests)
    sample = sorted(set(int(round(i * (batch - 1) / max(1, n - 1))) for i in range(n))) if n > 1 else [0]
    scale = 1.0 / HEAD_DIM ** 0.5
    for _ in range(args.warmup):
        ref_attention.per_leaf_attention(nodes, ptrs, q, k, v, scale, requests=sample)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ref_attention.per_leaf_attention(nodes, ptrs, q, k, v, scale, requests=sample)
    dt_s = (time.perf_counter() - t0) / args.steps
    us = dt_s * batch / len(sample) * 1e6
    what = f"{len(sample)} of {batch} requests per step (evenly spaced), scaled to the full step"
    line = {
        "impl": "reference", "metric": "tree_attn_decode_latency", "value": us, "unit": "us/step",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": us / 1e3,
        "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": dt, "data": "synthetic",
        "config": {"workload": f"{args.workload}: {desc}, {hq}q/{hkv}kv heads, head_dim {HEAD_DIM}, {dt}",
                   "requests": batch, "tokens": ptrs[-1]},
        "cpu_baseline": {"value": us, "unit": "us/step", "cores": cores, "kind": "port", "sample": what},
        "e2e": {"value": us, "unit": "us/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def emit(line):
    """The one JSON line goes to the process's original stdout; everything libraries print to fd 1
    (NCCL's version banner, for one) was redirected to stderr at start-up."""
    os.write(_JSON_FD, (json.dumps(line) + "\n").encode())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS) + sorted(RANDOM_WORKLOADS))
    ap.add_argument("--planner", default="b200", choices=["b200", "reference"])
    ap.add_argument("--path", default="auto", choices=["auto", "generic", "mma", "tcgen05"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--ref-requests", type=int, default=16, help="requests per step of the CPU arm")
    ap.add_argument("--prewarm-s", type=float, default=0.3, help="seconds of untimed steps before the warm-up (clock ramp)")
    ap.add_argument("--planner-opt", default="", help="comma-separated B200Model overrides, e.g. waves=3,min_chunk=64")
    ap.add_argument("--no-graph", action="store_true", help="launch every timed step from Python instead of a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--gather-output", action="store_true",
                    help="multi-GPU: all-gather the head-sharded outputs with NCCL inside every step")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch.distributed as dist
    import fasttree
    from ft_b200 import engine, lib, parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ["NCCL_DEBUG"] = os.environ.get("FT_BENCH_NCCL_DEBUG", "WARN")   # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=dev)
    lib.load()

    nodes, ptrs, batch, hq, hkv, dt, qs, desc = build_tree(args.workload, args.seed)
    dtype = DTYPES[dt]
    esize = 4 if dtype == torch.float32 else 2
    if hkv % world != 0:
        raise SystemExit(f"{hkv} kv heads cannot be sharded over {world} ranks")
    _q0, hq_l, _k0, hkv_l = parallel.head_shard(rank, world, hq, hkv)
    tokens = ptrs[-1]

    # ---- synthetic inputs, this rank's head slice, drawn on the device
    g = torch.Generator(device=dev).manual_seed(args.seed * 1000 + rank)
    kv_bytes = 2 * tokens * hkv_l * HEAD_DIM * esize
    copies = max(2, -(-2 * L2_BYTES // kv_bytes) + 1)
    copies = min(copies, 64)
    ks = [torch.randn(tokens, hkv_l, HEAD_DIM, generator=g, device=dev, dtype=torch.float32).to(dtype)
          for _ in range(copies)]
    vs = [torch.randn(tokens, hkv_l, HEAD_DIM, generator=g, device=dev, dtype=torch.float32).to(dtype)
          for _ in range(copies)]
    q = (torch.randn(batch, hq_l, HEAD_DIM, generator=g, device=dev, dtype=torch.float32) * qs).to(dtype)
    o = torch.empty_like(q)
    gather = world > 1 and args.gather_output
    o_all = torch.empty(world, batch, hq_l, HEAD_DIM, device=dev, dtype=dtype) if gather else None

    # ---- plan (host) with the LOCAL head counts
    params = fasttree.FastTreeParams()
    params.set_kv_group_num(hq_l // hkv_l)
    params.set_q_tile_sizes([max(1, 64 // (hq // hkv)), max(1, 16 // (hq // hkv))])
    params.set_kv_tile_sizes([32, 32])
    params.set_planner(args.planner)
    if args.planner_opt:
        from dataclasses import replace
        from ft_b200 import planner as ft_planner
        base = ft_planner.B200Model()
        if HEAD_DIM == 128:
            base = replace(base, rows_per_cta=128, ridge_flop_per_byte=4 * base.ridge_flop_per_byte)
        over = {}
        for kv in args.planner_opt.split(","):
            k, v = kv.split("=")
            over[k] = type(getattr(base, k))(float(v))
        params.b200_model = replace(base, **over)
    tree = to_product_tree(nodes)
    t0 = time.perf_counter()
    aux, _ = fasttree.fasttree_preparation(tree, ptrs, batch, hq_l, hkv_l, HEAD_DIM, [1024, 128], [132, 528],
                                           [132, 132], params, device=dev)
    plan_ms = (time.perf_counter() - t0) * 1e3
    tsq, tsk = list(params.TSQs), list(params.TSKs)
    scale = 1.0 / HEAD_DIM ** 0.5
    n_vnodes, n_rows = aux[1].numel(), aux[3].numel()

    def step(i):
        c = i % copies
        if args.path == "auto":
            fasttree.fasttree_decode(q, ks[c], vs[c], o, *aux, tsq, tsk, scale)
        else:
            engine.decode(q, ks[c], vs[c], o, *aux, tsq, tsk, scale, path=args.path)
        if gather:
            dist.all_gather_into_tensor(o_all, o)

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()

    # clock ramp-up and first-use costs (argument caches, NCCL channels), then W warm-up steps
    if world > 1:
        # every rank must issue the same number of collectives: a fixed count, not a time budget
        for i in range(int(args.prewarm_s * 4000)):
            step(i)
            if i % 64 == 63:
                torch.cuda.synchronize()
    else:
        t_end = time.perf_counter() + args.prewarm_s
        i = 0
        while time.perf_counter() < t_end:
            step(i)
            i += 1
            if i % 64 == 0:
                torch.cuda.synchronize()
    # The decode step is launch-bound from Python (a few microseconds of GPU work per call), so the
    # timed loop replays a CUDA graph holding `cycle` consecutive steps (one full K/V rotation or more).
    cycle = copies * max(1, -(-16 // copies))
    graph, launch_mode = None, "eager"
    launches_per_step = None
    if not args.no_graph and args.steps >= cycle:
        try:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for i in range(cycle):
                    step(i)
                side.synchronize()
                l0 = lib.launch_count()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for i in range(cycle):
                        step(i)
                launches_per_step = (lib.launch_count() - l0) / cycle
            torch.cuda.current_stream().wait_stream(side)
            launch_mode = f"cuda graph of {cycle} steps, replayed"
        except Exception as exc:                       # capture unsupported (e.g. a collective): launch eagerly
            graph, launch_mode = None, f"eager (graph capture failed: {type(exc).__name__})"
            torch.cuda.synchronize()

    def run_steps(n):
        if graph is None:
            for i in range(n):
                step(i)
            return
        for _ in range(n // cycle):
            graph.replay()
        for i in range(n % cycle):
            step(i)

    run_steps(max(args.warmup, cycle))
    fence()
    launches0 = lib.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    run_steps(args.steps)
    ev1.record()
    fence()
    if graph is None:
        launches = lib.launch_count() - launches0
    else:
        launches = int(round(launches_per_step * (args.steps // cycle) * cycle)) + (lib.launch_count() - launches0)
    elapsed_ms = ev0.elapsed_time(ev1)
    t = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = t.item() / args.steps

    # ---- dominant kernel (stage 1) timed alone, same rotation.  Launched back to back from a CUDA graph (events
    # around the replay, divided by the launches in it) so that Python's per-call time is not counted as kernel
    # time; eager launches with events around each one if capture is unavailable.
    n_rf = min(args.steps, 500)
    s1_ms, s1_timing = None, None
    if graph is not None:
        try:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                g1 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g1, stream=side):
                    for i in range(cycle):
                        engine.stage1(q, ks[i % copies], vs[i % copies], o, *aux, tsq, tsk, scale, path=args.path)
            torch.cuda.current_stream().wait_stream(side)
            reps = max(3, n_rf // cycle)
            g1.replay()
            fence()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                g1.replay()
            e1.record()
            fence()
            s1_ms = e0.elapsed_time(e1) / (reps * cycle)
            s1_timing = (f"mean over {reps * cycle} launches replayed from a CUDA graph of {cycle}, CUDA events around "
                         f"the replays, same KV rotation")
            del g1
        except Exception:
            s1_ms = None
            torch.cuda.synchronize()
    if s1_ms is None:
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_rf)]
        for i in range(n_rf):
            c = i % copies
            pairs[i][0].record()
            engine.stage1(q, ks[c], vs[c], o, *aux, tsq, tsk, scale, path=args.path)
            pairs[i][1].record()
            engine.stage2(q, ks[c], vs[c], o, *aux, tsq, tsk, scale)
        fence()
        s1_ms = statistics.mean(a.elapsed_time(b) for a, b in pairs)
        s1_timing = f"mean over {n_rf} launches, CUDA events around each stage-1 launch, same KV rotation"
    s1_path = engine.stage1_path_name(q, ks[0], vs[0], o, *aux, tsq, tsk, scale, path=args.path)
    algo_bytes = 2 * tokens * hkv_l * HEAD_DIM * esize + 2 * batch * hq_l * HEAD_DIM * esize
    peak, peak_kind = measured_peak()
    achieved = algo_bytes / (s1_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": recorded_traffic(args.workload, world), "peak_source": f"of {peak_kind}",
                "kernel": f"stage1_{s1_path}", "kernel_us": s1_ms * 1e3, "algorithmic_bytes": algo_bytes,
                "timing": s1_timing}
    # The same launch against the tensor roofline: 4*D flop per (query head, request, token on the request's path).
    # Whichever fraction is larger names the bound (a deep shared prefix with many requests is tensor-bound).
    depth = [0] * len(nodes)
    for i, nd in enumerate(nodes):
        depth[i] = nd.seqlen + (depth[nd.parent] if nd.parent >= 0 else 0)
    path_tokens = sum(depth[i] for i, nd in enumerate(nodes) if nd.num_children == 0)
    algo_flop = 4.0 * HEAD_DIM * hq_l * path_tokens
    tpeak, tpeak_kind = measured_tensor_peak()
    tflops = algo_flop / (s1_ms * 1e-3) / 1e12
    if tflops / tpeak > roofline["frac"]:
        roofline.update({"bound": "tensor", "achieved": tflops, "peak": tpeak, "unit": "TFLOP/s", "frac": tflops / tpeak,
                         "peak_source": f"of {tpeak_kind}", "algorithmic_flop": algo_flop,
                         "hbm_frac": achieved / peak})
    else:
        roofline["tensor_frac"] = tflops / tpeak

    # ---- end to end: query from pinned host memory in, output to pinned host memory out, every step
    e2e = None
    if not args.no_e2e:
        q_host = q.cpu().pin_memory()
        o_src = o_all if gather else o
        o_host = torch.empty(o_src.shape, dtype=dtype).pin_memory()
        n_e2e = min(args.steps, 1000)

        def e2e_step(i):
            q.copy_(q_host, non_blocking=True)
            step(i)
            o_host.copy_(o_src, non_blocking=True)
            torch.cuda.current_stream().synchronize()      # the next token depends on this output

        for i in range(min(args.warmup, 10)):
            e2e_step(i)
        fence()
        t0 = time.perf_counter()
        ev0.record()
        for i in range(n_e2e):
            e2e_step(i)
        ev1.record()
        fence()
        wall_ms = (time.perf_counter() - t0) * 1e3
        t = torch.tensor([max(ev0.elapsed_time(ev1), 0.0)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e = {"value": t.item() / n_e2e * 1e3, "unit": "us/step",
               "h2d_bytes_per_step": q_host.numel() * esize, "d2h_bytes_per_step": o_host.numel() * esize,
               "steps": n_e2e, "wall_us_per_step": wall_ms / n_e2e * 1e3,
               "call": "fasttree_decode(...) + NCCL all-gather" if gather else "fasttree_decode(...)"}
    clocks = sampler.finish()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        us, what, cores = cpu_baseline_sample(nodes, ptrs, q.cpu(), ks[0].cpu(), vs[0].cpu(), batch,
                                              max_requests=args.ref_requests)
        cpu = {"value": us, "unit": "us/step", "cores": cores, "kind": "port", "sample": what}

    if rank == 0:
        line = {
            "metric": "tree_attn_decode_latency", "value": ms_per_step * 1e3, "unit": "us/step",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": dt,
            "data": "synthetic (seeded N(0,1) Q/K/V drawn on the device, random-free tree shape)",
            "config": {
                "workload": f"{args.workload}: {desc}, {hq}q/{hkv}kv heads, head_dim {HEAD_DIM}, {dt}, "
                            f"one decode token per leaf",
                "requests": batch, "tokens": tokens, "planner": args.planner, "stage1_path": s1_path,
                "vnodes": n_vnodes, "partial_rows": n_rows, "plan_ms_host": plan_ms, "launch": launch_mode,
                "parallelism": (f"tp{world} (kv heads sharded, {hkv_l} per GPU; "
                                + ("outputs all-gathered with NCCL" if gather else "outputs stay head-sharded, no collective")
                                + ")") if world > 1 else "single GPU",
                "l2": f"K/V rotated over {copies} copies = {copies * kv_bytes / 2 ** 20:.0f} MiB per GPU (> 126 MiB L2)",
            },
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks,
            "gpu_launches": launches * world,
            "hbm_gbs_whole_step": algo_bytes * world / (ms_per_step * 1e-3) / 1e9,
        }
        emit(line)
    if world > 1:
        # drop the captured graph (it holds NCCL work) before tearing the group down; never hang on exit
        graph = None
        import gc
        gc.collect()
        torch.cuda.synchronize()
        watchdog = threading.Timer(30.0, lambda: os._exit(0))
        watchdog.daemon = True
        watchdog.start()
        dist.barrier()
        dist.destroy_process_group()
        watchdog.cancel()


if __name__ == "__main__":
    main()
