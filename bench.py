#!/usr/bin/env python
"""Decode-step benchmark of the B200 tree-attention engine.

    python bench.py --gpus N --steps K --warmup W            # this engine
    python bench.py --impl reference --steps K --warmup W    # CPU baseline arm

A step is one tree-attention decode call (one layer) over a synthetic radix
tree.  Default workload: N=[1,64] nodes per level, C=[4096,256] tokens per
node, 32 query / 8 KV heads, head_dim 128, fp16 - 64 decode requests sharing a
4096-token prefix.  Under torchrun the KV heads are sharded across ranks
(tensor parallel); the attention itself needs no exchange, and the step is
timed both without a collective (``value``: the output stays head-sharded, as
it does where it feeds a row-parallel projection) and with an NCCL all-gather
of the heads inside every step (``with_gather_us``).

Prints ONE JSON line on rank 0.  ``value`` is microseconds per step with
everything resident in HBM (median over the timed regions, each region exactly
``--steps`` steps replayed from a CUDA graph, max over ranks); ``e2e`` is the
same step fed from pinned host memory (query copied in, output copied out,
every step); ``roofline`` relates the stage-1 kernel to the measured HBM copy
bandwidth (or the tensor peak where that fraction is larger); ``cpu_baseline``
is the oracle's per-request path-concatenated attention on the host cores;
``reference_triton`` is the reference's own Triton kernels timed on the same
GPU and tensors; ``parity_max_abs`` is the largest deviation from the fp32
oracle on a sample of requests, checked before anything is timed;
``workloads`` repeats value / roofline / with_gather_us / parity for the other
head-sharded configurations.
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
GRAPH_CHUNK = 250         # steps per captured graph; longer timed regions replay it several times
PARITY_TOL = 2e-3         # 16-bit storage, max-abs against the fp32 oracle (bf16: plus one output ulp)


def build_tree(workload, seed):
    """The benchmark tree from the shipped generators (kernel_bench/tree_generation.py), with requests assigned."""
    import kv_tree_simple
    import tree_generation
    if workload in RANDOM_WORKLOADS:
        rows = tree_generation.generate_random_tree(RANDOM_WORKLOADS[workload], seed)
        hq, hkv, dt, qs = 32, 8, "fp16", 1.0
        desc = f"random tree, {RANDOM_WORKLOADS[workload]} node levels, seed {seed}"
    else:
        sizes, lens, hq, hkv, dt, qs = WORKLOADS[workload]
        rows = tree_generation.generate_tree(sizes, lens)
        desc = "N=%s C=%s" % (sizes, lens)
    nodes = kv_tree_simple.tree_from_rows(rows)
    batch, ptrs = kv_tree_simple.assign_requests(nodes)
    return nodes, ptrs, batch, hq, hkv, dt, qs, desc


def workload_label(workload, desc, hq, hkv, dt):
    """Identical in both arms, so that their lines name the same configuration."""
    return f"{workload}: {desc}, {hq}q/{hkv}kv heads, head_dim {HEAD_DIM}, {dt}, one decode token per leaf"


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


def even_sample(batch, n):
    n = min(batch, n)
    if n <= 1:
        return [0]
    return sorted(set(int(round(i * (batch - 1) / (n - 1))) for i in range(n)))


def cpu_baseline_sample(nodes, ptrs, q, k, v, batch, budget_s=12.0, max_requests=None):
    """Oracle per-request attention on the host cores over a bounded sample of
    requests; returns (us per full step, description, cores)."""
    from oracle import ref_attention
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    scale = 1.0 / HEAD_DIM ** 0.5
    sample = even_sample(batch, batch if max_requests is None else max_requests)
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
    """--impl reference: the reference has no CPU implementation of this path (its kernels are Triton), so the
    arm times the oracle's restatement of the reference's per-request PyTorch attention (path-concatenated K/V,
    fp32) on the host cores.  The reference's Triton kernels on the GPU are a leg of the engine's own line
    (``reference_triton``)."""
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
    sample = even_sample(batch, args.ref_requests)
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
        "config": {"workload": workload_label(args.workload, desc, hq, hkv, dt)},
        "cpu_baseline": {"value": us, "unit": "us/step", "cores": cores, "kind": "port", "sample": what},
        "e2e": {"value": us, "unit": "us/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "extra": {"requests": batch, "tokens": ptrs[-1]},
    }
    emit(line)


def emit(line):
    """The one JSON line goes to the process's original stdout; everything libraries print to fd 1
    (NCCL's version banner, for one) was redirected to stderr at start-up."""
    os.write(_JSON_FD, (json.dumps(line) + "\n").encode())


class Ctx:
    """Process-wide state of one benchmark run."""

    def __init__(self, args):
        import torch.distributed as dist
        self.args = args
        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device; there is no CPU path (use --impl reference for the CPU arm)")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)     # NCCL_DEBUG is left as the caller set it

    def fence(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, values):
        t = torch.tensor(list(values), device=self.dev, dtype=torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.tolist()


def capture_steps(ctx, step_fn, steps, count_launches=None):
    """CUDA graphs that together hold EXACTLY ``steps`` consecutive steps (rotation order preserved): a chunk of up
    to GRAPH_CHUNK steps replayed ``steps // chunk`` times plus a tail graph for the remainder.  The decode step is
    a few microseconds of GPU work, so launching it from Python would time Python.  Returns (replay function,
    description, launches per step) or (None, reason, None) when capture is not possible."""
    chunk = min(steps, GRAPH_CHUNK)
    tail = steps % chunk
    try:
        side = torch.cuda.Stream(device=ctx.dev)
        side.wait_stream(torch.cuda.current_stream())
        graphs = []
        per_step = None
        with torch.cuda.stream(side):
            for i in range(min(chunk, 8)):
                step_fn(i)                       # first-use costs outside the capture
            side.synchronize()
            for first, n in ((0, chunk), ((steps // chunk) * chunk, tail)):
                if n == 0:
                    continue
                l0 = count_launches() if count_launches else 0
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for i in range(first, first + n):
                        step_fn(i)
                if count_launches and per_step is None:
                    per_step = (count_launches() - l0) / n
                graphs.append((g, n))
        torch.cuda.current_stream().wait_stream(side)
    except Exception as exc:
        torch.cuda.synchronize()
        return None, f"eager (graph capture failed: {type(exc).__name__}: {exc})", None
    full = steps // chunk

    def replay():
        for _ in range(full):
            graphs[0][0].replay()
        if tail:
            graphs[-1][0].replay()

    what = f"cuda graph of {chunk} steps" + (f" x{full}" if full > 1 else "") + (f" + {tail}" if tail else "") + ", replayed"
    return replay, what, per_step


def time_regions(ctx, step_fn, steps, regions, count_launches=None, allow_graph=True):
    """``regions`` timed regions of exactly ``steps`` steps each, every region bracketed by a barrier and a
    device synchronisation on both sides and timed with CUDA events on the launching stream; per region the
    maximum over ranks, then the median over regions.  Returns a dict with us per step and how it was launched."""
    replay, mode, per_step = (None, "eager (--no-graph)", None)
    if allow_graph:
        replay, mode, per_step = capture_steps(ctx, step_fn, steps, count_launches)
    if replay is None:
        def replay():
            for i in range(steps):
                step_fn(i)
    replay()                      # one untimed region: the graph's first replay uploads it
    times = []
    launches = None
    for r in range(regions):
        ctx.fence()
        l0 = count_launches() if count_launches else 0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        replay()
        e1.record()
        ctx.fence()
        times.append(e0.elapsed_time(e1))
        if count_launches and launches is None:
            launches = count_launches() - l0
    times = ctx.max_over_ranks(times)
    med = statistics.median(times)
    if per_step is not None:
        launches = int(round(per_step * steps))
    return {"us": med / steps * 1e3, "min_us": min(times) / steps * 1e3, "max_us": max(times) / steps * 1e3,
            "mode": mode, "regions": regions, "launches_per_region": launches, "graph": per_step is not None}


class Problem:
    """One workload planned and resident on this rank's GPU (its head slice)."""

    def __init__(self, ctx, workload):
        import fasttree
        from ft_b200 import engine, parallel
        args = ctx.args
        self.ctx, self.workload = ctx, workload
        self.fasttree, self.engine = fasttree, engine
        nodes, ptrs, batch, hq, hkv, dt, qs, desc = build_tree(workload, args.seed)
        self.nodes, self.ptrs, self.batch, self.hq, self.hkv, self.dt, self.desc = nodes, ptrs, batch, hq, hkv, dt, desc
        self.dtype = DTYPES[dt]
        self.esize = 4 if self.dtype == torch.float32 else 2
        world, rank, dev = ctx.world, ctx.rank, ctx.dev
        if hkv % world != 0:
            raise SystemExit(f"{workload}: {hkv} kv heads cannot be sharded over {world} ranks")
        _q0, self.hq_l, _k0, self.hkv_l = parallel.head_shard(rank, world, hq, hkv)
        self.tokens = ptrs[-1]

        # ---- synthetic inputs, this rank's head slice, drawn on the device
        g = torch.Generator(device=dev).manual_seed(args.seed * 1000 + rank)
        self.kv_bytes = 2 * self.tokens * self.hkv_l * HEAD_DIM * self.esize
        copies = max(2, -(-2 * L2_BYTES // self.kv_bytes) + 1)
        self.copies = copies = min(copies, 64)

        def draw(*shape):
            return torch.randn(*shape, generator=g, device=dev, dtype=torch.float32)

        if args.kv_layout == "head_major":     # [Hkv, T, D] storage handed to the engine as a strided [T, Hkv, D] view
            self.ks = [draw(self.hkv_l, self.tokens, HEAD_DIM).to(self.dtype).transpose(0, 1) for _ in range(copies)]
            self.vs = [draw(self.hkv_l, self.tokens, HEAD_DIM).to(self.dtype).transpose(0, 1) for _ in range(copies)]
        else:                                  # the reference's layout: [T, Hkv, D], packed
            self.ks = [draw(self.tokens, self.hkv_l, HEAD_DIM).to(self.dtype) for _ in range(copies)]
            self.vs = [draw(self.tokens, self.hkv_l, HEAD_DIM).to(self.dtype) for _ in range(copies)]
        self.q = (draw(batch, self.hq_l, HEAD_DIM) * qs).to(self.dtype)
        self.o = torch.empty_like(self.q)
        self.o_all = torch.empty(world, batch, self.hq_l, HEAD_DIM, device=dev, dtype=self.dtype) if world > 1 else None

        # ---- plan (host) with the LOCAL head counts
        params = fasttree.FastTreeParams()
        params.set_kv_group_num(self.hq_l // self.hkv_l)
        params.set_q_tile_sizes([max(1, 64 // (hq // hkv)), max(1, 16 // (hq // hkv))])
        params.set_kv_tile_sizes([32, 32])
        params.set_kv_dtype(self.dtype)
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
        t0 = time.perf_counter()
        self.aux, _ = fasttree.fasttree_preparation(nodes, ptrs, batch, self.hq_l, self.hkv_l, HEAD_DIM, [1024, 128],
                                                    [132, 528], [132, 132], params, device=dev)
        self.plan_ms = (time.perf_counter() - t0) * 1e3
        self.tsq, self.tsk = list(params.TSQs), list(params.TSKs)
        self.scale = 1.0 / HEAD_DIM ** 0.5
        self.n_vnodes, self.n_rows = self.aux[1].numel(), self.aux[9].shape[0]
        self.path = args.path

    # ---- the step, on K/V copy i of the rotation
    def step(self, i):
        c = i % self.copies
        if self.path == "auto":
            self.fasttree.fasttree_decode(self.q, self.ks[c], self.vs[c], self.o, *self.aux, self.tsq, self.tsk, self.scale)
        else:
            self.engine.decode(self.q, self.ks[c], self.vs[c], self.o, *self.aux, self.tsq, self.tsk, self.scale,
                               path=self.path)

    def step_gather(self, i):
        self.step(i)
        self.ctx.dist.all_gather_into_tensor(self.o_all, self.o)

    def stage1(self, i):
        c = i % self.copies
        self.engine.stage1(self.q, self.ks[c], self.vs[c], self.o, *self.aux, self.tsq, self.tsk, self.scale, path=self.path)

    def stage1_name(self):
        return self.engine.stage1_path_name(self.q, self.ks[0], self.vs[0], self.o, *self.aux, self.tsq, self.tsk,
                                            self.scale, path=self.path)

    def label(self):
        return workload_label(self.workload, self.desc, self.hq, self.hkv, self.dt)

    def algo_bytes(self):
        return 2 * self.tokens * self.hkv_l * HEAD_DIM * self.esize + 2 * self.batch * self.hq_l * HEAD_DIM * self.esize

    def algo_flop(self):
        depth = [0] * len(self.nodes)
        for i, nd in enumerate(self.nodes):
            depth[i] = nd.seqlen + (depth[nd.parent] if nd.parent >= 0 else 0)
        path_tokens = sum(depth[i] for i, nd in enumerate(self.nodes) if nd.num_children == 0)
        return 4.0 * HEAD_DIM * self.hq_l * path_tokens

    # ---- checks and legs
    def parity(self, n_requests=8):
        """This rank's output on K/V copy 0 against the fp32 oracle on a sample of requests (its own head slice)."""
        from oracle import ref_attention
        from ft_b200 import lib
        self.o.fill_(float("nan"))
        self.step(0)
        torch.cuda.synchronize()
        if lib.read_device_status() != 0:
            raise SystemExit(f"{self.workload}: the kernels flagged bad plan data")
        sample = even_sample(self.batch, n_requests)
        idx = torch.tensor(sample, device=self.ctx.dev)
        truth, _ = ref_attention.per_leaf_attention(self.nodes, self.ptrs, self.q.cpu(), self.ks[0].cpu(), self.vs[0].cpu(),
                                                    self.scale, requests=sample)
        got = self.o.index_select(0, idx).float().cpu()
        err = (got - truth).abs().max().item()
        if not (err == err):
            raise SystemExit(f"{self.workload}: NaN in the output")
        tol = PARITY_TOL + (float(truth.abs().max()) * 2 ** -8 if self.dtype == torch.bfloat16 else 0.0)
        if self.dtype == torch.float32:
            tol = 2e-5
        return err, tol, len(sample)

    def roofline(self, steps, regions, allow_graph):
        from ft_b200 import lib
        t = time_regions(self.ctx, self.stage1, steps, regions, lib.launch_count, allow_graph)
        s1_us = t["us"]
        launches_per_step = (t["launches_per_region"] or steps) / steps
        kernel_us = s1_us / max(1.0, launches_per_step)      # average launch duration when stage 1 is two launches
        algo_bytes = self.algo_bytes()
        peak, peak_kind = measured_peak()
        achieved = algo_bytes / (s1_us * 1e-6) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": recorded_traffic(self.workload, self.ctx.world), "peak_source": f"of {peak_kind}",
                "kernel": self.stage1_name(), "kernel_us": s1_us, "launches_per_step": launches_per_step,
                "avg_launch_us": kernel_us, "algorithmic_bytes": algo_bytes,
                "timing": (f"stage 1 alone, {t['mode']}; median of {regions} regions of {steps} launches, CUDA events "
                           f"around each region, same K/V rotation")}
        # The same launch against the tensor roofline: 4*D flop per (query head, request, token on the request's
        # path).  Whichever fraction is larger names the bound (a deep shared prefix with many requests is
        # tensor-bound).
        algo_flop = self.algo_flop()
        tpeak, tpeak_kind = measured_tensor_peak()
        tflops = algo_flop / (s1_us * 1e-6) / 1e12
        if tflops / tpeak > roof["frac"]:
            roof.update({"bound": "tensor", "achieved": tflops, "peak": tpeak, "unit": "TFLOP/s", "frac": tflops / tpeak,
                         "peak_source": f"of {tpeak_kind}", "algorithmic_flop": algo_flop, "hbm_frac": achieved / peak})
        else:
            roof["tensor_frac"] = tflops / tpeak
        return roof

    def reference_triton(self, engine_us, steps, regions):
        """The reference's own planner + Triton kernels on the same tensors of this GPU (baseline leg; the staged
        reference files are test infrastructure and take no part in the engine's path)."""
        from oracle import ref_triton
        ok, why = ref_triton.availability()
        if not ok:
            return {"unavailable": why}
        if self.dtype == torch.float32 and self.workload != "cfg1":
            return {"unavailable": "fp32 workload"}
        try:
            ref = ref_triton.ReferenceRun(self.nodes, self.ptrs, self.batch, self.hq_l, self.hkv_l, HEAD_DIM)
            o_ref = torch.empty_like(self.q)

            def ref_step(i):
                c = i % self.copies
                ref.decode(self.q, self.ks[c], self.vs[c], o_ref)

            ref_step(0)                           # JIT compile
            torch.cuda.synchronize()
            self.step(0)
            torch.cuda.synchronize()
            diff = (o_ref.float() - self.o.float()).abs().max().item()
            n = max(1, min(steps, 100))
            t = time_regions(self.ctx, ref_step, n, max(3, min(regions, 10)))
            # the reference's own way of launching: eager calls from Python, back to back
            for i in range(5):
                ref_step(i)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(n):
                ref_step(i)
            e1.record()
            torch.cuda.synchronize()
            eager_us = e0.elapsed_time(e1) / n * 1e3
            return {"value_us": t["us"], "launch": t["mode"], "eager_us": eager_us, "ratio": t["us"] / engine_us,
                    "max_abs_vs_engine": diff, "vnodes": ref.vnodes, "partial_rows": ref.partial_rows,
                    "q_tiles": ref.tsq, "kv_tiles": ref.tsk,
                    "what": "reference planner (CLI defaults) + Triton stage-1/stage-2 kernels, same tensors and "
                            "K/V rotation; ratio = reference / engine"}
        except Exception as exc:                  # a reference that cannot run here is reported, not fatal
            torch.cuda.synchronize()
            return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}

    def e2e(self, steps, warmup):
        """Query from pinned host memory in, output to pinned host memory out, every step, through the
        reference-signature host-I/O entry point (one C-ABI call: copy in, decode, copy out, synchronise)."""
        ctx = self.ctx
        q_host = self.q.cpu().pin_memory()
        o_host = torch.empty(self.o.shape, dtype=self.dtype).pin_memory()
        n_e2e = min(steps, 1000)

        def e2e_step(i):
            c = i % self.copies
            self.fasttree.fasttree_decode_host_io(q_host, self.ks[c], self.vs[c], o_host, *self.aux, self.tsq, self.tsk,
                                                  self.scale)      # returns when o_host is valid

        for i in range(max(3, min(warmup, 10))):
            e2e_step(i)
        ctx.fence()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        ev0.record()
        for i in range(n_e2e):
            e2e_step(i)
        ev1.record()
        ctx.fence()
        wall_ms = (time.perf_counter() - t0) * 1e3
        dev_ms = ctx.max_over_ranks([max(ev0.elapsed_time(ev1), 0.0)])[0]
        return {"value": dev_ms / n_e2e * 1e3, "unit": "us/step",
                "h2d_bytes_per_step": q_host.numel() * self.esize, "d2h_bytes_per_step": o_host.numel() * self.esize,
                "steps": n_e2e, "wall_us_per_step": wall_ms / n_e2e * 1e3,
                "call": "fasttree_decode_host_io(...): ft_decode_host_io = query fetched from pinned (mapped) host "
                        "memory by a copy kernel, stage 1, stage 2 writing the output rows into pinned host memory, "
                        "stream synchronise - one C-ABI call per step"}

    def release(self):
        self.ks = self.vs = None
        self.aux = None
        self.engine._ARG_CACHE.clear()
        torch.cuda.empty_cache()


def measure(ctx, workload, primary):
    """All device-side legs of one workload.  Returns the dict that goes into the line."""
    from ft_b200 import lib
    args = ctx.args
    p = Problem(ctx, workload)
    allow_graph = not args.no_graph
    regions = args.regions
    out = {"workload": p.label()}

    err, tol, n_checked = p.parity()
    errs = ctx.max_over_ranks([err, tol])
    out["parity_max_abs"] = errs[0]
    out["parity"] = {"max_abs": errs[0], "tolerance": errs[1], "requests_checked_per_rank": n_checked,
                     "against": "fp32 per-request oracle on this rank's head slice, before timing"}
    if errs[0] > errs[1]:
        raise SystemExit(f"{workload}: parity check failed before timing: max-abs {errs[0]} > {errs[1]}")

    # clock ramp-up and first-use costs (argument caches, NCCL channels): a fixed count on every rank
    for i in range(max(args.warmup, int(args.prewarm_s * 4000))):
        p.step(i)
        if i % 64 == 63:
            torch.cuda.synchronize()
    ctx.fence()
    t = time_regions(ctx, p.step, args.steps, regions, lib.launch_count, allow_graph)
    out.update({"value": t["us"], "region_min_us": t["min_us"], "region_max_us": t["max_us"], "launch": t["mode"],
                "launches_per_region": t["launches_per_region"]})
    out["with_gather_us"] = None
    if ctx.world > 1:
        for i in range(max(args.warmup, 20)):
            p.step_gather(i)
        tg = time_regions(ctx, p.step_gather, args.steps, regions, None, allow_graph)
        out["with_gather_us"] = tg["us"]
        out["with_gather_launch"] = tg["mode"]
    out["roofline"] = p.roofline(min(args.steps, GRAPH_CHUNK), regions, allow_graph)
    out["plan"] = {"planner": args.planner, "vnodes": p.n_vnodes, "partial_rows": p.n_rows, "plan_ms_host": p.plan_ms,
                   "requests": p.batch, "tokens": p.tokens}
    out["kv_layout"] = args.kv_layout
    out["l2"] = f"K/V rotated over {p.copies} copies = {p.copies * p.kv_bytes / 2 ** 20:.0f} MiB per GPU (> 126 MiB L2)"
    out["hbm_gbs_whole_step"] = p.algo_bytes() * ctx.world / (t["us"] * 1e-6) / 1e9
    if ctx.world == 1 and not args.no_reference_triton:
        out["reference_triton"] = p.reference_triton(t["us"], args.steps, regions)
    elif not args.no_reference_triton:
        out["reference_triton"] = {"unavailable": "measured at 1 GPU only (the baseline leg is not sharded)"}
    if primary:
        out["e2e"] = None if args.no_e2e else p.e2e(args.steps, args.warmup)
        out["cpu"] = None
        if ctx.rank == 0 and ctx.world == 1 and not args.no_cpu_baseline:
            us, what, cores = cpu_baseline_sample(p.nodes, p.ptrs, p.q.cpu(), p.ks[0].cpu(), p.vs[0].cpu(), p.batch,
                                                  max_requests=args.ref_requests)
            out["cpu"] = {"value": us, "unit": "us/step", "cores": cores, "kind": "port", "sample": what}
        out["dt"], out["hkv_l"] = p.dt, p.hkv_l
    p.release()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS) + sorted(RANDOM_WORKLOADS))
    ap.add_argument("--also", default="cfg3,cfg4",
                    help="comma-separated further workloads reported under 'workloads' (value, roofline, with_gather_us); "
                         "'' for none")
    ap.add_argument("--regions", type=int, default=20, help="timed regions of --steps steps each; the median is reported")
    ap.add_argument("--planner", default="b200", choices=["b200", "reference"])
    ap.add_argument("--path", default="auto", choices=["auto", "generic", "mma", "mma_wide", "tcgen05", "stream", "persist"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--kv-layout", default="token_major", choices=["token_major", "head_major"],
                    help="token_major: K/V stored [T, Hkv, D] as the reference's tree tensors and SGLang's pool are; "
                         "head_major: stored [Hkv, T, D] and passed as a strided view (an experiment on DRAM locality)")
    ap.add_argument("--ref-requests", type=int, default=16, help="requests per step of the CPU arm")
    ap.add_argument("--prewarm-s", type=float, default=0.3, help="seconds' worth of untimed steps before the warm-up (clock ramp)")
    ap.add_argument("--planner-opt", default="", help="comma-separated B200Model overrides, e.g. waves=3,min_chunk=64")
    ap.add_argument("--no-graph", action="store_true", help="launch every timed step from Python instead of a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-reference-triton", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.regions < 1:
        args.regions = 1
    if args.impl == "reference":
        run_reference_arm(args)
        return

    from ft_b200 import lib
    ctx = Ctx(args)
    lib.load()
    sampler = ClockSampler(ctx.local_rank)
    sampler.start()

    main_out = measure(ctx, args.workload, primary=True)
    others = {}
    for name in [w for w in args.also.split(",") if w and w != args.workload]:
        if name not in WORKLOADS and name not in RANDOM_WORKLOADS:
            raise SystemExit(f"unknown workload {name}")
        nodes, ptrs, batch, hq, hkv, dt, qs, desc = build_tree(name, args.seed)
        if hkv % ctx.world != 0:
            continue
        o = measure(ctx, name, primary=False)
        others[name] = {k: o[k] for k in ("workload", "value", "with_gather_us", "roofline", "parity_max_abs", "launch",
                                          "plan", "reference_triton") if k in o}
        others[name]["unit"] = "us/step"
    clocks = sampler.finish()

    world = ctx.world
    if ctx.rank == 0:
        m = main_out
        line = {
            "metric": "tree_attn_decode_latency", "value": m["value"], "unit": "us/step",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": m["value"] / 1e3,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": m["dt"],
            "data": "synthetic (seeded N(0,1) Q/K/V drawn on the device, tree from the shipped generator)",
            "gpu_launches": (m["launches_per_region"] or 0) * world,
            "config": {"workload": m["workload"]},
            "run": {
                "regions": args.regions, "region_min_us": m["region_min_us"], "region_max_us": m["region_max_us"],
                "launch": m["launch"], "l2": m["l2"], **m["plan"],
                "parallelism": (f"tp{world} (kv heads sharded, {m['hkv_l']} per GPU; value: outputs stay head-sharded, "
                                f"no collective; with_gather_us: NCCL all-gather of the heads inside every step)")
                if world > 1 else "single GPU",
            },
            "roofline": m["roofline"], "cpu_baseline": m["cpu"], "e2e": m["e2e"], "clocks": clocks,
            "with_gather_us": m["with_gather_us"], "parity_max_abs": m["parity_max_abs"], "parity": m["parity"],
            "reference_triton": m.get("reference_triton"),
            "hbm_gbs_whole_step": m["hbm_gbs_whole_step"],
            "workloads": others,
        }
        emit(line)
    if world > 1:
        # captured graphs hold NCCL work: they were dropped with their Problem; never hang on exit
        import gc
        gc.collect()
        torch.cuda.synchronize()
        watchdog = threading.Timer(30.0, lambda: os._exit(0))
        watchdog.daemon = True
        watchdog.start()
        ctx.dist.barrier()
        ctx.dist.destroy_process_group()
        watchdog.cancel()


if __name__ == "__main__":
    main()
