"""GPU parity tests: the CUDA path, called through the C ABI, against
(a) the outputs the reference's own kernels wrote (golden fixtures),
(b) the CPU oracle on the same seeded inputs, and
(c) size-independent properties at the benchmark sizes.

Tolerances (stated once): 16-bit storage - max-abs error <= 2e-3 against the
fp32 ground truth and against the reference's output; partial and merged LSE
within 1e-4 relative (+1e-5 absolute).  fp32 storage - 2e-5.
"""
import numpy as np
import pytest
import torch

import cases
import gpu_utils
from oracle import ref_attention, ref_inputs

import fasttree
from ft_b200 import engine, lib

pytestmark = pytest.mark.gpu

ATOL16 = 2e-3
ATOL32 = 2e-5


def atol_for(dtype):
    return ATOL32 if dtype == torch.float32 else ATOL16


def paths_for(c):
    fast = c["dtype"] != torch.float32 and c["d"] in (64, 128)
    if not fast:
        return ["generic", "auto"]      # fp32 storage: the scalar kernel, and the tiled fp32 kernel that "auto" picks
    return ["generic", "mma", "mma_wide", "stream"] + (["tcgen05", "persist", "auto"] if c["d"] == 128 else [])


SMALL = [n for n in cases.DECODE_CASES if n != "cfg2_fp16"]


@pytest.mark.parametrize("name", SMALL)
@pytest.mark.parametrize("planner", ["reference", "b200"])
def test_golden_cases_match_reference_output(name, planner):
    c = cases.build_decode_case(name)
    gold = c["gold"]
    scale = 1.0 / c["d"] ** 0.5
    truth, truth_lse = ref_attention.per_leaf_attention(c["nodes"], c["ptrs"], c["q"], c["k"], c["v"], scale)
    tol = atol_for(c["dtype"])
    for path in paths_for(c):
        run, out = gpu_utils.run_case(c, planner=planner, path=path)
        assert lib.read_device_status() == 0
        assert torch.isfinite(out).all(), (name, planner, path)
        assert (out - torch.from_numpy(gold["o"])).abs().max().item() <= tol, (name, planner, path)
        assert (out - truth).abs().max().item() <= tol, (name, planner, path)
        np.testing.assert_allclose(run.o_lse.cpu().numpy(), truth_lse.numpy(), rtol=1e-4, atol=1e-5)
        if planner == "reference":
            # same plan as the reference -> the partial buffers are comparable row by row
            for tname, t in zip(cases.TABLES, run.aux[:9]):
                np.testing.assert_array_equal(t.cpu().numpy(), gold[tname], err_msg=tname)
            np.testing.assert_allclose(run.mid_lse.cpu().numpy(), gold["mid_lse"], rtol=1e-4, atol=1e-5)
            assert np.abs(run.mid_o.cpu().numpy() - gold["mid_o"]).max() <= tol


@pytest.mark.parametrize("planner", ["reference", "b200"])
def test_bf16_case(planner):
    """bf16 storage; the fixture holds the reference kernels' result on the exact
    fp32 up-cast of the same bf16 tensors."""
    c = cases.build_decode_case("mini3_bf16_as_fp32")
    assert c["dtype"] == torch.bfloat16
    for path in ("generic", "mma", "mma_wide", "stream", "tcgen05", "persist", "auto"):
        _, out = gpu_utils.run_case(c, planner=planner, path=path)
        # the output itself is rounded to bf16 (8 bits of mantissa): allow one bf16 ulp of the largest value
        bound = ATOL16 + float(np.abs(c["gold"]["o"]).max()) * 2 ** -8
        assert (out - torch.from_numpy(c["gold"]["o"])).abs().max().item() <= bound, path


@pytest.mark.parametrize("planner", ["reference", "b200"])
def test_full_size_fp16_config(planner):
    """Benchmark configuration 2 (N=[1,64], C=[4096,256], 32/8 heads, fp16) at full
    size against the reference kernels' output and the fp32 ground truth."""
    c = cases.build_decode_case("cfg2_fp16")
    truth, truth_lse = ref_attention.per_leaf_attention(c["nodes"], c["ptrs"], c["q"], c["k"], c["v"],
                                                        1.0 / 128 ** 0.5)
    run, out = gpu_utils.run_case(c, planner=planner, path="auto")
    assert lib.read_device_status() == 0
    assert (out - truth).abs().max().item() <= ATOL16
    assert (out - torch.from_numpy(c["gold"]["o"].astype(np.float32))).abs().max().item() <= ATOL16
    np.testing.assert_allclose(run.o_lse.cpu().numpy(), truth_lse.numpy(), rtol=1e-4, atol=1e-5)
    if planner == "reference":
        np.testing.assert_allclose(run.mid_lse.cpu().numpy(), c["gold"]["mid_lse"], rtol=1e-4, atol=1e-5)
    # the reference-signature entry point gives the same bits as the explicit call
    again = run.decode_via_dropin()
    assert torch.equal(again, out)


def adhoc(sizes, lens, hq, hkv, d, dtype, seed, q_scale=1.0):
    nodes = ref_inputs.layered_tree(sizes, lens)
    q, k, v, ptrs, batch = ref_inputs.draw_qkv(nodes, hq, hkv, d, dtype, seed, q_scale)
    return dict(nodes=nodes, q=q, k=k, v=v, ptrs=ptrs, batch=batch, hq=hq, hkv=hkv, d=d, dtype=dtype,
                tsq=cases.q_tiles_for_group(hq // hkv))


EDGE_TREES = [
    # (level sizes, level lens, hq, hkv, d)           what it exercises
    ([1], [1], 4, 4, 128),                            # single node, single token
    ([1], [300], 8, 8, 128),                          # single node, several tiles + tail
    ([1, 3, 9], [1, 1, 1], 16, 4, 128),               # one-token nodes
    ([1, 5], [63, 65], 8, 2, 128),                    # kv_len = tile -+ 1
    ([1, 5], [64, 128], 8, 2, 64),                    # exact tiles, head_dim 64
    ([1, 15], [200, 7], 32, 8, 128),                  # 15 requests x G=4 = 60 rows: last row block ragged
    ([1, 17], [130, 9], 32, 8, 128),                  # 17 requests -> two request tiles (16 + 1)
    ([1, 3], [90, 40], 64, 8, 128),                   # G=8: 24 rows -> two warps per row block
    ([1, 9], [150, 33], 24, 8, 128),                  # G=3: rows do not align with 16-row blocks
    ([1, 2, 4], [40, 30, 20], 16, 16, 64),            # MHA, head_dim 64
    ([1, 2], [700, 20], 128, 1, 128),                 # G=128: one request spans two 64-row blocks
    ([1, 600], [10, 33], 32, 32, 128),                # 19200 one-tile tasks: the persistent kernel walks > 48 per CTA
    ([1, 40], [70, 20], 32, 8, 128),                  # B200 plan: 40 short leaves -> groups of <= 32 requests, ragged ranges
    ([1, 4, 64], [100, 50, 12], 32, 32, 128),         # B200 plan: MHA, groups of 21 twelve-token leaves
    ([1, 3, 24], [30, 129, 31], 16, 4, 128),          # B200 plan: members that straddle tile boundaries
]


@pytest.mark.parametrize("spec", EDGE_TREES, ids=lambda s: "n%s_c%s_h%d-%d_d%d" % (
    "-".join(map(str, s[0])), "-".join(map(str, s[1])), s[2], s[3], s[4]))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32], ids=["fp16", "bf16", "fp32"])
def test_edge_shapes_against_oracle(spec, dtype):
    sizes, lens, hq, hkv, d = spec
    c = adhoc(sizes, lens, hq, hkv, d, dtype, seed=3, q_scale=0.5)
    scale = 1.0 / d ** 0.5
    truth, truth_lse = ref_attention.per_leaf_attention(c["nodes"], c["ptrs"], c["q"], c["k"], c["v"], scale)
    tol = atol_for(dtype)
    if dtype == torch.bfloat16:
        tol += float(truth.abs().max()) * 2 ** -8     # output rounding to bf16
    # fp32 storage additionally with the splitter told so (32-token cuts for the CUDA-core kernel)
    for planner, told in [("reference", False), ("b200", False)] + ([("b200", True)] if dtype == torch.float32 else []):
        for path in paths_for(c):
            run, out = gpu_utils.run_case(c, planner=planner, path=path, tell_dtype=told)
            assert lib.read_device_status() == 0
            assert (out - truth).abs().max().item() <= tol, (planner, path)
            np.testing.assert_allclose(run.o_lse.cpu().numpy(), truth_lse.numpy(), rtol=1e-4, atol=2e-5)
            # stage-1 partials against the oracle's per-vnode restatement on the very same plan
            tabs = [t.cpu().numpy() for t in run.aux[:6]]
            rows, ranges = engine.split_q_entries(run.aux[3])     # B200 plans that group short nodes carry ranges
            tabs[3] = tabs[3][:rows]
            mid_o, mid_lse = ref_attention.stage1_partials(
                c["q"], c["k"], c["v"], *tabs, scale, q_ranges=None if ranges is None else ranges.cpu().numpy())
            np.testing.assert_allclose(run.mid_lse.cpu().numpy(), mid_lse.numpy(), rtol=1e-4, atol=2e-5)
            assert (run.mid_o.cpu() - mid_o).abs().max().item() <= tol


@pytest.mark.parametrize("before", ["memcpy", "memset", "kernel", "nothing"])
def test_decode_captured_behind_any_kind_of_node(before):
    """Stage 1 is launched with permission to be scheduled before the preceding kernel has drained (programmatic
    dependent launch).  Captured in a CUDA graph right behind a copy node, a memset node, an ordinary kernel that
    produces the query, or nothing at all, the replayed step must still see that node's result."""
    c = adhoc([1, 4, 16], [300, 64, 40], 32, 8, 128, torch.float16, seed=21, q_scale=0.5)
    scale = 1.0 / 128 ** 0.5
    truth, _ = ref_attention.per_leaf_attention(c["nodes"], c["ptrs"], c["q"], c["k"], c["v"], scale)
    run = gpu_utils.EngineRun(c["nodes"], c["ptrs"], c["batch"], c["q"], c["k"], c["v"], 32, 8, 128, c["tsq"])
    run.decode()
    q_src = run.q.clone()
    half = (run.q.float() * 0.5).to(run.q.dtype)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            if before == "memcpy":
                run.q.copy_(q_src)
            elif before == "memset":
                run.o.zero_()
            elif before == "kernel":
                torch.add(half, half, out=run.q)          # the query is produced by the kernel right before stage 1
            engine.decode(run.q, run.k, run.v, run.o, *run.aux, run.tiles[0], run.tiles[1], run.scale)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        run.q.fill_(float("nan") if before in ("memcpy", "kernel") else 0.0)
        if before not in ("memcpy", "kernel"):
            run.q.copy_(q_src)
        run.o.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert lib.read_device_status() == 0
        assert (run.o.float().cpu() - truth).abs().max().item() <= ATOL16


@pytest.mark.parametrize("spec", [t for t in EDGE_TREES if t[0] in ([1, 40], [1, 4, 64], [1, 3, 24])],
                         ids=lambda s: "n%s" % "-".join(map(str, s[0])))
def test_short_nodes_run_as_groups_with_row_ranges(spec):
    """The B200 plan of these trees packs the short leaves into many-row tasks whose rows carry token ranges;
    every kernel family must give the path-concatenated attention on that plan."""
    sizes, lens, hq, hkv, d = spec
    c = adhoc(sizes, lens, hq, hkv, d, torch.float16, seed=11, q_scale=0.5)
    grouped = gpu_utils.EngineRun(c["nodes"], c["ptrs"], c["batch"], c["q"], c["k"], c["v"], hq, hkv, d, c["tsq"])
    rows, ranges = engine.split_q_entries(grouped.aux[3])
    assert ranges is not None and tuple(ranges.shape) == (rows, 2) and rows == grouped.mid_o.shape[0]
    n_big = grouped.aux[11][0]
    assert n_big > 0 and int((ranges[:, 0] > 0).sum()) > 0          # some rows start inside their chunk
    scale = 1.0 / d ** 0.5
    truth, _ = ref_attention.per_leaf_attention(c["nodes"], c["ptrs"], c["q"], c["k"], c["v"], scale)
    for path in paths_for(c):
        out = grouped.decode(path=path)
        assert lib.read_device_status() == 0
        assert (out - truth).abs().max().item() <= atol_for(torch.float16), path
    # the ranges live inside the vnode_to_q_entries table: a cloned / rebuilt tuple decodes to the same bits
    cloned = tuple(t.clone() if isinstance(t, torch.Tensor) else list(t) for t in grouped.aux)
    o2 = torch.full_like(grouped.o, float("nan"))
    fasttree.fasttree_decode(grouped.q, grouped.k, grouped.v, o2, *cloned, grouped.tiles[0], grouped.tiles[1],
                             grouped.scale)
    torch.cuda.synchronize()
    assert torch.equal(o2.float().cpu(), grouped.decode(path="auto"))


def test_argument_cache_keeps_no_query_tensors():
    """A serving loop hands the engine new q / o tensor objects on every layer and step.  The memoised argument
    structs are keyed on the persistent tensors only: 1000 calls with fresh q / o leave one entry and keep none
    of the q storages alive."""
    import gc
    import weakref
    c = cases.build_decode_case("mini3_fp16")
    run = gpu_utils.EngineRun(c["nodes"], c["ptrs"], c["batch"], c["q"], c["k"], c["v"], c["hq"], c["hkv"],
                              c["d"], c["tsq"], planner="b200")
    want = run.decode(path="auto")
    engine._ARG_CACHE.clear()
    refs = []
    for i in range(1000):
        q = run.q.clone()
        o = torch.empty_like(q)
        engine.decode(q, run.k, run.v, o, *run.aux, run.tiles[0], run.tiles[1], run.scale)
        if i % 100 == 0:
            refs.append(weakref.ref(q))
            torch.cuda.synchronize()
            assert torch.equal(o.float().cpu(), want)
    assert len(engine._ARG_CACHE) == 1
    del q, o
    gc.collect()
    assert all(r() is None for r in refs)


@pytest.mark.parametrize("seed", range(10))
def test_random_trees_of_short_nodes(seed):
    """Irregular trees whose nodes are mostly short enough to be grouped (random depth, fan-out, node lengths,
    head configuration and 16-bit type per seed), every kernel family, against path-concatenated attention."""
    rng = np.random.default_rng(1000 + seed)
    levels = int(rng.integers(2, 6))
    hi = int(rng.choice([8, 20, 70, 130, 300]))
    nodes = ref_inputs.random_tree(levels, seed, max_children=int(rng.choice([4, 12, 40])),
                                   lam=float(rng.choice([1.5, 3.0, 6.0])), len_lo=1, len_hi=hi)
    if len(nodes) > 3000:
        pytest.skip("tree too large for a quick test")
    hq, hkv = [(32, 8), (32, 32), (16, 1), (64, 8), (8, 2)][seed % 5]
    dtype = [torch.float16, torch.bfloat16][seed % 2]
    q, k, v, ptrs, batch = ref_inputs.draw_qkv(nodes, hq, hkv, 128, dtype, seed, 0.5)
    run = gpu_utils.EngineRun(nodes, ptrs, batch, q, k, v, hq, hkv, 128, cases.q_tiles_for_group(hq // hkv))
    scale = 1.0 / 128 ** 0.5
    truth, truth_lse = ref_attention.per_leaf_attention(nodes, ptrs, q, k, v, scale)
    tol = atol_for(dtype) + (float(truth.abs().max()) * 2 ** -8 if dtype == torch.bfloat16 else 0.0)
    for path in ("auto", "tcgen05", "persist", "mma", "mma_wide", "stream", "generic"):
        out = run.decode(path=path)
        assert lib.read_device_status() == 0
        assert (out - truth).abs().max().item() <= tol, path
        np.testing.assert_allclose(run.o_lse.cpu().numpy(), truth_lse.numpy(), rtol=1e-4, atol=2e-5)


ALL_PATHS = ("mma", "mma_wide", "generic", "tcgen05", "persist", "stream", "auto")


def wide_case():
    """15 requests x G=4 = 60 query rows on a 200-token root (a many-row task: the tcgen05 kernel's loaders,
    Q gather and row-range code run) plus 15 seven-token leaves (few-row tasks)."""
    return adhoc([1, 15], [200, 7], 32, 8, 128, torch.float16, seed=9, q_scale=0.5)


def indirection_case(kind):
    return cases.build_decode_case({"small": "rand3_fp16", "small3": "mini3_fp16"}[kind]) if kind != "wide" else wide_case()


@pytest.mark.parametrize("kind", ["small", "wide"])
def test_scattered_pool_rows_and_2d_index_table(kind):
    """Serving-style addressing: K/V rows live at arbitrary pool slots and the
    row-id list is a 2-D int32 table (req_to_token) addressed by flat offsets."""
    c = indirection_case(kind)
    run = gpu_utils.EngineRun(c["nodes"], c["ptrs"], c["batch"], c["q"], c["k"], c["v"], c["hq"], c["hkv"],
                              c["d"], c["tsq"], planner="b200")
    base = run.decode(path="mma")
    rows = c["k"].shape[0]
    g = torch.Generator().manual_seed(5)
    pool_rows = rows + 37
    slot_of = torch.randperm(pool_rows, generator=g)[:rows]
    k_pool = torch.randn(pool_rows, c["hkv"], c["d"], generator=g).to(c["dtype"])
    v_pool = torch.randn(pool_rows, c["hkv"], c["d"], generator=g).to(c["dtype"])
    k_pool[slot_of] = c["k"]
    v_pool[slot_of] = c["v"]
    entries = run.aux[0].cpu()
    remapped = torch.where(entries >= 0, slot_of[entries.clamp(min=0)].to(torch.int32), entries)
    width = 64
    pad = (-remapped.numel()) % width
    table = torch.cat([remapped, torch.full((pad,), -1, dtype=torch.int32)]).view(-1, width).cuda()
    aux = (table,) + run.aux[1:]
    o = torch.empty_like(run.q)
    k_dev, v_dev = k_pool.cuda(), v_pool.cuda()
    for path in ALL_PATHS:
        o.fill_(float("nan"))
        engine.decode(run.q, k_dev, v_dev, o, *aux, run.tiles[0], run.tiles[1], run.scale, path=path)
        torch.cuda.synchronize()
        assert lib.read_device_status() == 0, path
        assert (o.float().cpu() - base).abs().max().item() <= (0 if path == "mma" and kind == "small" else ATOL16), path


@pytest.mark.parametrize("kind", ["small3", "wide"])
def test_strided_kv_buffers(kind):
    """K and V interleaved in one buffer: row stride and head stride are not the
    packed ones; last axis stays contiguous (the reference passes strides 0 and 1
    of each buffer, kernel_bench/fasttree.py:456-461).  The tcgen05 kernel and the
    persistent workers then read through TMA descriptors built from those strides."""
    c = indirection_case(kind)
    run = gpu_utils.EngineRun(c["nodes"], c["ptrs"], c["batch"], c["q"], c["k"], c["v"], c["hq"], c["hkv"],
                              c["d"], c["tsq"], planner="b200")
    base = run.decode(path="mma")
    both = torch.stack([c["k"], c["v"]], dim=2).cuda()          # [rows, hkv, 2, d]
    k_view, v_view = both[:, :, 0], both[:, :, 1]
    assert k_view.stride(1) == 2 * c["d"]
    o = torch.empty_like(run.q)
    for path in ALL_PATHS:
        o.fill_(float("nan"))
        engine.decode(run.q, k_view, v_view, o, *run.aux, run.tiles[0], run.tiles[1], run.scale, path=path)
        torch.cuda.synchronize()
        assert lib.read_device_status() == 0, path
        assert (o.float().cpu() - base).abs().max().item() <= (0 if path == "mma" and kind == "small3" else ATOL16), path
    # a strided query / output as well (views of wider tensors)
    q_wide = torch.zeros(c["batch"], c["hq"], 2 * c["d"], dtype=run.q.dtype, device="cuda")
    o_wide = torch.full_like(q_wide, float("nan"))
    q_wide[..., :c["d"]] = run.q
    for path in ("auto", "tcgen05", "generic"):
        engine.decode(q_wide[..., :c["d"]], k_view, v_view, o_wide[..., :c["d"]], *run.aux, run.tiles[0], run.tiles[1],
                      run.scale, path=path)
        torch.cuda.synchronize()
        assert lib.read_device_status() == 0, path
        assert (o_wide[..., :c["d"]].float().cpu() - base).abs().max().item() <= ATOL16, path


@pytest.mark.parametrize("kind", ["small3", "wide"])
def test_bad_plan_data_is_flagged_not_faulted(kind):
    """Out-of-range row ids, request ids and partial-row ids are skipped and reported through the device status
    word by every kernel family; the context stays usable and the next clean call gives the clean answer."""
    c = indirection_case(kind)
    run = gpu_utils.EngineRun(c["nodes"], c["ptrs"], c["batch"], c["q"], c["k"], c["v"], c["hq"], c["hkv"],
                              c["d"], c["tsq"], planner="b200")
    good = run.decode(path="mma")
    assert lib.read_device_status() == 0
    entries = run.aux[0]
    saved = entries[3].item()
    for path in ALL_PATHS:
        for bad in (10 ** 8, -7):
            entries[3] = bad
            run.decode(path=path)
            assert lib.read_device_status() & lib.FT_DEV_BAD_KV_INDEX, (path, bad)
        entries[3] = saved
        assert lib.read_device_status() == 0
        assert torch.equal(run.decode(path="mma"), good)
    q_entries = run.aux[3]
    saved = q_entries[0].item()
    for path in ALL_PATHS:
        q_entries[0] = c["batch"] + 5
        run.decode(path=path)
        assert lib.read_device_status() & lib.FT_DEV_BAD_Q_INDEX, path
        q_entries[0] = saved
        assert torch.equal(run.decode(path="mma"), good)
    # partial buffers three rows too short: the rows that do not fit are neither written nor merged, and flagged
    rows = run.mid_o.shape[0]
    short = run.aux[:9] + (run.mid_o[:rows - 3], run.mid_lse[:rows - 3]) + run.aux[11:]
    o = torch.empty_like(run.q)
    for path in ALL_PATHS:
        engine.decode(run.q, run.k, run.v, o, *short, run.tiles[0], run.tiles[1], run.scale, path=path)
        torch.cuda.synchronize()
        assert lib.read_device_status() & lib.FT_DEV_BAD_ROW_INDEX, path
    assert torch.equal(run.decode(path="mma"), good)


def test_bounded_waits_give_up_and_report():
    """The stage-1 kernels never spin without a limit.  A one-warp self-test kernel of the library waits, with the
    kernels' own wait routines, on an mbarrier nothing arrives at (no copy, MMA or tensor memory in flight): both
    waits must return "gave up", the kernel raises FT_DEV_WAIT_TIMEOUT like a real kernel would, the status word
    reads back and clears, and the context keeps working."""
    import ctypes
    L = lib.load()
    res = (ctypes.c_int * 2)(7, 7)
    stream = torch.cuda.current_stream().cuda_stream
    assert L.ft_selftest_bounded_wait(2000, res, ctypes.c_void_p(stream)) == 0
    assert list(res) == [0, 0]
    assert lib.read_device_status() & lib.FT_DEV_WAIT_TIMEOUT
    assert lib.read_device_status() == 0
    assert L.ft_selftest_bounded_wait(0, res, ctypes.c_void_p(stream)) != 0          # limit out of range
    c = cases.build_decode_case("mini3_fp16")
    _, out = gpu_utils.run_case(c, planner="b200", path="auto")
    assert torch.isfinite(out).all() and lib.read_device_status() == 0


def test_decode_from_and_to_pinned_host_memory():
    """ft_decode_host_io: query in from pinned host memory, output back out, one C-ABI call; same bits as the
    device-resident call."""
    c = wide_case()
    run = gpu_utils.EngineRun(c["nodes"], c["ptrs"], c["batch"], c["q"], c["k"], c["v"], c["hq"], c["hkv"],
                              c["d"], c["tsq"], planner="b200")
    want = run.decode(path="auto")
    q_host = c["q"].clone().pin_memory()
    o_host = torch.full(tuple(run.o.shape), float("nan"), dtype=run.o.dtype).pin_memory()
    for _ in range(2):
        fasttree.fasttree_decode_host_io(q_host, run.k, run.v, o_host, *run.aux, run.tiles[0], run.tiles[1], run.scale)
        assert torch.equal(o_host.float(), want)
        o_host.fill_(float("nan"))
    with pytest.raises(ValueError):            # pageable host memory is refused
        fasttree.fasttree_decode_host_io(c["q"].clone(), run.k, run.v, o_host, *run.aux, run.tiles[0], run.tiles[1],
                                         run.scale)


def test_argument_errors():
    c = cases.build_decode_case("mini3_fp16")
    run = gpu_utils.EngineRun(c["nodes"], c["ptrs"], c["batch"], c["q"], c["k"], c["v"], c["hq"], c["hkv"],
                              c["d"], c["tsq"], planner="b200")
    args = [run.q, run.k, run.v, run.o, *run.aux, run.tiles[0], run.tiles[1], run.scale]
    with pytest.raises(ValueError):                       # CPU tensor: no CPU path
        engine.decode(run.q.cpu(), *args[1:])
    with pytest.raises(ValueError):                       # mismatching dtypes
        engine.decode(run.q.float(), *args[1:])
    with pytest.raises(ValueError):                       # int64 table
        engine.decode(*args[:5], run.aux[1].long(), *args[6:])
    with pytest.raises(lib.FastTreeError) as err:          # fp32 cannot take the tensor-core path
        engine.decode(run.q.float(), run.k.float(), run.v.float(), run.o.float(), *args[4:], path="mma")
    assert err.value.code == -2
    q96 = torch.zeros(c["batch"], c["hq"], 96, dtype=torch.float16, device="cuda")
    kv96 = torch.zeros(run.k.shape[0], c["hkv"], 96, dtype=torch.float16, device="cuda")
    mid96 = torch.zeros(run.mid_o.shape[0], c["hq"], 96, device="cuda")
    with pytest.raises(lib.FastTreeError) as err:          # head_dim outside {16,32,64,128,256}
        engine.decode(q96, kv96, kv96, torch.empty_like(q96), *run.aux[:9], mid96, run.aux[10], *args[15:])
    assert err.value.code == -2


def test_bump_kv_lens():
    lens = torch.tensor([5, 6, 7, 8], dtype=torch.int32, device="cuda")
    last = torch.tensor([3, 1], dtype=torch.int32, device="cuda")
    engine.bump_kv_lens(lens, last)
    torch.cuda.synchronize()
    assert lens.tolist() == [5, 7, 7, 9]


@pytest.mark.parametrize("name", ["mini3_fp16", "rand3_fp16"])
def test_decode_captured_in_a_cuda_graph(name):
    """The decode call (fused stage 1 + dependent stage 2, no allocation, no host sync) is captured into a CUDA
    graph; replays with new query values in the same buffers must match eager calls bit for bit."""
    c = cases.build_decode_case(name)
    run, first = gpu_utils.run_case(c, planner="b200", path="auto")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        fasttree.fasttree_decode(run.q, run.k, run.v, run.o, *run.aux, run.tiles[0], run.tiles[1], run.scale)
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            fasttree.fasttree_decode(run.q, run.k, run.v, run.o, *run.aux, run.tiles[0], run.tiles[1], run.scale)
    torch.cuda.current_stream().wait_stream(side)
    for seed in (1, 2):
        g = torch.Generator().manual_seed(seed)
        run.q.copy_(torch.randn(run.q.shape, generator=g).to(run.q.dtype))
        run.o.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        replayed = run.o.float().cpu()
        eager = run.decode_via_dropin()
        assert torch.isfinite(replayed).all()
        assert torch.equal(replayed, eager)
    assert lib.read_device_status() == 0


# ------------------------------------------------------------ benchmark sizes
FULL = {
    "cfg3": dict(sizes=[1, 16, 256], lens=[2048, 512, 64], hq=32, hkv=8, dtype=torch.bfloat16, q_scale=0.5),
    "cfg4": dict(sizes=[1, 1024], lens=[16384, 32], hq=64, hkv=8, dtype=torch.bfloat16, q_scale=1.0),
}


def gpu_inputs(nodes, hq, hkv, d, dtype, seed, q_scale):
    """Seeded inputs drawn on the GPU (sizes here are too large for the CPU draw
    order to matter; the oracle reads them back for its sample)."""
    batch = ref_inputs.assign_requests(nodes)
    ptrs = ref_inputs.kv_prefix_sums(nodes)
    g = torch.Generator(device="cuda").manual_seed(seed)
    k = torch.randn(ptrs[-1], hkv, d, generator=g, device="cuda", dtype=torch.float32).to(dtype)
    v = torch.randn(ptrs[-1], hkv, d, generator=g, device="cuda", dtype=torch.float32).to(dtype)
    q = (torch.randn(batch, hq, d, generator=g, device="cuda", dtype=torch.float32) * q_scale).to(dtype)
    return q, k, v, ptrs, batch


@pytest.mark.parametrize("name", sorted(FULL))
def test_benchmark_sizes_properties(name):
    """At full benchmark size: (1) 64 evenly spaced requests against the fp32 oracle (every group of short
    leaves is hit: cfg3 packs its 64-token leaves 32 to a task, cfg4 its 32-token leaves 16 to a task),
    (2) both planners agree, (3) linearity in V: decode(V1 + V2) = decode(V1) + decode(V2)
    because the softmax weights depend on Q and K only, (4) deterministic repeat."""
    f = FULL[name]
    d = 128
    nodes = ref_inputs.layered_tree(f["sizes"], f["lens"])
    q, k, v, ptrs, batch = gpu_inputs(nodes, f["hq"], f["hkv"], d, f["dtype"], 17, f["q_scale"])
    tsq = cases.q_tiles_for_group(f["hq"] // f["hkv"])
    runs = {pl: gpu_utils.EngineRun(nodes, ptrs, batch, q, k, v, f["hq"], f["hkv"], d, tsq, planner=pl)
            for pl in ("b200", "reference")}
    outs = {pl: r.decode() for pl, r in runs.items()}
    assert lib.read_device_status() == 0
    sample = sorted(set(int(round(i * (batch - 1) / 63)) for i in range(64)))     # 64 evenly spaced requests
    truth, truth_lse = ref_attention.per_leaf_attention(nodes, ptrs, q.cpu(), k.cpu(), v.cpu(), 1.0 / d ** 0.5,
                                                        requests=sample)
    tol = ATOL16 + float(truth.abs().max()) * 2 ** -8
    for pl in outs:
        assert (outs[pl][sample] - truth).abs().max().item() <= tol, pl
        np.testing.assert_allclose(runs[pl].o_lse.cpu().numpy()[sample], truth_lse.numpy(), rtol=1e-4, atol=2e-5)
    assert (outs["b200"] - outs["reference"]).abs().max().item() <= 2 * tol
    r = runs["b200"]
    assert torch.equal(r.decode(), outs["b200"])
    v2 = torch.randn_like(v)
    r.v = v2
    o2 = r.decode()
    r.v = (v.float() + v2.float()).to(f["dtype"])
    o12 = r.decode()
    lin_tol = 3 * tol + float(o12.abs().max()) * 2 ** -7       # V1+V2 is itself rounded to bf16
    assert (o12 - (outs["b200"] + o2)).abs().max().item() <= lin_tol


# ------------------------------------------------------------ the reference's own kernels on this GPU
def reference_or_skip():
    from oracle import ref_triton
    ok, why = ref_triton.availability()
    if not ok:
        pytest.skip(why)
    return ref_triton


REF_CASES = {
    # name: level sizes, level lengths, hq, hkv, dtype, q scale   (benchmark configurations and their 8-way head shards)
    "cfg2": ([1, 64], [4096, 256], 32, 8, torch.float16, 1.0),
    "cfg3": ([1, 16, 256], [2048, 512, 64], 32, 8, torch.bfloat16, 0.5),
    "cfg4": ([1, 1024], [16384, 32], 64, 8, torch.bfloat16, 1.0),
    "cfg3_tp8": ([1, 16, 256], [2048, 512, 64], 4, 1, torch.bfloat16, 0.5),
    "cfg4_tp8": ([1, 1024], [16384, 32], 8, 1, torch.bfloat16, 1.0),
    "cfg2_tp4": ([1, 64], [4096, 256], 8, 2, torch.float16, 1.0),
}


@pytest.mark.parametrize("name", sorted(REF_CASES))
def test_engine_matches_reference_triton_kernels(name):
    """Every request of the benchmark configurations (and of their head-sharded plans: one or two local KV
    heads give smaller chunks and more vnodes) against the output of the reference's unmodified planner + Triton
    kernels on the same GPU tensors, in the configuration's own 16-bit type.  Both sides round P and O to the
    storage type; the bound is the stated 2e-3 plus one output ulp for bf16 on each side."""
    ref_triton = reference_or_skip()
    sizes, lens, hq, hkv, dtype, q_scale = REF_CASES[name]
    d = 128
    nodes = ref_inputs.layered_tree(sizes, lens)
    q, k, v, ptrs, batch = gpu_inputs(nodes, hq, hkv, d, dtype, 23, q_scale)
    ref = ref_triton.ReferenceRun(nodes, ptrs, batch, hq, hkv, d)
    o_ref = torch.full_like(q, float("nan"))
    ref.decode(q, k, v, o_ref)
    torch.cuda.synchronize()
    o_ref = o_ref.float().cpu()
    assert torch.isfinite(o_ref).all()
    tol = ATOL16 + (2 * float(o_ref.abs().max()) * 2 ** -8 if dtype == torch.bfloat16 else 0.0)
    for planner in ("b200", "reference"):
        run = gpu_utils.EngineRun(nodes, ptrs, batch, q, k, v, hq, hkv, d, cases.q_tiles_for_group(hq // hkv),
                                  planner=planner)
        out = run.decode()
        assert lib.read_device_status() == 0
        assert (out - o_ref).abs().max().item() <= tol, planner
        if planner == "reference":
            # same plan on both sides: the partial LSEs written by the reference kernels are comparable row by row
            for mine, theirs in zip(run.aux[:9], ref.aux[:9]):
                assert torch.equal(mine, theirs)
            np.testing.assert_allclose(run.mid_lse.cpu().numpy(), ref.aux[10].cpu().numpy(), rtol=1e-4, atol=2e-5)


@pytest.mark.parametrize("levels,seed,sample", [(4, 0, None), (4, 1, None), (4, 2, None), (6, 0, 48)])
def test_random_tree_configuration_at_benchmark_size(levels, seed, sample):
    """Benchmark configuration 5 (irregular tree, per-node context ~ Uniform[16, 2048], branching 1 + Poisson(3)
    capped at 32, 32/8 heads, fp16) at its full size: the 4-level trees against the fp32 oracle on EVERY request,
    the 6-level tree (several hundred requests, ~0.8 M tokens) on 48 evenly spaced requests; and, where the
    reference is staged, every request against the reference kernels' output."""
    hq, hkv, d, dtype = 32, 8, 128, torch.float16
    nodes = ref_inputs.random_tree(levels, seed)
    q, k, v, ptrs, batch = gpu_inputs(nodes, hq, hkv, d, dtype, 100 + seed, 1.0)
    run = gpu_utils.EngineRun(nodes, ptrs, batch, q, k, v, hq, hkv, d, cases.q_tiles_for_group(hq // hkv))
    out = run.decode()
    assert lib.read_device_status() == 0
    reqs = list(range(batch)) if sample is None else sorted(set(int(round(i * (batch - 1) / (sample - 1)))
                                                                 for i in range(sample)))
    truth, truth_lse = ref_attention.per_leaf_attention(nodes, ptrs, q.cpu(), k.cpu(), v.cpu(), 1.0 / d ** 0.5,
                                                        requests=reqs)
    assert (out[reqs] - truth).abs().max().item() <= ATOL16
    np.testing.assert_allclose(run.o_lse.cpu().numpy()[reqs], truth_lse.numpy(), rtol=1e-4, atol=2e-5)
    from oracle import ref_triton
    if ref_triton.availability()[0]:
        ref = ref_triton.ReferenceRun(nodes, ptrs, batch, hq, hkv, d)
        o_ref = torch.empty_like(q)
        ref.decode(q, k, v, o_ref)
        torch.cuda.synchronize()
        assert (out - o_ref.float().cpu()).abs().max().item() <= ATOL16
