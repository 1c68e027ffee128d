"""Host planner of the plugin (reference:
fasttree_sglang_plugin_v0_2_13/schedule.py:12-283).

``prepare_for_fasttree_meta`` turns the running batch and SGLang's radix cache
into vnode tables addressed THROUGH ``req_to_token``: a tree vnode's KV run is
``stride * req_pool_idx[first request] + token offset`` into the flattened
table, which the kernels dereference to KV-pool slots.  Every request also gets
private "tail" vnodes over the positions the radix cache does not hold
(generated tokens and the token being decoded).  ``prepare_for_fasttree_step``
lengthens each request's last tail vnode by one between the steps of a burst.

Two planners, selected by ``FastTreeMetadata.planner``:

* ``"reference"`` reproduces the reference's tables bit for bit, including its
  quirks (the edge heuristic never fires because the child loop iterates over
  ``enumerate`` tuples, schedule.py:96-98; the 128-token KV-split fallback is a
  no-op, :130; a tile-size collapse copies the REQUEST tile into the KV tile
  sizes, :138-141; CTA counting uses the KV tile, not the split, :115; head
  counts are the unsharded ones).
* ``"b200"`` plans with the 148-SM splitter of ``ft_b200.planner`` (working edge
  decisions, chunk sizes from a byte budget, 128-row tiles for the tcgen05
  kernel) and starts each tail where the radix walk actually stopped, so prompt
  tokens that are not in the cache are still attended to.
"""
from collections import defaultdict, deque

import numpy as np
import torch

from ft_b200 import engine as _engine
from ft_b200 import planner as _planner


def _walk_requests(batch):
    """Per request, follow the radix tree along prompt + generated tokens
    (schedule.py:18-35).  Returns (node -> request ids, tokens covered per request)."""
    root = batch.tree_cache.root_node
    node_to_reqs = defaultdict(list)
    covered = []
    for rid, req in enumerate(batch.reqs):
        tokens = list(req.origin_input_ids) + list(req.output_ids)
        node, pos = root, 0
        while pos < len(tokens):
            child = node.children.get(tokens[pos])
            if not child:
                break
            node_to_reqs[child].append(rid)
            node = child
            pos += len(child.key)
        covered.append(pos)
    return node_to_reqs, covered


def _bfs(batch, node_to_reqs):
    """Populated radix nodes in breadth-first order with their token offsets (schedule.py:74-85)."""
    order, offsets, parents = [], [], []
    todo = deque([(batch.tree_cache.root_node, 0, -1)])
    while todo:
        node, off, par = todo.popleft()
        me = len(order)
        order.append(node)
        offsets.append(off)
        parents.append(par)
        nxt = off + len(node.value)
        for child in node.children.values():
            if child in node_to_reqs:
                todo.append((child, nxt, me))
    return order, offsets, parents


def _upload(md, tabs, last_vnodes, tail_state=None, src_table=None):
    nv, rows, bsz = tabs["vnode_to_kv_offs"].size, tabs["vnode_to_q_entries"].size, tabs["req_to_vnode_offs"].size
    if nv > md.max_vnodes or rows > md.max_vnode_to_q_entries or bsz > md.max_batch_size:
        raise ValueError(f"plan ({nv} vnodes, {rows} partial rows, batch {bsz}) exceeds the capacity of "
                         f"FastTreeMetadata ({md.max_vnodes}, {md.max_vnode_to_q_entries}, {md.max_batch_size})")
    segs = tabs.get("aux_segments")
    n_seg = 0 if segs is None else int(segs.shape[0])
    if getattr(md, "group_tails", False):
        if n_seg > md.aux_segments.shape[1] or int(tabs.get("aux_entries", 0)) > md.kv_entries_aux.numel():
            raise ValueError(f"plan ({n_seg} grouped runs, {tabs.get('aux_entries', 0)} auxiliary row ids) exceeds the "
                             f"capacity of FastTreeMetadata ({md.aux_segments.shape[1]}, {md.kv_entries_aux.numel()})")

    def put(dst, arr):
        t = torch.from_numpy(np.ascontiguousarray(arr, dtype=np.int32))
        dst[:t.numel()].copy_(t, non_blocking=True)

    put(md.vnode_to_q_entries, tabs["vnode_to_q_entries"])
    put(md.vnode_to_q_offs, tabs["vnode_to_q_offs"])
    put(md.vnode_to_q_lens, tabs["vnode_to_q_lens"])
    put(md.vnode_to_kv_offs, tabs["vnode_to_kv_offs"])
    put(md.vnode_to_kv_lens, tabs["vnode_to_kv_lens"])
    put(md.req_to_vnode_entries, tabs["req_to_vnode_entries"])
    put(md.req_to_vnode_offs, tabs["req_to_vnode_offs"])
    put(md.req_to_vnode_lens, tabs["req_to_vnode_lens"])
    put(md.req_last_vnodes_dev, np.asarray(last_vnodes, dtype=np.int32))
    put(md.phase_info_dev, np.asarray(list(tabs["phase_node_nums"]) + list(tabs["phase_node_offsets"]), dtype=np.int32))
    state = np.full((bsz, 4), -1, dtype=np.int32)
    if tail_state is None:                      # every tail is a vnode of its own
        state[:, 2] = np.asarray(last_vnodes, dtype=np.int32)
    else:
        state[:] = tail_state
    md.tail_state[:bsz].copy_(torch.from_numpy(state), non_blocking=True)
    stale = getattr(md, "tail_rows", 0)
    if stale > bsz:                             # entries of a larger earlier batch must read "unused"
        md.tail_state[bsz:stale].fill_(-1)
    md.tail_rows = bsz
    md.num_grouped_tails = int((state[:, 0] >= 0).sum())
    md.steps_since_plan = 0
    if getattr(md, "group_tails", False):
        # the decode call always passes the range table: rows of plain vnodes see their whole chunk
        ranges = tabs.get("vnode_q_kv_ranges")
        if ranges is None:
            ranges = np.zeros((rows, 2), dtype=np.int32)
            ranges[:, 1] = np.iinfo(np.int32).max
        md.vnode_q_kv_ranges[:rows].copy_(torch.from_numpy(np.ascontiguousarray(ranges, dtype=np.int32)), non_blocking=True)
        if n_seg:
            md.aux_segments[:, :n_seg].copy_(torch.from_numpy(np.ascontiguousarray(segs.T, dtype=np.int32)), non_blocking=True)
            if md.kv_entries_aux.is_cuda:
                _engine.gather_kv_entries(src_table, md.aux_segments[0], md.aux_segments[1], md.aux_segments[2],
                                          md.aux_segments[3], n_seg, md.kv_entries_aux)
            else:       # plan tables kept on the host (planner tests, tools): the same table, built with torch
                flat = src_table.reshape(-1)
                for src, length, dst, room in segs.tolist():
                    md.kv_entries_aux[dst:dst + length] = flat[src:src + length]
                    md.kv_entries_aux[dst + length:dst + length + room] = flat[src]
        md.refresh_pending = md.num_grouped_tails > 0 or (md.graph_safe and md.refresh_layer is None)
    md.phase_node_nums = list(tabs["phase_node_nums"])
    md.phase_node_offsets = list(tabs["phase_node_offsets"])
    md.req_last_vnodes = [int(v) for v in last_vnodes]
    md.num_vnodes, md.num_partial_rows = int(nv), int(rows)


# --------------------------------------------------------------- reference-compatible
def _plan_reference(batch, md, node_to_reqs, order, offsets, req_idx, stride):
    tsq, tsk = list(md.TSQs), list(md.TSKs)
    split = [md.kv_split_sizes[0], md.kv_split_sizes[0]]
    heads = md.num_kv_heads
    counts = [len(node_to_reqs[n]) if n in node_to_reqs else 0 for n in order]
    lens = [len(n.value) for n in order]

    def cta_counts():                                   # schedule.py:87-118 with the heuristic inert
        par = [0, 0]
        for cnt, ln in zip(counts, lens):
            if cnt > 0:
                ph = 0 if cnt > tsq[1] else 1
                par[ph] += -(-cnt // tsq[ph]) * -(-ln // tsk[ph])
        return [c * heads for c in par]

    for rnd in range(3):                                # schedule.py:120-143
        par = cta_counts()
        if rnd == 0:
            if not any(0 < par[ph] < md.para_threshs1[ph] for ph in range(2)):
                break                                    # (the split-size assignment of the reference is a no-op)
        elif rnd == 1:
            if 0 < par[0] < md.para_threshs2[0]:
                tsq = [tsq[1], tsq[1]]
                tsk = [tsq[1], tsq[1]]
            elif 0 < par[1] < md.para_threshs2[1]:
                tsq = [tsq[0], tsq[0]]
                tsk = [tsq[0], tsq[0]]
            else:
                break
    md.phase_q_tile_sizes, md.phase_kv_tile_sizes = tsq, tsk

    vnodes = []
    for node, cnt, ln, off in zip(order, counts, lens, offsets):            # schedule.py:159-210
        if cnt == 0:
            continue
        kids = [c for c in node.children.values() if c in node_to_reqs]
        group = kids if kids else [node]
        reqs = [r for n in group for r in node_to_reqs[n]]
        first = node_to_reqs[group[0]][0]
        start = stride * int(req_idx[first]) + off
        ph = 0 if cnt > tsq[1] else 1
        # the reference sizes the request tiles from `cnt` but lists `reqs`; they agree whenever
        # every request of a node continues into one of its children (true for its workloads)
        if len(reqs) != cnt:
            raise ValueError("a request ends exactly at an inner radix node; the reference planner's tables are "
                             "inconsistent for such batches (use planner='b200')")
        vnodes.append(_planner.VirtualNode([(start, start + ln)], np.asarray(reqs, dtype=np.int32),
                                           q_tile=tsq[ph], kv_split=split[ph]))
    tails = []
    for rid, req in enumerate(batch.reqs):                                  # schedule.py:212-232
        start = stride * int(req_idx[rid]) + len(req.origin_input_ids)
        tails.append(_planner.VirtualNode([(start, start + len(req.output_ids) + 1)],
                                          np.asarray([rid], dtype=np.int32), q_tile=tsq[1], kv_split=split[1]))
    perm = []
    tabs = _planner.emit_tables(vnodes + tails, len(batch.reqs), small_tile=tsq[1], direct_offsets=True,
                                order_out=perm)
    # tail tasks are the last ones before and after the stable phase split: each request's last chunk
    n_tasks = tabs["vnode_to_kv_offs"].size
    last, acc = [], n_tasks - sum(-(-(len(r.output_ids) + 1) // split[1]) for r in batch.reqs)
    for req in batch.reqs:
        acc += -(-(len(req.output_ids) + 1) // split[1])
        last.append(acc - 1)
    tabs["req_to_vnode_entries"] = tabs["req_to_vnode_entries"][:-_planner.PAD_ENTRIES]   # the plugin uploads no padding
    return tabs, last


# ------------------------------------------------------------------------ B200 splitter
class _RadixView:
    """Radix node as the tree record the splitter expects."""
    __slots__ = ("parent", "id", "seqlen", "num_children", "requests")

    def __init__(self, parent, nid, seqlen, requests):
        self.parent, self.id, self.seqlen, self.num_children, self.requests = parent, nid, seqlen, 0, requests


def _plan_b200(batch, md, node_to_reqs, covered, order, offsets, parents, req_idx, stride):
    model = _planner.b200_model_for(md, md.head_dim)
    all_reqs = list(range(len(batch.reqs)))
    tree = []
    for i, (node, par) in enumerate(zip(order, parents)):
        reqs = all_reqs if i == 0 else sorted(node_to_reqs[node])
        tree.append(_RadixView(par, i, len(node.value), reqs))
        if par >= 0:
            tree[par].num_children += 1

    def ranges_of(assign, i):
        # a node and the ancestors it carries are one contiguous run in the row of any request below it
        start, up = offsets[i], i
        while assign[up] == 1:
            up = tree[up].parent
            start = offsets[up]
        first = tree[i].requests[0]
        base = stride * int(req_idx[first])
        return [(base + start, base + offsets[i] + tree[i].seqlen)]

    # Radix nodes that only one request passes through (the unique end of its prompt) are contiguous with that
    # request's tail in its row of req_to_token: they leave the tree and the tail starts where they began, which
    # makes one few-row task per request out of two or more.
    tail_start = list(covered)
    if getattr(md, "merge_private_nodes", True):
        for i in range(len(tree) - 1, 0, -1):      # children come after their parents in breadth-first order
            if len(tree[i].requests) == 1 and tree[i].num_children <= 1:
                rid = tree[i].requests[0]
                tail_start[rid] = min(tail_start[rid], offsets[i])
                tree[i].requests = []
                tree[tree[i].parent].num_children -= 1
    extra = []
    for rid, req in enumerate(batch.reqs):
        end = len(req.origin_input_ids) + len(req.output_ids) + 1
        base = stride * int(req_idx[rid])
        extra.append(([(base + tail_start[rid], base + end)], [rid]))
    def run(tail_room, model):
        if getattr(md, "native_planner", True):
            # the native splitter of the shared library; the Python branch below is its specification
            node_base = [stride * int(req_idx[nd.requests[0]]) if nd.requests else 0 for nd in tree]
            return _planner.b200_tables_native_direct(
                tree, node_base, offsets, [(r[0][0], r[0][1], q[0]) for r, q in extra], len(batch.reqs),
                md.num_qo_heads, md.num_kv_heads, md.head_dim, model, tail_room=tail_room)
        vnodes, _assign, q_tile, small_tile, _target = _planner.b200_virtual_nodes(
            tree, md.num_qo_heads, md.num_kv_heads, md.head_dim, model, ranges_of, extra=extra, tail_room=tail_room)
        tabs = _planner.emit_tables(vnodes, len(batch.reqs), small_tile=small_tile, direct_offsets=True,
                                    order_key=_planner.b200_task_order)
        return tabs, q_tile, small_tile, model.tile_tokens

    tabs, q_tile, small_tile, tile_tokens = run(-1, model)
    if getattr(md, "group_tails", False):
        # Groups pay when the few-row tasks alone would queue up several deep behind the resident CTAs; then the
        # burst is planned again with short runs packed into many-row vnodes.  A group needs more than 16 query
        # rows anyway (only the many-row kernels honour row ranges); past that, a handful of one-tile tails
        # already costs less as one task than as one task each.
        few_row_ctas = tabs["phase_node_nums"][1] * md.num_kv_heads
        if few_row_ctas >= md.group_tails_min_load * model.num_sms * model.ctas_per_sm:
            from dataclasses import replace
            tabs, q_tile, small_tile, tile_tokens = run(
                md.tail_room, replace(model, group_min_members=min(model.group_min_members, 4)))
    md.phase_q_tile_sizes = [q_tile, small_tile]
    md.phase_kv_tile_sizes = [tile_tokens, tile_tokens]
    # the task holding the END of each request's tail (the one that grows during the burst)
    ends = {}
    for rid, req in enumerate(batch.reqs):
        ends[stride * int(req_idx[rid]) + len(req.origin_input_ids) + len(req.output_ids) + 1] = rid
    last = [-1] * len(batch.reqs)
    kv_offs = tabs["vnode_to_kv_offs"].astype(np.int64)
    kv_end = kv_offs + tabs["vnode_to_kv_lens"]
    for task in np.flatnonzero((tabs["vnode_to_q_lens"] == 1) & (kv_offs < _planner.AUX_BIT)):
        rid = ends.get(int(kv_end[task]))
        if rid is not None and int(tabs["vnode_to_q_entries"][tabs["vnode_to_q_offs"][task]]) == rid:
            last[rid] = int(task)
    # tails that became members of a group: the run that ends where the request ends and has room behind it
    state = np.full((len(batch.reqs), 4), -1, dtype=np.int32)
    segs = tabs.get("aux_segments")
    if segs is not None and len(segs):
        groups = np.flatnonzero(kv_offs >= _planner.AUX_BIT)
        g_base = kv_offs[groups] - _planner.AUX_BIT
        by_base = np.argsort(g_base)
        for src, length, dst, room in segs.tolist():
            rid = ends.get(src + length)
            if rid is None or room <= 0:
                continue
            task = int(groups[by_base[np.searchsorted(g_base[by_base], dst, side="right") - 1]])
            q0, qn = int(tabs["vnode_to_q_offs"][task]), int(tabs["vnode_to_q_lens"][task])
            hit = np.flatnonzero(tabs["vnode_to_q_entries"][q0:q0 + qn] == rid)
            if hit.size != 1:
                raise RuntimeError("internal error: a grouped tail has no partial row of its own")
            state[rid] = (dst + length, src + length, q0 + int(hit[0]), room)
            last[rid] = task
    if min(last, default=0) < 0:
        raise RuntimeError("internal error: a request has no tail task")
    for rid in range(len(batch.reqs)):
        if state[rid, 0] < 0:
            state[rid, 2] = last[rid]
    tabs["req_to_vnode_entries"] = tabs["req_to_vnode_entries"][:-_planner.PAD_ENTRIES]
    tabs["tail_state"] = state
    return tabs, last


def prepare_for_fasttree_meta(batch, fasttree_metadata):
    """Plan one decode burst and upload the tables into ``fasttree_metadata``
    (reference: schedule.py:12-275).  Binds the metadata to the batch."""
    md = fasttree_metadata
    node_to_reqs, covered = _walk_requests(batch)
    order, offsets, parents = _bfs(batch, node_to_reqs)
    req_idx = batch.req_pool_indices.cpu()
    stride = batch.req_to_token_pool.req_to_token.stride(0)
    if md.planner == "reference":
        tabs, last = _plan_reference(batch, md, node_to_reqs, order, offsets, req_idx, stride)
    else:
        tabs, last = _plan_b200(batch, md, node_to_reqs, covered, order, offsets, parents, req_idx, stride)
    _upload(md, tabs, last, tail_state=tabs.get("tail_state"),
            src_table=batch.req_to_token_pool.req_to_token if getattr(md, "group_tails", False) else None)
    batch.fasttree_metadata = md


def prepare_for_fasttree_step(batch, fasttree_metadata):
    """Between two steps of a burst: the token just decoded joins each request's
    last private chunk (reference: schedule.py:278-283).  One tiny kernel, no
    host-to-device copy."""
    md = fasttree_metadata
    md.steps_since_plan += 1
    if md.num_grouped_tails and md.steps_since_plan > md.tail_room:
        raise RuntimeError(f"a burst of more than {md.tail_room} steps after one plan: raise FastTreeMetadata.tail_room")
    if md.tail_state.is_cuda:
        _engine.bump_tails(md.tail_state, len(batch.reqs), md.vnode_q_kv_ranges, md.vnode_to_kv_lens)
    else:               # plan tables kept on the host (planner tests, tools)
        for rid in range(len(batch.reqs)):
            aux_pos, _src, index, room = md.tail_state[rid].tolist()
            if aux_pos < 0:
                md.vnode_to_kv_lens[index] += 1
            else:
                md.vnode_q_kv_ranges[index, 1] += 1
                md.tail_state[rid] += torch.tensor([1, 1, 0, -1], dtype=torch.int32)
    md.refresh_pending = md.num_grouped_tails > 0
