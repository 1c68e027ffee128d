"""Host planner: radix tree -> vnode tables for the decode kernels.

Two splitters share one table emitter:

* ``plan_reference``  reproduces the reference planner bit for bit
  (kernel_bench/fasttree.py:64-262: greedy split-K/split-Q edge heuristic on a
  padding cost model, CTA-count driven KV-split / tile adaptation tuned for a
  132-SM part).  Kept so that plans, partial buffers and outputs can be compared
  one-to-one with the reference.
* ``plan_b200``       the splitter sized for a 148-SM B200: tasks are
  (node KV chunk x request group); chunk lengths are balanced so the grid fills
  the machine a few times over, with as few partial rows as possible, and nodes
  with enough query rows are routed to the 128-row tensor-core tile.

Both are pure functions of (tree, parameters): no randomness, no dependence on
dict/set iteration order, ties broken by node id.

The emitted table family is the reference's (fasttree.py:282-296):
``vnode_to_kv_entries/offs/lens``, ``vnode_to_q_entries/offs/lens``,
``req_to_vnode_entries/offs/lens`` (entries are partial-ROW ids),
``phase_node_nums/offsets``.
"""
import heapq
import math
from collections import deque
from dataclasses import dataclass, field, replace

import numpy as np

PAD_ENTRIES = 32  # the reference appends 32 x -1 to both index lists (fasttree.py:261-262)
AUX_BIT = 1 << 30     # FT_KV_OFFSET_AUX: a vnode_to_kv_offs value with this bit indexes the auxiliary row-id table
GROUP_MAX_TILES_DIRECT = 24  # ... and a group of the serving path never more than this
GROUP_MAX_TILES = 16  # a group of short nodes never spans more KV tiles than this (same constant in csrc/ft_planner.cu)


@dataclass
class VirtualNode:
    """One context-queries pairing before it is cut into tasks."""
    kv_ranges: list        # [(row_begin, row_end), ...] root-most segment first
    requests: np.ndarray   # request ids, in partial-row order
    q_tile: int            # requests per task
    kv_split: int          # tokens per task
    row_ranges: list = None  # group of short nodes: per request the (begin, end) tokens of the chunk it attends to
    room: int = 0            # serving path: spare row ids kept behind this pairing when it joins a group (a tail grows)
    member_room: list = None  # group in the serving path: the room behind each of its ranges


@dataclass
class Plan:
    vnode_to_kv_entries: np.ndarray
    vnode_to_kv_offs: np.ndarray
    vnode_to_kv_lens: np.ndarray
    vnode_to_q_entries: np.ndarray
    vnode_to_q_offs: np.ndarray
    vnode_to_q_lens: np.ndarray
    req_to_vnode_entries: np.ndarray
    req_to_vnode_offs: np.ndarray
    req_to_vnode_lens: np.ndarray
    phase_node_nums: list
    phase_node_offsets: list
    node_assignments: list
    vnode_q_kv_ranges: np.ndarray = None   # optional [partial rows, 2]: tokens of its chunk a partial row attends to
    aux_segments: np.ndarray = None        # serving plans with groups: [n, 4] {source, length, position, room} of the auxiliary row-id table
    aux_entries: int = 0
    phase_q_tile_sizes: list = field(default_factory=list)
    phase_kv_tile_sizes: list = field(default_factory=list)
    kv_split_sizes: list = field(default_factory=list)
    info: dict = field(default_factory=dict)

    @property
    def num_partial_rows(self):
        return int(self.vnode_to_q_entries.size)

    @property
    def num_vnodes(self):
        return int(self.vnode_to_kv_offs.size)

    def tables(self):
        return (self.vnode_to_kv_entries, self.vnode_to_kv_offs, self.vnode_to_kv_lens,
                self.vnode_to_q_entries, self.vnode_to_q_offs, self.vnode_to_q_lens,
                self.req_to_vnode_entries, self.req_to_vnode_offs, self.req_to_vnode_lens)


# --------------------------------------------------------------------- emitter
def emit_tables(vnodes, batch_size, small_tile, order_key=None, order_out=None, direct_offsets=False):
    """Cut every virtual node into (KV chunk x request tile) tasks and build the
    reference-format tables.  Tasks whose request count exceeds ``small_tile``
    form phase 0, the others phase 1 (stable partition, fasttree.py:246-259).
    ``order_key(kv_len, q_len)`` optionally sorts the tasks inside each phase
    (stable, descending) so that long tasks are scheduled first.
    ``direct_offsets``: every virtual node has ONE row range and the ranges already
    are offsets into an existing row-id table (the serving path's flattened
    ``req_to_token``); no ``vnode_to_kv_entries`` array is built and
    ``vnode_to_kv_offs`` are those offsets."""
    kv_chunks, kv_offs, kv_lens, q_chunks, q_offs, q_lens = [], [], [], [], [], []
    range_chunks, any_ranges = [], False
    kv_total = q_total = aux_total = 0
    aux_segments = []
    for vn in vnodes:
        reqs = np.asarray(vn.requests, dtype=np.int32)
        nreq = int(reqs.size)
        if nreq == 0:
            continue
        if direct_offsets and vn.member_room is not None:
            # a group of the serving path: its row ids are gathered into an auxiliary table
            kv_base, length = AUX_BIT + aux_total, 0
            for (rb, re_), room in zip(vn.kv_ranges, vn.member_room):
                if rb >= AUX_BIT or aux_total + length + (re_ - rb) + room >= AUX_BIT:
                    raise ValueError("plan does not fit the auxiliary table's 30-bit offsets")
                aux_segments.append((int(rb), int(re_ - rb), aux_total + length, int(room)))
                length += int(re_ - rb) + int(room)
            aux_total += length
        elif direct_offsets:
            (rb, re_), = vn.kv_ranges
            length = int(re_ - rb)
            if length <= 0:
                continue
            kv_base = int(rb)
        else:
            segs = [np.arange(b, e, dtype=np.int32) for (b, e) in vn.kv_ranges]
            length = int(sum(s.size for s in segs))
            if length == 0:
                continue
            kv_chunks.extend(segs)
            kv_base = kv_total
        n_kv = -(-length // vn.kv_split)
        n_q = -(-nreq // vn.q_tile)
        c_off = np.arange(n_kv, dtype=np.int64) * vn.kv_split
        c_len = np.minimum(c_off + vn.kv_split, length) - c_off
        t_off = np.arange(n_q, dtype=np.int64) * vn.q_tile
        t_len = np.minimum(t_off + vn.q_tile, nreq) - t_off
        # chunk-major, request-tile-minor; every chunk repeats the full request list
        kv_offs.append(np.repeat(kv_base + c_off, n_q))
        kv_lens.append(np.repeat(c_len, n_q))
        q_base = q_total + np.arange(n_kv, dtype=np.int64) * nreq
        q_offs.append((q_base[:, None] + t_off[None, :]).reshape(-1))
        q_lens.append(np.tile(t_len, n_kv))
        q_chunks.append(np.tile(reqs, n_kv))
        if vn.row_ranges is not None:
            if n_kv != 1 or n_q != 1:
                raise ValueError("a group of short nodes must be one task")
            range_chunks.append(np.asarray(vn.row_ranges, dtype=np.int32).reshape(nreq, 2))
            any_ranges = True
        else:                                  # every row of chunk c sees the whole chunk
            full = np.zeros((n_kv, nreq, 2), dtype=np.int32)
            # (serving path: a chunk may grow during the burst, so the end is left open; the kernels clip it)
            full[:, :, 1] = np.iinfo(np.int32).max if direct_offsets else c_len[:, None]
            range_chunks.append(full.reshape(-1, 2))
        kv_total += length
        q_total += n_kv * nreq

    def cat(parts, dtype=np.int64):
        return np.concatenate(parts).astype(dtype) if parts else np.zeros(0, dtype=dtype)

    kv_offs, kv_lens, q_offs, q_lens = cat(kv_offs), cat(kv_lens), cat(q_offs), cat(q_lens)
    q_entries = cat(q_chunks, np.int32)
    if kv_total + PAD_ENTRIES >= 2 ** 31 or q_total >= 2 ** 31 or (kv_offs.size and int(kv_offs.max()) >= 2 ** 31):
        raise ValueError("plan does not fit int32 tables")

    # request -> partial rows: rows grouped by request id, original order kept inside a group
    order = np.argsort(q_entries, kind="stable").astype(np.int32)
    counts = np.bincount(q_entries, minlength=batch_size).astype(np.int64)
    if counts.size > batch_size:
        raise ValueError("a request id in the tree is >= batch_size")
    r2v_lens = counts.astype(np.int32)
    r2v_offs = (np.cumsum(counts) - counts).astype(np.int32)

    big = np.flatnonzero(q_lens > small_tile)
    small = np.flatnonzero(q_lens <= small_tile)
    if order_key is not None:
        big = big[np.argsort(-order_key(kv_lens[big], q_lens[big]), kind="stable")]
        small = small[np.argsort(-order_key(kv_lens[small], q_lens[small]), kind="stable")]
    perm = np.concatenate([big, small])
    pad = np.full(PAD_ENTRIES, -1, dtype=np.int32)
    if order_out is not None:        # task i of the emitted tables is task order_out[i] of the emission order
        order_out.append(perm)
    return dict(
        vnode_to_kv_entries=None if direct_offsets else np.concatenate([cat(kv_chunks, np.int32), pad]),
        vnode_to_kv_offs=kv_offs[perm].astype(np.int32), vnode_to_kv_lens=kv_lens[perm].astype(np.int32),
        vnode_to_q_entries=q_entries,
        vnode_to_q_offs=q_offs[perm].astype(np.int32), vnode_to_q_lens=q_lens[perm].astype(np.int32),
        req_to_vnode_entries=np.concatenate([order, pad]),
        req_to_vnode_offs=r2v_offs, req_to_vnode_lens=r2v_lens,
        vnode_q_kv_ranges=np.ascontiguousarray(np.concatenate(range_chunks)) if any_ranges else None,
        phase_node_nums=[int(big.size), int(small.size)],
        phase_node_offsets=[0, int(big.size)],
        aux_segments=np.asarray(aux_segments, dtype=np.int32).reshape(-1, 4), aux_entries=int(aux_total),
    )


# ------------------------------------------------------- reference-compatible
def _children(tree):
    kids = [[] for _ in tree]
    for i in range(1, len(tree)):
        kids[tree[i].parent].append(i)
    return kids


def _pad_cost(n_q, n_k, tsq, tsk, alpha, beta, group):
    """alpha * (empty rows of the last request tile) * G * n_k
       + beta * (empty columns of a short KV tile) * n_q * G     (fasttree.py:30-45)"""
    ph = 0 if n_q > tsq[1] else 1
    empty_rows = tsq[ph] - ((n_q - 1) % tsq[ph] + 1)
    empty_cols = max(0, tsk[ph] - n_k)
    return alpha * empty_rows * group * n_k + beta * empty_cols * n_q * group


def greedy_edge_assignments(tree, params):
    """Per parent->child edge: 1 if the child's requests should take the
    parent's accumulated KV along (no extra partial row to merge), 0 if the
    child keeps a vnode of its own (fasttree.py:64-96)."""
    kids = _children(tree)
    tsq, tsk = params.TSQs, params.TSKs
    a, b, g, grp = params.alpha, params.beta, params.gamma, params.kv_group_num
    run_len = [nd.seqlen for nd in tree]
    assign = [0] * len(tree)
    frontier = deque((0,))
    while frontier:
        v = frontier.popleft()
        n_here = len(tree[v].requests)
        for c in kids[v]:
            n_c = len(tree[c].requests)
            own = (_pad_cost(n_here, run_len[v], tsq, tsk, a, b, grp)
                   + _pad_cost(n_c, run_len[c], tsq, tsk, a, b, grp) + g * n_c)
            carried = (_pad_cost(n_here - n_c, run_len[v], tsq, tsk, a, b, grp)
                       + _pad_cost(n_c, run_len[c] + run_len[v], tsq, tsk, a, b, grp))
            if own > carried:
                assign[c] = 1
                n_here -= n_c
                run_len[c] += run_len[v]
            frontier.append(c)
    return assign


def _requests_served(tree, assign):
    """Requests each node's own vnode serves: a leaf serves its request, an inner
    node the requests of every child subtree that did not carry its KV away.
    The order inside a node follows the reference's leaf-to-root queue
    (fasttree.py:126-141), which fixes the partial-row order."""
    n = len(tree)
    served = [[] for _ in range(n)]
    waiting = [nd.num_children for nd in tree]
    ready = deque()
    for i, nd in enumerate(tree):
        if nd.num_children == 0:
            served[i] = list(nd.requests)
            ready.append(i)
    while ready:
        v = ready.popleft()
        par = tree[v].parent
        if v != 0 and assign[v] == 0:
            served[par].extend(tree[v].requests)
        waiting[par] -= 1            # par == -1 at the root lands on the last node, as in the reference
        if waiting[par] == 0:
            ready.append(par)
    return served


def _chain_ranges(tree, kv_ptrs, assign, i):
    """Row ranges of node i preceded by every ancestor it carries (assign == 1)."""
    chain = [(kv_ptrs[i], kv_ptrs[i + 1])]
    up = i
    while assign[up] == 1:
        up = tree[up].parent
        chain.append((kv_ptrs[up], kv_ptrs[up + 1]))
    chain.reverse()
    return chain


def plan_reference(tree, kv_ptrs, batch_size, num_kv_heads, kv_split_sizes, para_threshs1, para_threshs2,
                   params, log=None):
    """Bit-exact re-implementation of the reference planner.  Mutates
    ``params.TSQs/TSKs`` exactly where the reference does (fasttree.py:181-186)."""
    tsq = list(params.TSQs)
    split = [kv_split_sizes[0], kv_split_sizes[0]]
    assign, served = None, None
    for rnd in range(3):
        assign = greedy_edge_assignments(tree, params)
        served = _requests_served(tree, assign)
        ctas = [0, 0]
        for i, reqs in enumerate(served):
            if not reqs:
                continue
            length = sum(e - b for b, e in _chain_ranges(tree, kv_ptrs, assign, i))
            ph = 0 if len(reqs) > tsq[1] else 1
            ctas[ph] += -(-len(reqs) // tsq[ph]) * -(-length // split[ph])
        ctas = [c * num_kv_heads for c in ctas]
        if log is not None:
            log.append(("parallelisms", list(ctas)))
        if rnd == 0:
            short = [ph for ph in range(2) if 0 < ctas[ph] < para_threshs1[ph]]
            for ph in short:
                split[ph] = kv_split_sizes[1]
            if not short:
                break
        elif rnd == 1:
            if 0 < ctas[0] < para_threshs2[0]:
                keep = 1
            elif 0 < ctas[1] < para_threshs2[1]:
                keep = 0
            else:
                break
            tsq = [tsq[keep], tsq[keep]]
            params.set_q_tile_sizes(tsq)
            params.set_kv_tile_sizes([params.TSKs[keep], params.TSKs[keep]])

    vnodes = []
    for i, reqs in enumerate(served):
        if not reqs:
            continue
        ph = 0 if len(reqs) > tsq[1] else 1
        vnodes.append(VirtualNode(_chain_ranges(tree, kv_ptrs, assign, i), np.asarray(reqs, dtype=np.int32),
                                  q_tile=tsq[0], kv_split=split[ph]))   # request tiles always use the big tile (:194,215)
    tabs = emit_tables(vnodes, batch_size, small_tile=tsq[1])
    return Plan(node_assignments=assign, phase_q_tile_sizes=list(tsq), phase_kv_tile_sizes=list(params.TSKs),
                kv_split_sizes=split, info={"planner": "reference"}, **tabs)


# ------------------------------------------------------------------ B200 splitter
@dataclass(frozen=True)
class B200Model:
    """Machine constants the splitter plans against (one B200: 148 SMs; the
    warp-MMA stage-1 kernel keeps two 112 KiB CTAs resident per SM)."""
    num_sms: int = 148
    ctas_per_sm: int = 2
    waves: float = 1.0              # aim for this many rounds of resident CTAs (measured: more chunks cost more in partial rows than they gain in balance)
    tile_tokens: int = 64           # KV tile of the stage-1 kernels
    rows_per_cta: int = 64          # query rows (requests x group) one CTA holds
    min_chunk: int = 128            # never cut a node's KV finer than this many tokens
    nominal_split: int = 512        # chunk length assumed while deciding the edges
    ridge_flop_per_byte: float = 90.0   # warp-MMA flops that cost as much time as one streamed byte
    task_overhead_bytes: int = 16384    # fixed cost of one more CTA, in streamed-byte equivalents
    elem_bytes: int = 2
    group_member_tokens: int = 128      # nodes up to this long (and few enough rows for the few-row kernels) may be grouped; 0: never
    group_min_members: int = 6          # a group must hold at least this many nodes to beat one task per node


def _task_cost(n_req, length, group, head_dim, m):
    """Cost, in streamed-byte equivalents per KV head, of pairing ``n_req``
    requests with ``length`` tokens: KV streamed once per 64-row block (or the
    tensor-core time if larger), fp32 partial rows written and read back once per
    chunk, and a fixed cost per CTA."""
    if n_req <= 0 or length <= 0:
        return 0.0
    rows = n_req * group
    row_blocks = -(-rows // m.rows_per_cta)
    chunks = -(-length // m.nominal_split)
    stream = row_blocks * length * 2 * head_dim * m.elem_bytes
    tensor = (-(-rows // 16) * 16) * length * 4 * head_dim / m.ridge_flop_per_byte
    partial = chunks * rows * (head_dim + 1) * 4 * 2
    return max(stream, tensor) + partial + row_blocks * chunks * m.task_overhead_bytes


def b200_edge_assignments(tree, group, head_dim, m):
    """Which children take their parent's accumulated KV along (1) and which keep a
    vnode of their own (0).  Breadth first, one parent at a time, on a cost model
    that charges what a B200 pays for: re-reading the parent's KV for a carrying
    child, partial-row traffic, and per-CTA overhead.  Three candidates per
    parent: the reference's greedy walk over the children in id order (the
    parent's remaining request count shrinking as children carry its KV away),
    no child carrying, and every child carrying - which is the only one that
    removes the parent's own tasks, something the edge-by-edge walk cannot see
    before its last child.  The cheapest wins (ties: greedy, then none)."""
    kids = _children(tree)
    run_len = [nd.seqlen for nd in tree]
    assign = [0] * len(tree)
    frontier = deque((0,))
    while frontier:
        v = frontier.popleft()
        n_v, len_v = len(tree[v].requests), run_len[v]
        if kids[v]:
            n_here, greedy, greedy_cost = n_v, [], 0.0
            for c in kids[v]:
                n_c = len(tree[c].requests)
                own = _task_cost(n_here, len_v, group, head_dim, m) + _task_cost(n_c, run_len[c], group, head_dim, m)
                carried = (_task_cost(n_here - n_c, len_v, group, head_dim, m)
                           + _task_cost(n_c, run_len[c] + len_v, group, head_dim, m))
                take = carried < own
                greedy.append(1 if take else 0)
                if take:
                    n_here -= n_c
                greedy_cost += _task_cost(n_c, run_len[c] + (len_v if take else 0), group, head_dim, m)
            greedy_cost += _task_cost(n_here, len_v, group, head_dim, m)
            none_cost = _task_cost(n_v, len_v, group, head_dim, m)
            all_cost, n_left = 0.0, n_v
            for c in kids[v]:
                n_c = len(tree[c].requests)
                none_cost += _task_cost(n_c, run_len[c], group, head_dim, m)
                all_cost += _task_cost(n_c, run_len[c] + len_v, group, head_dim, m)
                n_left -= n_c
            all_cost += _task_cost(n_left, len_v, group, head_dim, m)   # requests that end at v itself keep its vnode
            choice = greedy
            best = greedy_cost
            if none_cost < best:
                choice, best = [0] * len(kids[v]), none_cost
            if all_cost < best:
                choice, best = [1] * len(kids[v]), all_cost
            for c, take in zip(kids[v], choice):
                if take:
                    assign[c] = 1
                    run_len[c] += len_v
                frontier.append(c)
    return assign


def plan_b200(tree, kv_ptrs, batch_size, num_qo_heads, num_kv_heads, head_dim, params, model=None):
    """Tree -> balanced (node KV chunk x request group) tasks for one B200.

    1. edges: :func:`b200_edge_assignments`;
    2. request groups: ``rows_per_cta // G`` requests per task;
    3. KV chunks: a global per-task byte target = streamed bytes of the whole step
       / (SMs x resident CTAs x waves); each virtual node is cut into equal chunks
       (multiples of the 64-token tile, never below ``min_chunk``) so that no task
       exceeds the target - long shared prefixes are split, short leaves are not,
       which keeps the number of partial rows low;
    4. order: longest tasks first inside each phase (stable).

    ``num_kv_heads`` is the LOCAL head count of this GPU (the grid is tasks x
    local KV heads), so a head-sharded rank plans finer chunks.  Writes the
    request/KV tile sizes it used back into ``params`` like the reference does."""
    m = b200_model_for(params, head_dim, model)
    vnodes, assign, q_tile, small_tile, target = b200_virtual_nodes(
        tree, num_qo_heads, num_kv_heads, head_dim, m, lambda a, i: _chain_ranges(tree, kv_ptrs, a, i))
    if head_dim == 128 and m.elem_bytes == 2:      # the kernels that honour row ranges exist for this shape
        vnodes = b200_group_short_nodes(vnodes, q_tile, small_tile, m,
                                        int(math.floor(target / (2 * head_dim * m.elem_bytes))), num_kv_heads=num_kv_heads)
    vnodes = b200_split_tail(vnodes, q_tile, small_tile, m, num_kv_heads)
    tabs = emit_tables(vnodes, batch_size, small_tile=small_tile, order_key=b200_task_order)
    params.set_q_tile_sizes([q_tile, small_tile])
    params.set_kv_tile_sizes([m.tile_tokens, m.tile_tokens])
    return Plan(node_assignments=assign, phase_q_tile_sizes=[q_tile, small_tile],
                phase_kv_tile_sizes=[m.tile_tokens, m.tile_tokens], kv_split_sizes=[],
                info={"planner": "b200", "target_bytes": float(target), "vnodes": len(vnodes)}, **tabs)


def b200_group_short_nodes(vnodes, q_tile, small_tile, m, target_tokens, direct=False, num_kv_heads=1):
    """Packs short virtual nodes with pairwise disjoint request sets into groups
    that run as ONE many-row task: the members' KV is concatenated, their requests
    are concatenated, and each request attends only to its own member's tokens
    (``row_ranges``).  A tree of many short nodes otherwise becomes thousands of
    partly filled 64-token tiles, each a task with its own start-up and epilogue.

    Candidates are the virtual nodes with at most ``small_tile`` requests and at
    most ``group_member_tokens`` tokens, taken in order; a group is closed when
    the next candidate would exceed ``q_tile`` requests or 16 tiles of tokens,
    would exceed the per-task token target (at least 4 tiles) once the group has
    more than ``small_tile`` requests, or shares a request with it.  Groups
    with fewer than ``group_min_members`` members, or not more requests than
    ``small_tile``, are dissolved.  Result: the other virtual nodes in their
    order, then groups and dissolved candidates in the order they were closed.
    ``direct`` (serving path): every candidate is one run of an existing row-id
    table and a member's ``room`` - spare entries behind a tail that grows during
    the burst - counts as part of its length."""
    if m.group_member_tokens <= 0:
        return vnodes
    tile = m.tile_tokens
    hard_cap = GROUP_MAX_TILES * tile
    cap = min(max(target_tokens // tile * tile, 4 * tile), hard_cap)
    if direct:
        # serving path: the groups are sized so that the step fills two rounds of resident CTAs, the other tasks
        # included (measured on the 512-request burst, 16 other tasks on 37 slots: 36 / 53 / 73 / 80 / 120 tasks run
        # 69.7 / 61.9 / 55.7 / 68.5 / 76.1 us - their tiles are gathered row by row, and two shorter groups per slot
        # hide that latency better than one long one, while a third round costs more than it hides), up to 24 tiles
        cand_tokens = other = 0
        for vn in vnodes:
            length = sum(e - b for b, e in vn.kv_ranges)
            if len(vn.requests) <= small_tile and length + vn.room <= m.group_member_tokens:
                cand_tokens += length + vn.room
            else:
                other += -(-length // vn.kv_split) * -(-len(vn.requests) // vn.q_tile)
        round_ = max(int(m.num_sms * m.ctas_per_sm * m.waves) // max(num_kv_heads, 1), 1)
        free_tasks = max(2 * round_ - other, round_ // 2, 2)
        hard_cap = GROUP_MAX_TILES_DIRECT * tile
        cap = min(max(-(-(-(-cand_tokens // free_tasks)) // tile) * tile, 4 * tile), hard_cap)
    else:
        # One round: when the tasks at the default cap would spill a little past one round of resident CTAs while
        # longer groups keep everything inside it, the cap grows to what fills the round exactly (cfg3 on a 4-head
        # shard: 32 + 16 other tasks and 32 groups of 8 leaves are 80 tasks on 74 slots; 26 groups of 10 fit).
        cand_tokens = other = 0
        for vn in vnodes:
            length = sum(e - b for b, e in vn.kv_ranges)
            if len(vn.requests) <= small_tile and length <= m.group_member_tokens:
                cand_tokens += length
            else:
                other += -(-length // vn.kv_split) * -(-len(vn.requests) // vn.q_tile)
        round_ = max((m.num_sms * m.ctas_per_sm) // max(num_kv_heads, 1), 1)
        if other < round_ and other + -(-cand_tokens // cap) > round_:
            fill = -(-(-(-cand_tokens // (round_ - other))) // tile) * tile
            if fill <= hard_cap:
                cap = max(cap, fill)
    kept, tail = [], []
    cur, cur_reqs, cur_tokens, cur_n = [], set(), 0, 0

    def close():
        if len(cur) >= m.group_min_members and cur_n > small_tile:
            ranges, row_ranges, rooms, start = [], [], [], 0
            for vn, length in cur:
                ranges.extend(vn.kv_ranges)
                row_ranges.extend([(start, start + length)] * len(vn.requests))
                rooms.append(vn.room)
                start += length + vn.room
            tail.append(VirtualNode(ranges, np.concatenate([vn.requests for vn, _ in cur]), q_tile=q_tile,
                                    kv_split=-(-start // tile) * tile, row_ranges=row_ranges,
                                    member_room=rooms if direct else None))
        else:
            tail.extend(vn for vn, _ in cur)

    for vn in vnodes:
        length = sum(e - b for b, e in vn.kv_ranges)
        span = length + vn.room
        n = len(vn.requests)
        if n <= small_tile and span <= m.group_member_tokens:
            # (serving path: a group is closed once it has reached the cap, not before it would pass it, so that
            # the groups number no more than the tasks they were sized for)
            full = cur_tokens >= cap if direct else cur_tokens + span > cap
            if cur and (cur_n + n > q_tile or cur_tokens + span > hard_cap
                        or (full and cur_n > small_tile)
                        or any(int(r) in cur_reqs for r in vn.requests)):
                close()
                cur, cur_reqs, cur_tokens, cur_n = [], set(), 0, 0
            cur.append((vn, length))
            cur_reqs.update(int(r) for r in vn.requests)
            cur_tokens += span
            cur_n += n
        else:
            kept.append(vn)
    close()
    return kept + tail


TAIL_START_COST = (5, 4)   # fixed cost of a many-row / few-row task, in units of one 64-token tile's time
TAIL_ROUNDS = 1            # a late task is halved this many times at most (measured: quarters cost more in partial rows than they gain)


def b200_simulated_schedule(vnodes, q_tile, small_tile, m, slots):
    """List schedule of the tasks the virtual nodes will be cut into, in emission
    order (phase, then longest chunk first), on ``slots`` task slots - a task being
    the CTAs of all KV heads of one (chunk, request tile), which start side by side.
    Integer time: :data:`TAIL_START_COST` per task plus one unit per KV tile.
    Returns (makespan, total time of all tasks, per virtual node the time its last
    task ends)."""
    tasks = []
    for vi, vn in enumerate(vnodes):
        length = sum(e - b for b, e in vn.kv_ranges)
        nreq = len(vn.requests)
        if nreq == 0 or length <= 0:
            continue
        n_kv = -(-length // vn.kv_split)
        n_q = -(-nreq // vn.q_tile)
        for c in range(n_kv):
            c_len = min((c + 1) * vn.kv_split, length) - c * vn.kv_split
            for t in range(n_q):
                q_len = min((t + 1) * vn.q_tile, nreq) - t * vn.q_tile
                phase = 0 if q_len > small_tile else 1
                tasks.append((phase, -(c_len * 64 + min(q_len, 63)), len(tasks), vi,
                              TAIL_START_COST[phase] + -(-c_len // m.tile_tokens)))
    tasks.sort(key=lambda t: t[:3])
    free = [0] * max(slots, 1)
    heapq.heapify(free)
    last_end = [0] * len(vnodes)
    makespan = total = 0
    for _, _, _, vi, dur in tasks:
        start = heapq.heappop(free)
        heapq.heappush(free, start + dur)
        last_end[vi] = max(last_end[vi], start + dur)
        makespan = max(makespan, start + dur)
        total += dur
    return makespan, total, last_end


def b200_split_tail(vnodes, q_tile, small_tile, m, num_kv_heads):
    """Halves the KV chunks of the virtual nodes whose tasks end the step.  The
    hardware hands CTAs to slots in grid order, so a step of 2.05 or 2.6 rounds
    ends with a round in which a fraction of the slots run whole tasks while the
    rest of the GPU idles, and a step of one round lasts as long as its longest
    task; tasks half as long end it sooner at the price of a few more partial rows
    (cfg2: stage 1 25.0 -> 23.8 us, cfg3: 36.2 -> 33.7 us).  Decided on a simulated
    schedule (:func:`b200_simulated_schedule`): when the makespan exceeds the
    perfectly packed time by more than an eighth, every plain (ungrouped) virtual
    node with a task that ends in the later half of that excess is cut to half its
    chunk length (never below ``min_chunk``); the cut is kept if the simulated
    makespan drops."""
    slots = max((m.num_sms * m.ctas_per_sm) // max(num_kv_heads, 1), 1)
    for _ in range(TAIL_ROUNDS):
        makespan, total, last_end = b200_simulated_schedule(vnodes, q_tile, small_tile, m, slots)
        bound = -(-total // slots)
        if (makespan - bound) * 8 <= makespan:
            break
        late_from = makespan - (makespan - bound + 1) // 2
        trial, any_cut = list(vnodes), False
        for vi, vn in enumerate(vnodes):
            if vn.row_ranges is not None or last_end[vi] <= late_from:
                continue
            cur = min(vn.kv_split, sum(e - b for b, e in vn.kv_ranges))
            half = -(-(-(-cur // 2)) // m.tile_tokens) * m.tile_tokens
            if half >= m.min_chunk and half < cur:
                trial[vi] = replace(vn, kv_split=half)
                any_cut = True
        if not any_cut or b200_simulated_schedule(trial, q_tile, small_tile, m, slots)[0] >= makespan:
            break
        vnodes = trial
    return vnodes


def _tree_arrays(tree):
    n = len(tree)
    parent = np.fromiter((nd.parent for nd in tree), dtype=np.int32, count=n)
    seqlen = np.fromiter((nd.seqlen for nd in tree), dtype=np.int32, count=n)
    counts = np.fromiter((len(nd.requests) for nd in tree), dtype=np.int64, count=n)
    req_offs = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(counts, out=req_offs[1:])
    req_ids = np.zeros(max(int(req_offs[-1]), 1), dtype=np.int32)
    for i, nd in enumerate(tree):
        if counts[i]:
            req_ids[req_offs[i]:req_offs[i + 1]] = nd.requests
    return parent, seqlen, req_offs, req_ids


def _native_tables(build, direct):
    """Run one of the library's plan builders (``build(handle_ref) -> status``) and copy its tables out."""
    import ctypes
    from . import lib as _lib
    L = _lib.load()
    as32 = lambda a: a.ctypes.data_as(ctypes.POINTER(ctypes.c_int32))
    handle = ctypes.c_void_p()
    _lib.check(build(L, ctypes.byref(handle)))
    try:
        info = _lib.PlanInfo()
        _lib.check(L.ft_plan_get_info(handle, ctypes.byref(info)))
        tabs = dict(
            vnode_to_kv_entries=np.empty(info.kv_entries, dtype=np.int32),
            vnode_to_kv_offs=np.empty(info.vnodes, dtype=np.int32), vnode_to_kv_lens=np.empty(info.vnodes, dtype=np.int32),
            vnode_to_q_entries=np.empty(info.partial_rows, dtype=np.int32),
            vnode_to_q_offs=np.empty(info.vnodes, dtype=np.int32), vnode_to_q_lens=np.empty(info.vnodes, dtype=np.int32),
            req_to_vnode_entries=np.empty(info.partial_rows + PAD_ENTRIES, dtype=np.int32),
            req_to_vnode_offs=np.empty(info.batch, dtype=np.int32), req_to_vnode_lens=np.empty(info.batch, dtype=np.int32))
        assign = np.empty(info.nodes, dtype=np.int32)
        _lib.check(L.ft_plan_copy_tables(handle, *(as32(t) for t in tabs.values()), as32(assign)))
        if info.has_row_ranges:
            tabs["vnode_q_kv_ranges"] = np.empty((info.partial_rows, 2), dtype=np.int32)
            _lib.check(L.ft_plan_copy_row_ranges(handle, as32(tabs["vnode_q_kv_ranges"])))
        tabs["aux_segments"] = np.empty((info.aux_segments, 4), dtype=np.int32)
        tabs["aux_entries"] = int(info.aux_entries)
        if info.aux_segments:
            _lib.check(L.ft_plan_copy_aux_segments(handle, as32(tabs["aux_segments"])))
    finally:
        L.ft_plan_free(handle)
    if direct:
        tabs["vnode_to_kv_entries"] = None
    tabs["phase_node_nums"] = [int(x) for x in info.phase_node_nums]
    tabs["phase_node_offsets"] = [int(x) for x in info.phase_node_offsets]
    return tabs, [int(a) for a in assign], info


def _model_struct(m):
    from . import lib as _lib
    return _lib.B200ModelStruct(m.num_sms, m.ctas_per_sm, m.waves, m.tile_tokens, m.rows_per_cta, m.min_chunk,
                                m.nominal_split, m.ridge_flop_per_byte, m.task_overhead_bytes, m.elem_bytes,
                                m.group_member_tokens, m.group_min_members)


def plan_b200_native(tree, kv_ptrs, batch_size, num_qo_heads, num_kv_heads, head_dim, params, model=None):
    """:func:`plan_b200` computed by the native splitter of the shared library
    (``ft_plan_b200_build``, csrc/ft_planner.cu).  Same arguments, same result -
    the tests hold the two to identical tables; this one is one to two orders of
    magnitude faster on large trees.  Node 0 must be the root and parents must
    precede their children, as in the reference tree format."""
    import ctypes
    parent, seqlen, req_offs, req_ids = _tree_arrays(tree)
    ptrs = np.ascontiguousarray(np.asarray(kv_ptrs, dtype=np.int64))
    if ptrs.size != len(tree) + 1:
        raise ValueError("kv_ptrs must have one entry more than the tree has nodes")
    ms = _model_struct(b200_model_for(params, head_dim, model))
    i32p, i64p = ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int64)
    as32, as64 = (lambda a: a.ctypes.data_as(i32p)), (lambda a: a.ctypes.data_as(i64p))
    tabs, assign, info = _native_tables(
        lambda L, out: L.ft_plan_b200_build(as32(parent), as32(seqlen), len(tree), as64(req_offs), as32(req_ids),
                                            as64(ptrs), batch_size, num_qo_heads, num_kv_heads, head_dim,
                                            ctypes.byref(ms), out), direct=False)
    params.set_q_tile_sizes([info.q_tile, info.small_tile])
    params.set_kv_tile_sizes([info.tile_tokens, info.tile_tokens])
    return Plan(node_assignments=assign, phase_q_tile_sizes=[info.q_tile, info.small_tile],
                phase_kv_tile_sizes=[info.tile_tokens, info.tile_tokens], kv_split_sizes=[],
                info={"planner": "b200", "target_bytes": float(info.target_bytes), "vnodes": int(info.virtual_nodes)},
                **tabs)


def b200_tables_native_direct(tree, node_base, node_offset, extra, batch_size, num_qo_heads, num_kv_heads, head_dim,
                              model, tail_room=-1):
    """The serving path's tables from the native splitter (``ft_plan_b200_build_direct``): what
    :func:`b200_virtual_nodes` + :func:`emit_tables` (``direct_offsets=True``, ordered by
    :func:`b200_task_order`) produce for a tree whose node i covers positions
    ``[node_base[i] + node_offset[top carried ancestor], node_base[i] + node_offset[i] + seqlen_i)`` of an
    existing row-id table, plus the ``extra`` pairings ``(begin, end, request)``.
    Returns (tables dict, request tile, small request tile, tile tokens)."""
    import ctypes
    parent, seqlen, req_offs, req_ids = _tree_arrays(tree)
    base = np.ascontiguousarray(np.asarray(node_base, dtype=np.int64))
    offs = np.ascontiguousarray(np.asarray(node_offset, dtype=np.int64))
    ex = np.asarray(extra, dtype=np.int64).reshape(-1, 3)
    eb, ee = np.ascontiguousarray(ex[:, 0]), np.ascontiguousarray(ex[:, 1])
    er = np.ascontiguousarray(ex[:, 2].astype(np.int32))
    ms = _model_struct(model)
    i32p, i64p = ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int64)
    as32, as64 = (lambda a: a.ctypes.data_as(i32p)), (lambda a: a.ctypes.data_as(i64p))
    tabs, _assign, info = _native_tables(
        lambda L, out: L.ft_plan_b200_build_direct(as32(parent), as32(seqlen), len(tree), as64(req_offs), as32(req_ids),
                                                   as64(base), as64(offs), int(ex.shape[0]), as64(eb), as64(ee), as32(er),
                                                   int(tail_room), batch_size, num_qo_heads, num_kv_heads, head_dim,
                                                   ctypes.byref(ms), out), direct=True)
    return tabs, int(info.q_tile), int(info.small_tile), int(info.tile_tokens)


def b200_model_for(params, head_dim, model=None):
    explicit = model or getattr(params, "b200_model", None)
    m = explicit or B200Model()
    if explicit is None and head_dim == 128:
        # the tcgen05 stage-1 kernel holds 128 query rows per CTA (head_dim 128 only)
        m = replace(m, rows_per_cta=128, ridge_flop_per_byte=4 * m.ridge_flop_per_byte)
    if explicit is None and getattr(params, "kv_elem_bytes", 2) == 4:
        # fp32 storage runs on the CUDA-core kernel: 32-token tiles, one warp per scheduler, so a chunk costs
        # several microseconds per tile and a small problem is better cut down to single tiles
        m = replace(m, elem_bytes=4, tile_tokens=32, min_chunk=32)
    return m


def b200_task_order(kv_len, q_len):
    """Sort key of the tasks inside a phase: longest KV chunk first, more requests first."""
    return kv_len * 64 + np.minimum(q_len, 63)


def b200_virtual_nodes(tree, num_qo_heads, num_kv_heads, head_dim, m, ranges_of, extra=(), tail_room=-1):
    """Steps 1-3 of :func:`plan_b200` on any tree of node records (``parent``,
    ``seqlen``, ``num_children``, ``requests``).  ``ranges_of(assign, i)`` gives the
    KV row ranges of node i preceded by the ancestors it carries.  ``extra`` is a
    list of ``(ranges, requests)`` pairings outside the tree (per-request private
    tails) that take part in the byte budget and come last in emission order.
    ``tail_room >= 0`` (serving path, head_dim 128, 16-bit K/V): short pairings are
    then packed into groups (:func:`b200_group_short_nodes`, ``direct=True``), each
    ``extra`` member followed by ``tail_room`` spare row ids.
    Returns (virtual nodes, assignments, request tile, small request tile, byte target)."""
    group = max(1, num_qo_heads // num_kv_heads)
    q_tile = max(1, m.rows_per_cta // group)
    small_tile = max(1, min(q_tile, 16 // group if group <= 16 else 1))
    assign = b200_edge_assignments(tree, group, head_dim, m)

    carried_away = [set() for _ in tree]
    for i in range(1, len(tree)):
        if assign[i] == 1:
            carried_away[tree[i].parent].update(tree[i].requests)
    specs = []
    row_bytes = 2 * head_dim * m.elem_bytes
    total_stream = 0
    for i, nd in enumerate(tree):
        reqs = sorted(set(nd.requests) - carried_away[i])
        if not reqs:
            continue
        ranges = ranges_of(assign, i)
        length = sum(e - b for b, e in ranges)
        if length <= 0:
            continue
        specs.append((ranges, reqs, length, 0))
        total_stream += -(-len(reqs) // q_tile) * length * row_bytes
    for ranges, reqs in extra:
        length = sum(e - b for b, e in ranges)
        if length > 0 and len(reqs) > 0:
            specs.append((ranges, list(reqs), length, max(tail_room, 0)))
            total_stream += -(-len(reqs) // q_tile) * length * row_bytes
    slots = m.num_sms * m.ctas_per_sm * m.waves
    target = max(total_stream * num_kv_heads / slots, m.min_chunk * row_bytes)

    vnodes = []
    for ranges, reqs, length, room in specs:
        want = int(round(length * row_bytes / target))
        n_chunks = max(1, min(want, -(-length // m.min_chunk)))
        chunk = -(-length // n_chunks)
        chunk = -(-chunk // m.tile_tokens) * m.tile_tokens
        vnodes.append(VirtualNode(ranges, np.asarray(reqs, dtype=np.int32), q_tile=q_tile, kv_split=chunk, room=room))
    if tail_room >= 0 and head_dim == 128 and m.elem_bytes == 2:
        vnodes = b200_group_short_nodes(vnodes, q_tile, small_tile, m, int(math.floor(target / row_bytes)), direct=True,
                                        num_kv_heads=num_kv_heads)
    return vnodes, assign, q_tile, small_tile, target
