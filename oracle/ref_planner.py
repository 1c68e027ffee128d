"""Oracle restatement of the reference's host planner (test infrastructure only).

Follows kernel_bench/fasttree.py:

* hyper-parameter bag                          :7-27
* padding cost model                           :30-61
* greedy split-K / split-Q edge heuristic      :64-96
* parallelism count and the 3-pass adaptation  :126-188
* vnode / partial-row table emission           :193-231
* request -> partial-row CSR                   :233-244
* stable two-phase partition                   :246-259
* 32-entry ``-1`` tails on the two index lists :261-262

The tables come back as numpy int32 arrays (the reference uploads them as
int32 CUDA tensors, :265-274).  Device scratch (``mid_o``/``mid_lse``) is not
created here; its row count is ``len(plan.q_entries)``.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import numpy as np


class OracleParams:
    """Same defaults and setters as the reference bag (fasttree.py:7-27)."""

    def __init__(self):
        self.alpha = 0.66
        self.beta = 0.33
        self.gamma = 0.1
        self.TSQs = [64, 16]
        self.TSKs = [32, 128]
        self.kv_group_num = 1

    def set_values(self, alpha, beta, gamma):
        self.alpha, self.beta, self.gamma = alpha, beta, gamma

    def set_kv_group_num(self, g):
        self.kv_group_num = g

    def set_q_tile_sizes(self, tsqs):
        self.TSQs = tsqs

    def set_kv_tile_sizes(self, tsks):
        self.TSKs = tsks


# ----------------------------------------------------------------- cost model
def pad_q(tile, n):
    """Empty rows in the last query tile (fasttree.py:30-31)."""
    return tile - ((n - 1) % tile + 1)


def pad_k(tile, n):
    """Empty columns when a KV segment is shorter than one tile (:34-35)."""
    return max(0, tile - n)


def cost_mm(n_q, n_k, p):
    """Padding cost of pairing n_q requests with n_k tokens (:38-45)."""
    ph = 0 if n_q > p.TSQs[1] else 1
    return (p.alpha * pad_q(p.TSQs[ph], n_q) * p.kv_group_num * n_k
            + p.beta * pad_k(p.TSKs[ph], n_k) * n_q * p.kv_group_num)


def cost_keep_child_vnode(n_cur, n_child, len_child, len_par, p):
    """"Split-K": child keeps its own vnode, one more partial to merge
    (:48-49, :56-61)."""
    return cost_mm(n_cur, len_par, p) + cost_mm(n_child, len_child, p) + p.gamma * n_child


def cost_absorb_parent(n_cur, n_child, len_par, len_child, p):
    """"Split-Q": the child's queries take the parent's KV with them (:52-53)."""
    return cost_mm(n_cur - n_child, len_par, p) + cost_mm(n_child, len_child + len_par, p)


def greedy_assignments(tree, p):
    """Breadth-first walk from node 0; assignment 1 means "this node's vnode
    also carries the KV accumulated on its parent" (:64-96)."""
    n = len(tree)
    kids = [[] for _ in range(n)]
    for i in range(1, n):
        kids[tree[i].parent].append(i)
    acc_len = [tree[i].seqlen for i in range(n)]
    assign = [0] * n
    todo = deque([0])
    while todo:
        v = todo.popleft()
        n_cur = len(tree[v].requests)
        len_v = acc_len[v]
        for c in kids[v]:
            n_c = len(tree[c].requests)
            len_c = acc_len[c]
            keep = cost_keep_child_vnode(n_cur, n_c, len_c, len_v, p)
            absorb = cost_absorb_parent(n_cur, n_c, len_v, len_c, p)
            if keep > absorb:
                assign[c] = 1
                n_cur -= n_c
                acc_len[c] = len_c + len_v
            else:
                assign[c] = 0
            todo.append(c)
    return assign


@dataclass
class OraclePlan:
    kv_entries: np.ndarray
    kv_offs: np.ndarray
    kv_lens: np.ndarray
    q_entries: np.ndarray
    q_offs: np.ndarray
    q_lens: np.ndarray
    r2v_entries: np.ndarray
    r2v_offs: np.ndarray
    r2v_lens: np.ndarray
    phase_node_nums: list
    phase_node_offsets: list
    node_assignments: list
    q_tiles: list = field(default_factory=list)     # effective per-phase request tile
    kv_splits: list = field(default_factory=list)   # effective per-phase KV split
    parallelism_log: list = field(default_factory=list)


def plan_reference(tree, kv_ptrs, batch_size, num_kv_heads, kv_split_sizes,
                   para_threshs1, para_threshs2, p):
    """fasttree_preparation restated (fasttree.py:99-296).  ``p`` is mutated the
    way the reference mutates its parameter bag (:181-186)."""
    n = len(tree)
    q_tiles = p.TSQs
    kv_split = [kv_split_sizes[0], kv_split_sizes[0]]
    assign = None
    log = []

    def count_ctas():
        # :126-161.  Requests bubble up from the leaves through every child that
        # keeps its own vnode; a child with assignment 1 does not hand its
        # requests to the parent.
        reqs = [[] for _ in range(n)]
        pending = [tree[i].num_children for i in range(n)]
        todo = deque()
        for i in range(n):
            if tree[i].num_children == 0:
                todo.append(i)
                reqs[i] = list(tree[i].requests)
        while todo:
            v = todo.popleft()
            par = tree[v].parent          # -1 for the root: Python wraps to the last node (:139)
            if assign[v] == 0 and v != 0:
                reqs[par] += tree[v].requests
            pending[par] -= 1
            if pending[par] == 0:
                todo.append(par)
        par_count = [0, 0]
        for i in range(n):
            r = len(reqs[i])
            if r == 0:
                continue
            length = tree[i].seqlen
            up = i
            while assign[up] == 1:
                up = tree[up].parent
                length += tree[up].seqlen
            ph = 0 if r > q_tiles[1] else 1
            par_count[ph] += ((r - 1) // q_tiles[ph] + 1) * ((length - 1) // kv_split[ph] + 1)
        return [c * num_kv_heads for c in par_count], reqs

    reqs = None
    for rnd in range(3):                                           # :163-188
        assign = greedy_assignments(tree, p)
        par_count, reqs = count_ctas()
        log.append(list(par_count))
        if rnd == 0:
            stop = True
            for ph in range(2):
                if 0 < par_count[ph] < para_threshs1[ph]:
                    kv_split[ph] = kv_split_sizes[1]
                    stop = False
            if stop:
                break
        elif rnd == 1:
            if 0 < par_count[0] < para_threshs2[0]:
                q_tiles = [q_tiles[1], q_tiles[1]]
                p.set_q_tile_sizes(q_tiles)
                p.set_kv_tile_sizes([p.TSKs[1], p.TSKs[1]])
            elif 0 < par_count[1] < para_threshs2[1]:
                q_tiles = [q_tiles[0], q_tiles[0]]
                p.set_q_tile_sizes(q_tiles)
                p.set_kv_tile_sizes([p.TSKs[0], p.TSKs[0]])
            else:
                break

    kv_entries = []
    kv_offs, kv_lens, q_entries, q_offs, q_lens = [], [], [], [], []
    big_tile = q_tiles[0]
    for i in range(n):                                             # :193-231
        r = len(reqs[i])
        if r == 0:
            continue
        ph = 0 if r > q_tiles[1] else 1
        split = kv_split[ph]
        chain = [i]
        while assign[chain[-1]] == 1:
            chain.append(tree[chain[-1]].parent)
        rows = []
        for nd in reversed(chain):                                 # root-most segment first
            rows.extend(range(kv_ptrs[nd], kv_ptrs[nd + 1]))
        length = len(rows)
        base = len(kv_entries)
        kv_entries.extend(rows)
        for c in range((length - 1) // split + 1):
            q_base = len(q_entries)
            q_entries.extend(reqs[i])
            c_off = c * split
            c_len = min(c_off + split, length) - c_off
            for t in range((r - 1) // big_tile + 1):
                t_off = t * big_tile
                kv_offs.append(base + c_off)
                kv_lens.append(c_len)
                q_offs.append(q_base + t_off)
                q_lens.append(min(t_off + big_tile, r) - t_off)

    per_req = [[] for _ in range(batch_size)]                      # :233-244
    for row, rq in enumerate(q_entries):
        per_req[rq].append(row)
    r2v_offs, r2v_lens, r2v_entries = [], [], []
    for rq in range(batch_size):
        r2v_offs.append(len(r2v_entries))
        r2v_lens.append(len(per_req[rq]))
        r2v_entries.extend(per_req[rq])

    thr = q_tiles[1]                                               # :246-259
    big = [j for j, ql in enumerate(q_lens) if ql > thr]
    small = [j for j, ql in enumerate(q_lens) if ql <= thr]
    order = big + small

    def take(lst):
        return np.asarray([lst[j] for j in order], dtype=np.int32)

    i32 = lambda lst: np.asarray(lst, dtype=np.int32)
    return OraclePlan(
        kv_entries=i32(kv_entries + [-1] * 32),                    # :261
        kv_offs=take(kv_offs), kv_lens=take(kv_lens),
        q_entries=i32(q_entries),
        q_offs=take(q_offs), q_lens=take(q_lens),
        r2v_entries=i32(r2v_entries + [-1] * 32),                  # :262
        r2v_offs=i32(r2v_offs), r2v_lens=i32(r2v_lens),
        phase_node_nums=[len(big), len(small)],
        phase_node_offsets=[0, len(big)],
        node_assignments=assign,
        q_tiles=list(q_tiles), kv_splits=list(kv_split), parallelism_log=log,
    )
