"""Oracle restatement of the reference's input side (test infrastructure only).

Covers, with citations into the reference tree:

* the node record                     kernel_bench/kv_tree_simple.py:4-10
* the tree text format                kernel_bench/tree_generation.py:78-94 (writer)
                                      kernel_bench/kv_tree_simple.py:50-64  (reader)
* the layered-tree parent rule        kernel_bench/tree_generation.py:47-71
* request assignment + Q/K/V draws    kernel_bench/flash_attn_wrap.py:5-79

plus the seeded irregular tree used as a stand-in for the random-tree
benchmark configuration (not part of the reference).
"""
from __future__ import annotations

import numpy as np
import torch


class OracleNode:
    """Same five fields as the reference node (kv_tree_simple.py:4-10)."""

    def __init__(self, parent=-1, id=-1, seqlen=0, num_children=0):
        self.parent = parent
        self.id = id
        self.seqlen = seqlen
        self.num_children = num_children
        self.requests = []

    def __repr__(self):
        return (f"OracleNode(parent={self.parent}, id={self.id}, seqlen={self.seqlen}, "
                f"num_children={self.num_children}, requests={self.requests})")


def layered_tree(level_sizes, level_lens):
    """Regular tree: ``level_sizes[k]`` nodes of ``level_lens[k]`` tokens on
    level k.  Child j of a level hangs under parent ``(j * prev) // size`` of
    the previous level (tree_generation.py:59-60); ids are assigned level by
    level."""
    if len(level_sizes) != len(level_lens):
        raise ValueError("level_sizes and level_lens must have equal length")
    nodes, prev, nxt = [], [], 0
    for depth, (size, slen) in enumerate(zip(level_sizes, level_lens)):
        cur = []
        for j in range(size):
            par = -1 if depth == 0 else prev[(j * len(prev)) // size]
            nodes.append(OracleNode(par, nxt, int(slen), 0))
            if par >= 0:
                nodes[par].num_children += 1
            cur.append(nxt)
            nxt += 1
        prev = cur
    return nodes


def random_tree(levels, seed, max_children=32, lam=3.0, len_lo=16, len_hi=2048):
    """Irregular tree with ``levels`` node-levels.  Nodes get BFS ids.  For each
    node in BFS order one context length ~ Uniform{len_lo..len_hi} is drawn,
    then (unless it sits on the last level) a child count
    ``min(max_children, 1 + Poisson(lam))``; generator is
    ``numpy.random.default_rng(seed)``."""
    rng = np.random.default_rng(seed)
    nodes = [OracleNode(-1, 0, 0, 0)]
    depth_of = [0]
    head = 0
    while head < len(nodes):
        nd = nodes[head]
        nd.seqlen = int(rng.integers(len_lo, len_hi + 1))
        if depth_of[head] < levels - 1:
            kids = int(min(max_children, 1 + rng.poisson(lam)))
            nd.num_children = kids
            for _ in range(kids):
                nodes.append(OracleNode(head, len(nodes), 0, 0))
                depth_of.append(depth_of[head] + 1)
        head += 1
    return nodes


def write_tree_file(nodes, path):
    """Line 1: node count; then ``parent id seqlen out_degree`` per node
    (tree_generation.py:78-94)."""
    with open(path, "w", encoding="utf-8") as fh:
        fh.write(f"{len(nodes)}\n")
        for nd in nodes:
            fh.write(f"{nd.parent} {nd.id} {nd.seqlen} {nd.num_children}\n")


def read_tree_file(path):
    """Inverse of :func:`write_tree_file` (kv_tree_simple.py:50-64); requests
    start empty."""
    with open(path, "r", encoding="utf-8") as fh:
        count = int(fh.readline())
        out = []
        for _ in range(count):
            par, nid, slen, deg = (int(tok) for tok in fh.readline().split())
            out.append(OracleNode(par, nid, slen, deg))
    return out


def assign_requests(nodes):
    """Leaves, visited in id order, receive request ids 0,1,2,...; every
    ancestor of a leaf also records that id (flash_attn_wrap.py:24-33).
    Returns the batch size."""
    for nd in nodes:
        nd.requests = []
    nreq = 0
    for nd in nodes:
        if nd.num_children == 0:
            cur = nd.id
            while cur != -1:
                nodes[cur].requests.append(nreq)
                cur = nodes[cur].parent
            nreq += 1
    return nreq


def kv_prefix_sums(nodes):
    """``KV_ptrs``: row range of node i in the flat tree tensors is
    ``[ptrs[i], ptrs[i+1])`` (flash_attn_wrap.py:13,22)."""
    ptrs = [0]
    for nd in nodes:
        ptrs.append(ptrs[-1] + nd.seqlen)
    return ptrs


def draw_qkv(nodes, num_qo_heads, num_kv_heads, head_dim, dtype, seed, q_scale=1.0):
    """Seeded CPU draws in the reference's order: for every node in id order a
    K block then a V block of shape (1, seqlen, Hkv, D) (flash_attn_wrap.py:16-21),
    and Q (B, Hq, D) drawn last (:69).  Request assignment is done here as in the
    reference.  The padded per-request caches of the reference are not built.

    Returns (Q, K_tree[T,Hkv,D], V_tree[T,Hkv,D], KV_ptrs, batch_size)."""
    gen_state = torch.random.get_rng_state()
    try:
        torch.manual_seed(seed)
        ks, vs = [], []
        for nd in nodes:
            ks.append(torch.randn(1, nd.seqlen, num_kv_heads, head_dim, dtype=dtype))
            vs.append(torch.randn(1, nd.seqlen, num_kv_heads, head_dim, dtype=dtype))
        batch = assign_requests(nodes)
        q = torch.randn(batch, num_qo_heads, head_dim, dtype=dtype)
    finally:
        torch.random.set_rng_state(gen_state)
    if q_scale != 1.0:
        q = (q.float() * q_scale).to(dtype)
    k_tree = torch.cat(ks, dim=1).reshape(-1, num_kv_heads, head_dim)
    v_tree = torch.cat(vs, dim=1).reshape(-1, num_kv_heads, head_dim)
    return q, k_tree, v_tree, kv_prefix_sums(nodes), batch


def algorithmic_work(nodes, num_qo_heads, num_kv_heads, head_dim, esize):
    """Algorithmic bytes and flops of one decode step over the tree: every
    node's K and V rows once plus Q read and O write; 4*D flops per
    (query head, token, request-under-node)."""
    total_tokens = sum(nd.seqlen for nd in nodes)
    batch = sum(1 for nd in nodes if nd.num_children == 0)
    nbytes = 2 * total_tokens * num_kv_heads * head_dim * esize \
        + 2 * batch * num_qo_heads * head_dim * esize
    flops = 4 * head_dim * num_qo_heads * sum(nd.seqlen * len(nd.requests) for nd in nodes)
    return nbytes, flops
