"""Oracle arithmetic for tree-attention decode (test infrastructure only).

* :func:`per_leaf_attention` - the ground truth and the timed CPU baseline:
  for every request, concatenate the K/V rows of its root->leaf path
  (layout of kernel_bench/flash_attn_wrap.py:43-67) and evaluate
  softmax(q K^T * scale) V in fp32 with grouped-query heads.  Also returns the
  per-(request, head) log-sum-exp.
* :func:`stage1_partials` - what kernel_bench/fasttree.py:299-413 writes: for
  each vnode (KV chunk x request tile) the normalised partial output and
  ``log(sum)+max`` per (partial row, head).
* :func:`stage2_merge` - kernel_bench/fasttree.py:482-546: log-sum-exp
  weighted merge of each request's partial rows.

All math is fp32 on the CPU regardless of the storage dtype of Q/K/V.
"""
from __future__ import annotations

import numpy as np
import torch


def leaf_paths(nodes):
    """Request id -> list of node ids from the root down to the leaf."""
    paths = {}
    for nd in nodes:
        if nd.num_children == 0:
            chain, cur = [], nd.id
            while cur != -1:
                chain.append(cur)
                cur = nodes[cur].parent
            paths[nd.requests[0]] = chain[::-1]
    return [paths[r] for r in range(len(paths))]


def _attend(q, k, v, scale, group):
    """q [Hq,D] fp32, k/v [L,Hkv,D] fp32 -> (o [Hq,D], lse [Hq])."""
    hq, d = q.shape
    hkv = k.shape[1]
    qg = q.view(hkv, group, d)                             # heads kvh*G .. kvh*G+G-1 share kv head kvh
    s = torch.einsum("hgd,lhd->hgl", qg, k) * scale
    m = s.max(dim=-1, keepdim=True).values
    p = torch.exp(s - m)
    den = p.sum(dim=-1, keepdim=True)
    o = torch.einsum("hgl,lhd->hgd", p / den, v)
    lse = (torch.log(den) + m).reshape(hq)
    return o.reshape(hq, d), lse


def per_leaf_attention(nodes, kv_ptrs, q, k_tree, v_tree, scale, requests=None):
    """fp32 path-concatenated attention.  ``requests`` restricts the evaluation to
    a subset of request ids (used to bound the timed CPU sample).  Returns
    (O [n,Hq,D] fp32, LSE [n,Hq] fp32) in the order of ``requests``."""
    paths = leaf_paths(nodes)
    if requests is None:
        requests = range(len(paths))
    hq, hkv = q.shape[1], k_tree.shape[1]
    group = hq // hkv
    outs, lses = [], []
    for r in requests:
        rows = torch.cat([torch.arange(kv_ptrs[n], kv_ptrs[n + 1]) for n in paths[r]])
        k = k_tree.index_select(0, rows).float()
        v = v_tree.index_select(0, rows).float()
        o, lse = _attend(q[r].float(), k, v, scale, group)
        outs.append(o)
        lses.append(lse)
    return torch.stack(outs), torch.stack(lses)


def stage1_partials(q, k_buf, v_buf, kv_entries, kv_offs, kv_lens, q_entries, q_offs, q_lens,
                    scale, round_p_to=None, q_ranges=None):
    """Per-vnode partial attention.  Index tables are 1-D integer arrays in the
    reference's format.  Returns (mid_o [R,Hq,D], mid_lse [R,Hq]) fp32; rows no
    vnode covers stay NaN.  ``round_p_to`` optionally rounds the un-normalised
    probabilities to a storage dtype before the PV product, which is what the
    reference does with ``exp_logics.to(v.type)`` (fasttree.py:391).
    ``q_ranges`` ([R,2] integers, optional; an extension of the engine's own plan
    format with no counterpart in the reference) restricts partial row r to the
    tokens ``[begin, end)`` of its vnode's chunk; a row left with no token gets a
    zero partial and an LSE of -inf."""
    kv_entries = np.asarray(kv_entries).reshape(-1)
    q_entries = np.asarray(q_entries)
    rows_total = len(q_entries)
    hq, d = q.shape[1], q.shape[2]
    hkv = k_buf.shape[1]
    group = hq // hkv
    mid_o = torch.full((rows_total, hq, d), float("nan"), dtype=torch.float32)
    mid_lse = torch.full((rows_total, hq), float("nan"), dtype=torch.float32)
    for vn in range(len(kv_offs)):
        ko, kl, qo, ql = int(kv_offs[vn]), int(kv_lens[vn]), int(q_offs[vn]), int(q_lens[vn])
        if ql == 0 or kl == 0:
            continue
        rows = torch.as_tensor(kv_entries[ko:ko + kl].astype(np.int64))
        k = k_buf.index_select(0, rows).float()
        v = v_buf.index_select(0, rows).float()
        reqs = torch.as_tensor(q_entries[qo:qo + ql].astype(np.int64))
        qq = q.index_select(0, reqs).float().view(ql, hkv, group, d)
        s = torch.einsum("rhgd,lhd->rhgl", qq, k) * scale
        if q_ranges is not None:
            rng = torch.as_tensor(np.asarray(q_ranges).reshape(-1, 2)[qo:qo + ql].astype(np.int64))
            pos = torch.arange(kl).view(1, kl)
            seen = (pos >= rng[:, :1]) & (pos < rng[:, 1:])                      # [ql, kl]
            s = s.masked_fill(~seen.view(ql, 1, 1, kl), float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        m = torch.where(torch.isinf(m), torch.zeros_like(m), m)                  # rows that see no token
        p = torch.exp(s - m)
        den = p.sum(dim=-1, keepdim=True)
        if round_p_to is not None:
            p = p.to(round_p_to).float()
        o = torch.einsum("rhgl,lhd->rhgd", p, v) / den.clamp_min(1e-38)
        lse = torch.where(den > 0, torch.log(den) + m, torch.full_like(den, float("-inf")))
        mid_o[qo:qo + ql] = o.reshape(ql, hq, d)
        mid_lse[qo:qo + ql] = lse.reshape(ql, hq)
    return mid_o, mid_lse


def stage2_merge(mid_o, mid_lse, r2v_entries, r2v_offs, r2v_lens):
    """Per-(request, head) merge of partial rows.  Returns (O [B,Hq,D] fp32,
    LSE [B,Hq] fp32).  The reference does not expose the merged LSE; it is
    returned here because the engine can optionally write it."""
    r2v_entries = np.asarray(r2v_entries)
    bsz = len(r2v_offs)
    hq, d = mid_o.shape[1], mid_o.shape[2]
    out = torch.zeros((bsz, hq, d), dtype=torch.float32)
    lse = torch.zeros((bsz, hq), dtype=torch.float32)
    for r in range(bsz):
        rows = torch.as_tensor(r2v_entries[int(r2v_offs[r]):int(r2v_offs[r]) + int(r2v_lens[r])]
                               .astype(np.int64))
        part_lse = mid_lse.index_select(0, rows)            # [n,Hq]
        part_o = mid_o.index_select(0, rows)                # [n,Hq,D]
        m = part_lse.max(dim=0, keepdim=True).values
        w = torch.exp(part_lse - m)
        den = w.sum(dim=0)
        out[r] = (w.unsqueeze(-1) * part_o).sum(dim=0) / den.unsqueeze(-1)
        lse[r] = torch.log(den) + m.squeeze(0)
    return out, lse


def tree_decode(q, k_buf, v_buf, plan, scale):
    """Stage 1 followed by stage 2 on an :class:`OraclePlan`-like object."""
    mid_o, mid_lse = stage1_partials(q, k_buf, v_buf, plan.kv_entries, plan.kv_offs, plan.kv_lens,
                                     plan.q_entries, plan.q_offs, plan.q_lens, scale,
                                     q_ranges=getattr(plan, "q_ranges", None))
    return stage2_merge(mid_o, mid_lse, plan.r2v_entries, plan.r2v_offs, plan.r2v_lens)
