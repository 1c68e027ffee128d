"""Synthetic inputs of the micro-benchmark (the reference's qkv_preparation,
kernel_bench/flash_attn_wrap.py:5-79).

Draw order is the reference's: for every node in id order a K block then a V
block of shape (1, seqlen, Hkv, D); Q (B, Hq, D) last.  Leaves, in id order, get
request ids 0,1,2,... which are recorded on the leaf and on all its ancestors.

The padded per-request caches ``K_cache/V_cache [B, max_path, Hkv, D]`` only
feed the reference's dense baselines; pass ``padded_cache=False`` to skip them
(they reach tens of GiB on wide trees) - the two entries then come back None.
"""
import torch


def qkv_preparation(tree_info, num_qo_heads, num_kv_heads, head_dim, device="cuda", dtype=torch.float16,
                    padded_cache=True):
    k_blocks, v_blocks, ptrs = [], [], [0]
    paths = []
    for nd in tree_info:
        k_blocks.append(torch.randn(1, nd.seqlen, num_kv_heads, head_dim, device=device, dtype=dtype))
        v_blocks.append(torch.randn(1, nd.seqlen, num_kv_heads, head_dim, device=device, dtype=dtype))
        ptrs.append(ptrs[-1] + nd.seqlen)
        if nd.num_children == 0:
            chain, cur = [], nd.id
            while cur != -1:
                tree_info[cur].requests.append(len(paths))
                chain.append(cur)
                cur = tree_info[cur].parent
            paths.append(chain[::-1])
    batch = len(paths)
    seqlens = [sum(tree_info[n].seqlen for n in chain) for chain in paths]
    K_cache = V_cache = None
    if padded_cache:
        longest = max(seqlens) if seqlens else 0
        K_cache = torch.empty(batch, longest, num_kv_heads, head_dim, device=device, dtype=dtype)
        V_cache = torch.empty_like(K_cache)
        for r, chain in enumerate(paths):
            K_cache[r, :seqlens[r]] = torch.cat([k_blocks[n][0] for n in chain], dim=0)
            V_cache[r, :seqlens[r]] = torch.cat([v_blocks[n][0] for n in chain], dim=0)
    Q = torch.randn(batch, num_qo_heads, head_dim, device=device, dtype=dtype)
    cache_seqlens = torch.tensor(seqlens, dtype=torch.int32, device=device)
    K_tree = torch.cat(k_blocks, dim=1).reshape(-1, num_kv_heads, head_dim)
    V_tree = torch.cat(v_blocks, dim=1).reshape(-1, num_kv_heads, head_dim)
    return Q, K_cache, V_cache, cache_seqlens, K_tree, V_tree, ptrs
