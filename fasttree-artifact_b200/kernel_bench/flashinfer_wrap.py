"""FlashInfer paged-decode yard-stick (reference: kernel_bench/flashinfer_wrap.py:5-46,
the "sglang_flashinfer" engine of kernel_bench/benchmark.py).

The reference feeds FlashInfer the padded per-request cache with page size 1.
Here the pages are the rows of the flat tree tensors themselves: request r's
page list is its root->leaf row sequence in ``K_tree``/``V_tree``, which is what
a radix-cache server hands FlashInfer (shared prefixes are shared pages) and
needs no padded copy.  Written for the plan()/run() API of flashinfer >= 0.2;
FlashInfer is an optional baseline - nothing in the engine depends on it.
"""
import torch


def request_paths(tree_info, KV_ptrs, batch_size):
    """Per request the K/V rows of its root->leaf path, as (indptr, indices) int32 lists."""
    leaf_of = [None] * batch_size
    for i, nd in enumerate(tree_info):
        if nd.num_children == 0:
            for r in nd.requests:
                leaf_of[r] = i
    indptr, indices = [0], []
    for r in range(batch_size):
        chain, cur = [], leaf_of[r]
        while cur is not None and cur != -1:
            chain.append(cur)
            cur = tree_info[cur].parent
        for node in reversed(chain):
            indices.extend(range(KV_ptrs[node], KV_ptrs[node + 1]))
        indptr.append(len(indices))
    return indptr, indices


def flashinfer_preparation(tree_info, KV_ptrs, batch_size, num_qo_heads, num_kv_heads, head_dim, dtype, device="cuda"):
    from flashinfer import BatchDecodeWithPagedKVCacheWrapper
    indptr, indices = request_paths(tree_info, KV_ptrs, batch_size)
    kv_indptr = torch.tensor(indptr, dtype=torch.int32, device=device)
    kv_indices = torch.tensor(indices, dtype=torch.int32, device=device)
    last_page_len = torch.ones(batch_size, dtype=torch.int32, device=device)
    workspace = torch.empty(384 * 1024 * 1024, dtype=torch.uint8, device=device)
    wrapper = BatchDecodeWithPagedKVCacheWrapper(workspace, "NHD", use_tensor_cores=num_qo_heads > num_kv_heads)
    wrapper.plan(kv_indptr, kv_indices, last_page_len, num_qo_heads, num_kv_heads, head_dim, 1,
                 q_data_type=dtype, kv_data_type=dtype)
    return wrapper


def flashinfer_decode(wrapper, Q, K_tree, V_tree):
    """K_tree/V_tree [T, Hkv, D] are viewed as T pages of one token each."""
    return wrapper.run(Q, (K_tree.unsqueeze(1), V_tree.unsqueeze(1)))
