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


def cascade_levels(tree_info, KV_ptrs, batch_size):
    """The tree as FlashInfer's multi-level cascade wants it (reference: kernel_bench/bench_cascade.py:117-159):
    per tree depth the nodes of that depth in id order, each node's K/V rows as its pages and the (consecutive)
    requests below it as its query range.  Works for any tree whose requests below a node are consecutive ids and
    whose leaves all sit on the last level (the layered and the seeded irregular trees of this package)."""
    depth = [0] * len(tree_info)
    for i, nd in enumerate(tree_info):
        depth[i] = 0 if nd.parent < 0 else depth[nd.parent] + 1
    levels = max(depth) + 1
    qo_indptr, kv_indptr, kv_indices = [], [], []
    for lv in range(levels):
        nodes = [i for i in range(len(tree_info)) if depth[i] == lv]
        qo, kv, idx = [0], [0], []
        covered = 0
        for i in nodes:
            reqs = sorted(tree_info[i].requests)
            if not reqs:
                continue
            if reqs != list(range(reqs[0], reqs[0] + len(reqs))) or reqs[0] != covered:
                raise ValueError("cascade needs every level to split the requests into consecutive ranges")
            covered += len(reqs)
            qo.append(covered)
            idx.extend(range(KV_ptrs[i], KV_ptrs[i + 1]))
            kv.append(len(idx))
        if covered != batch_size:
            raise ValueError("cascade needs every request to pass through every level")
        qo_indptr.append(qo)
        kv_indptr.append(kv)
        kv_indices.append(idx)
    return qo_indptr, kv_indptr, kv_indices


def cascade_preparation(tree_info, KV_ptrs, batch_size, num_qo_heads, num_kv_heads, head_dim, dtype, device="cuda"):
    """FlashInfer's MultiLevelCascadeAttentionWrapper over the flat tree tensors, page size 1: the engine of the
    reference's cascade yard-stick (kernel_bench/bench_cascade.py), an optional baseline like the paged decode."""
    from flashinfer import MultiLevelCascadeAttentionWrapper
    qo_indptr, kv_indptr, kv_indices = cascade_levels(tree_info, KV_ptrs, batch_size)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
    workspace = torch.empty(512 * 1024 * 1024, dtype=torch.uint8, device=device)
    wrapper = MultiLevelCascadeAttentionWrapper(len(qo_indptr), workspace, "NHD")
    wrapper.plan([i32(q) for q in qo_indptr], [i32(k) for k in kv_indptr], [i32(x) for x in kv_indices],
                 [torch.ones(len(k) - 1, dtype=torch.int32, device=device) for k in kv_indptr],
                 num_qo_heads, num_kv_heads, head_dim, 1, q_data_type=dtype)
    return wrapper


def cascade_decode(wrapper, Q, K_tree, V_tree):
    return wrapper.run(Q, (K_tree.unsqueeze(1), V_tree.unsqueeze(1)))
