"""Head-sharded (tensor-parallel) path on CPU ranks: two gloo processes each
own half of the KV heads, evaluate their slice with the oracle (no GPU here),
all-gather the outputs and compare with the unsharded result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ft_b200 import parallel


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for p in (root, os.path.join(root, "fasttree-artifact_b200")):
        sys.path.insert(0, p)
    from oracle import ref_attention, ref_inputs
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        nodes = ref_inputs.layered_tree([1, 3, 6], [50, 20, 9])
        q, k, v, ptrs, batch = ref_inputs.draw_qkv(nodes, 8, 4, 64, torch.float32, seed=5)
        full, _ = ref_attention.per_leaf_attention(nodes, ptrs, q, k, v, 0.125)
        ql, kl, vl = parallel.slice_heads(q, k, v, rank, world)
        assert ql.shape[1] == 8 // world and kl.shape[1] == 4 // world
        local, _ = ref_attention.per_leaf_attention(nodes, ptrs, ql.contiguous(), kl.contiguous(), vl.contiguous(),
                                                    0.125)
        gathered = parallel.gather_heads(local)
        ok = torch.allclose(gathered, full, atol=1e-6) and gathered.shape == full.shape
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_rank_head_sharding_matches_unsharded():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def test_head_shard_arithmetic():
    assert parallel.head_shard(0, 1, 32, 8) == (0, 32, 0, 8)
    assert parallel.head_shard(3, 8, 32, 8) == (12, 4, 3, 1)
    assert parallel.head_shard(1, 2, 64, 8) == (32, 32, 4, 4)
    with pytest.raises(ValueError):
        parallel.head_shard(0, 3, 32, 8)
    with pytest.raises(ValueError):
        parallel.head_shard(2, 2, 32, 8)
