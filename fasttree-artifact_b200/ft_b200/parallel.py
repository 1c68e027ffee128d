"""Head (tensor) parallelism for the stand-alone multi-GPU path.

Tree attention is independent per KV head (the reference grid is
(vnodes, kv heads), kernel_bench/fasttree.py:448-451, and its kernels read the
head counts from the local tensor shapes, :605-607), so rank r of P owns KV heads
[r*Hkv/P, (r+1)*Hkv/P) and the matching query heads, plans with its LOCAL head
count, and needs no communication inside attention.  The only exchange is the
all-gather of the per-head outputs at the end of the step.
"""
import torch
import torch.distributed as dist


def head_shard(rank, world, num_qo_heads, num_kv_heads):
    """(first query head, query heads, first kv head, kv heads) owned by ``rank``."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    if num_kv_heads % world != 0 or num_qo_heads % num_kv_heads != 0:
        raise ValueError(f"{num_kv_heads} kv heads / {num_qo_heads} query heads cannot be sharded over {world} ranks")
    hkv = num_kv_heads // world
    group = num_qo_heads // num_kv_heads
    return rank * hkv * group, hkv * group, rank * hkv, hkv


def slice_heads(q, k_buffer, v_buffer, rank, world):
    """Views of this rank's heads of full tensors ``q [B,Hq,D]``, ``k/v [rows,Hkv,D]``."""
    q0, nq, k0, nk = head_shard(rank, world, q.shape[1], k_buffer.shape[1])
    return q[:, q0:q0 + nq], k_buffer[:, k0:k0 + nk], v_buffer[:, k0:k0 + nk]


def gather_heads(o_local, out=None, group=None):
    """All-gather ``o_local [B, Hq/P, D]`` into ``[B, Hq, D]`` (rank-major head
    order, which is the original head order under :func:`head_shard`).  ``out`` may
    be a pre-allocated ``[P, B, Hq/P, D]`` staging tensor."""
    world = dist.get_world_size(group)
    if world == 1:
        return o_local
    if out is None:
        out = torch.empty((world,) + tuple(o_local.shape), dtype=o_local.dtype, device=o_local.device)
    o_local = o_local.contiguous()
    if o_local.is_cuda:
        dist.all_gather_into_tensor(out, o_local, group=group)
    else:                                   # gloo: list form
        dist.all_gather(list(out.unbind(0)), o_local, group=group)
    b, h, d = o_local.shape
    return out.permute(1, 0, 2, 3).reshape(b, world * h, d)
