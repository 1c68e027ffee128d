"""Helpers for the GPU parity tests: run the product path (planner -> C ABI
kernels) on a decode case built by ``cases.build_decode_case`` or on an ad-hoc
tree."""
import torch

import fasttree
from ft_b200 import engine
from kv_tree_simple import KVTreeNode


def product_tree(onodes):
    out = [KVTreeNode(n.parent, n.id, n.seqlen, n.num_children) for n in onodes]
    for nd, src in zip(out, onodes):
        nd.requests = list(src.requests)
    return out


def make_params(hq, hkv, tsq, planner):
    p = fasttree.FastTreeParams()
    p.set_values(0.66, 0.33, 0.1)
    p.set_q_tile_sizes(list(tsq))
    p.set_kv_tile_sizes([32, 32])
    p.set_kv_group_num(hq // hkv)
    p.set_planner(planner)
    return p


class EngineRun:
    """One planned decode problem resident on the GPU."""

    def __init__(self, nodes, ptrs, batch, q, k, v, hq, hkv, d, tsq, planner="b200", device="cuda", tell_dtype=False):
        self.tree = product_tree(nodes)
        self.params = make_params(hq, hkv, tsq, planner)
        if tell_dtype:      # the splitter then cuts fp32 problems for the 32-token CUDA-core kernel
            self.params.set_kv_dtype(k.dtype)
        self.aux, self.assign = fasttree.fasttree_preparation(
            self.tree, ptrs, batch, hq, hkv, d, [1024, 128], [132, 528], [132, 132], self.params, device=device)
        self.q, self.k, self.v = q.to(device), k.to(device), v.to(device)
        self.o = torch.empty_like(self.q)
        self.o_lse = torch.empty(batch, hq, dtype=torch.float32, device=device)
        self.scale = 1.0 / d ** 0.5
        self.tiles = (list(self.params.TSQs), list(self.params.TSKs))

    @property
    def mid_o(self):
        return self.aux[9]

    @property
    def mid_lse(self):
        return self.aux[10]

    def decode(self, path="auto", poison=True, with_lse=True):
        if poison:
            self.mid_o.fill_(float("nan"))
            self.mid_lse.fill_(float("nan"))
            self.o.fill_(float("nan"))
        engine.decode(self.q, self.k, self.v, self.o, *self.aux, self.tiles[0], self.tiles[1], self.scale,
                      path=path, o_lse=self.o_lse if with_lse else None)
        torch.cuda.synchronize()
        return self.o.float().cpu()

    def decode_via_dropin(self):
        """Through the reference-signature entry point."""
        fasttree.fasttree_decode(self.q, self.k, self.v, self.o, *self.aux, self.tiles[0], self.tiles[1],
                                 self.scale)
        torch.cuda.synchronize()
        return self.o.float().cpu()


def run_case(c, planner="b200", path="auto", tell_dtype=False):
    run = EngineRun(c["nodes"], c["ptrs"], c["batch"], c["q"], c["k"], c["v"], c["hq"], c["hkv"], c["d"],
                    c["tsq"], planner=planner, tell_dtype=tell_dtype)
    out = run.decode(path=path)
    return run, out
