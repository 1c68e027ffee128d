"""Pre-allocated plan buffers of one TP worker (reference:
fasttree_sglang_plugin_v0_2_13/metadata.py:5-66): hyper-parameters, fixed-capacity
int32 plan tables and the fp32 partial-result scratch, allocated once so that the
decode path never allocates."""
from typing import List, Tuple

import torch


class FastTreeMetadata:
    def __init__(
        self,
        num_qo_heads: int,
        num_kv_heads: int,
        head_dim: int,
        device="cuda",
        alpha: float = 0.6,
        beta: float = 0.3,
        gamma: float = 0.1,
        TSQs: Tuple[int, int] = None,
        TSKs: Tuple[int, int] = (32, 32),
        kv_split_sizes: Tuple[int, int] = (1024, 128),
        para_threshs1: Tuple[int, int] = (132, 132),
        para_threshs2: Tuple[int, int] = (132, 528),
        max_vnodes: int = 16384,
        max_vnode_to_q_entries: int = 81920,
        max_batch_size: int = 8192,
        planner: str = "b200",
        graph_safe: bool = False,
        group_tails: bool = True,
        tail_room: int = 12,
        group_tails_min_load: float = 4.0,
        max_aux_entries: int = 1 << 20,
    ):
        if planner not in ("b200", "reference"):
            raise ValueError("planner must be 'b200' or 'reference'")
        self.num_qo_heads = num_qo_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.kv_group_num = num_qo_heads // num_kv_heads
        self.device = device
        self.alpha, self.beta, self.gamma = alpha, beta, gamma
        self.TSQs = TSQs if TSQs is not None else (64 // self.kv_group_num, 16 // self.kv_group_num)
        self.TSKs = TSKs
        self.kv_split_sizes = kv_split_sizes
        self.para_threshs1 = para_threshs1
        self.para_threshs2 = para_threshs2
        self.planner = planner
        self.native_planner = True      # "b200": the library's native splitter (False: its Python specification)
        # graph_safe: the decode call reads the phase split from the device (phase_info_dev) and runs the
        # persistent stage-1 kernel, whose launch does not depend on the plan - a decode step captured in a CUDA
        # graph then stays valid from burst to burst (16-bit KV, head_dim 128).  No counterpart in the reference.
        self.graph_safe = bool(graph_safe)
        # group_tails ("b200" planner, head_dim 128): short private runs - above all the per-request tails, one
        # one-tile task per request and KV head otherwise - are packed into many-row vnodes with per-row token
        # ranges.  Their row ids are gathered into kv_entries_aux once per burst; every tail is followed by
        # tail_room spare entries, which bounds the steps of a burst (SGLang v0.2.13 runs 10).  No counterpart
        # in the reference (schedule.py:212-232 emits one tail task per request).
        self.group_tails = bool(group_tails) and planner == "b200" and head_dim == 128
        self.tail_room = int(tail_room)
        # Grouping pays when the tails alone would queue up behind the machine's resident CTAs: a burst is planned
        # with groups only if (private tails x local KV heads) is at least this many times the resident CTA count
        # (measured on the four traffic shapes: below about 4 the one-task-per-tail plan is the faster one).
        self.group_tails_min_load = float(group_tails_min_load)
        if self.group_tails and self.tail_room < 1:
            raise ValueError("tail_room must be at least 1 when tails are grouped")
        self.merge_private_nodes = True   # single-request radix nodes join the request's tail ("b200" planner)
        self.max_vnodes = max_vnodes
        self.max_vnode_to_q_entries = max_vnode_to_q_entries
        self.max_batch_size = max_batch_size

        def i32(n):
            return torch.empty(n, dtype=torch.int32, device=device)

        self.vnode_to_q_entries = i32(max_vnode_to_q_entries)
        self.vnode_to_q_offs = i32(max_vnodes)
        self.vnode_to_q_lens = i32(max_vnodes)
        self.vnode_to_kv_offs = i32(max_vnodes)
        self.vnode_to_kv_lens = i32(max_vnodes)
        self.req_to_vnode_entries = i32(max_vnode_to_q_entries)
        self.req_to_vnode_offs = i32(max_batch_size)
        self.req_to_vnode_lens = i32(max_batch_size)
        self.req_last_vnodes_dev = i32(max_batch_size)      # device copy of req_last_vnodes for the per-step bump
        self.phase_info_dev = torch.zeros(4, dtype=torch.int32, device=device)   # n0, n1, o0, o1 of the current plan
        # per request {aux_pos | -1, src_pos, partial row | vnode, room}: what the per-step bump advances
        self.tail_state = torch.full((max_batch_size, 4), -1, dtype=torch.int32, device=device)
        if self.group_tails:
            self.kv_entries_aux = i32(max_aux_entries)
            self.vnode_q_kv_ranges = i32(2 * max_vnode_to_q_entries).view(max_vnode_to_q_entries, 2)
            self.aux_segments = i32(4 * (max_batch_size + max_vnodes)).view(4, max_batch_size + max_vnodes)
        else:
            self.kv_entries_aux = self.vnode_q_kv_ranges = self.aux_segments = None
        self.mid_o = torch.empty((max_vnode_to_q_entries, num_qo_heads, head_dim), dtype=torch.float32, device=device)
        self.mid_lse = torch.empty((max_vnode_to_q_entries, num_qo_heads), dtype=torch.float32, device=device)

        self.phase_node_nums: Tuple[int, int] = None
        self.phase_node_offsets: Tuple[int, int] = None
        self.phase_q_tile_sizes: Tuple[int, int] = None
        self.phase_kv_tile_sizes: Tuple[int, int] = None
        self.req_last_vnodes: List[int] = None
        self.num_vnodes = 0
        self.num_partial_rows = 0
        self.num_grouped_tails = 0      # tails of the current plan that are members of a group
        self.steps_since_plan = 0
        self.refresh_pending = False    # the newest row id of every grouped tail is copied by the step's first attention call
        self.refresh_layer = None       # graph-safe mode: the layer whose attention call makes that copy
