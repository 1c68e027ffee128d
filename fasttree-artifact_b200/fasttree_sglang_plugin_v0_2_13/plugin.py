"""Monkey-patch layer for SGLang v0.2.13 (reference:
fasttree_sglang_plugin_v0_2_13/plugin.py:9-238).

``load_fasttree_plugin`` wraps ``ModelTpServer.__init__`` so that, inside every
TP worker process, (1) ``forward_step`` plans one FastTree schedule per burst of
decode steps and patches it between steps, (2) ``InputMetadata`` carries the
schedule to the attention layers and (3) ``RadixAttention.decode_forward`` runs
the tree-attention kernels.  SGLang is imported lazily inside the patch
functions, as in the reference, so importing this module needs no SGLang.

Differences from the reference: the per-worker metadata is sized with the
worker's LOCAL head counts under tensor parallelism (the reference passes the
unsharded ones, plugin.py:221-226); the NVTX ranges come from
``torch.cuda.nvtx`` (the ``nvtx`` package is optional).
"""
from types import MethodType

import os

import torch

from ft_b200 import engine as _engine

from .attn_kernels import fasttree_decode
from .metadata import FastTreeMetadata


def _replace_radix_attn():
    from sglang.srt.layers.radix_attention import RadixAttention

    if getattr(RadixAttention, "_fasttree_patched", False):
        return
    original_init = RadixAttention.__init__

    def decode_forward_fasttree(self, q, k, v, input_metadata):
        if self.qk_head_dim != self.v_head_dim:
            o = q.new_empty((q.shape[0], self.tp_q_head_num * self.v_head_dim))
        else:
            o = torch.empty_like(q)
        self.store_kv_cache(k, v, input_metadata)       # the new token's K/V must be in the pool first
        md = input_metadata.fasttree
        if md.refresh_pending or (md.graph_safe and md.group_tails and md.refresh_layer == self.layer_id):
            # First attention call of a step: the newest token of every request has its KV-pool slot by now, and
            # the grouped tails take its row id into their table.  In graph-safe mode the layer that did this
            # first keeps doing it on every call (over the whole state table; unused entries are skipped), so a
            # captured step carries the copy whenever it was captured.
            _engine.refresh_tails(md.tail_state, md.max_batch_size if md.graph_safe else q.shape[0],
                                  input_metadata.req_to_token_pool.req_to_token, md.kv_entries_aux)
            md.refresh_pending = False
            if md.refresh_layer is None:
                md.refresh_layer = self.layer_id
        fasttree_decode(
            q.view(-1, self.tp_q_head_num, self.qk_head_dim),
            input_metadata.token_to_kv_pool.get_key_buffer(self.layer_id),
            input_metadata.token_to_kv_pool.get_value_buffer(self.layer_id),
            o.view(-1, self.tp_q_head_num, self.v_head_dim),
            input_metadata.req_to_token_pool.req_to_token,
            md.vnode_to_kv_offs, md.vnode_to_kv_lens,
            md.vnode_to_q_entries, md.vnode_to_q_offs, md.vnode_to_q_lens,
            md.req_to_vnode_entries, md.req_to_vnode_offs, md.req_to_vnode_lens,
            md.mid_o, md.mid_lse,
            md.phase_node_nums, md.phase_node_offsets, md.phase_q_tile_sizes, md.phase_kv_tile_sizes,
            sm_scale=self.scaling, logit_cap=self.logit_cap,
            phase_info=md.phase_info_dev if md.graph_safe else None,
            row_ranges=md.vnode_q_kv_ranges if md.group_tails else None,
            kv_entries_aux=md.kv_entries_aux if md.group_tails else None,
        )
        return o

    def patched_init(self, *args, **kwargs):
        original_init(self, *args, **kwargs)
        self.decode_forward = MethodType(decode_forward_fasttree, self)

    RadixAttention.__init__ = patched_init
    RadixAttention._fasttree_patched = True


def _annotate(module, func_name):
    original = getattr(module, func_name)

    def wrapped(*args, **kwargs):
        torch.cuda.synchronize()
        torch.cuda.nvtx.range_push(func_name)
        try:
            return original(*args, **kwargs)
        finally:
            torch.cuda.synchronize()
            torch.cuda.nvtx.range_pop()

    setattr(module, func_name, wrapped)


def _replace_tp_server_fwd(enable_fasttree=True, annotate_breakdown=False):
    from sglang.srt.managers.tp_worker import ModelTpServer, global_config
    from . import schedule as fasttree_schedule

    if annotate_breakdown:
        _annotate(ModelTpServer, "forward_prefill_batch")
        _annotate(ModelTpServer, "forward_decode_batch")
        if enable_fasttree:
            _annotate(fasttree_schedule, "prepare_for_fasttree_meta")
            _annotate(fasttree_schedule, "prepare_for_fasttree_step")

    @torch.inference_mode()
    def forward_step(self):
        new_batch = self.get_new_prefill_batch()
        if new_batch is not None:
            self.forward_prefill_batch(new_batch)
            if not new_batch.is_empty():
                if self.running_batch is None:
                    self.running_batch = new_batch
                else:
                    self.running_batch.merge(new_batch)
            return
        if self.running_batch is None:
            self.check_memory()
            self.new_token_ratio = global_config.init_new_token_ratio
            return
        # one schedule per burst of decode steps, patched in place between the steps
        burst = global_config.num_continue_decode_steps
        if enable_fasttree:
            # grouped tails reserve room for the tokens of this burst: never less than its number of steps
            md = self.fasttree_metadata
            md.tail_room = max(getattr(md, "tail_room", 0), burst)
            fasttree_schedule.prepare_for_fasttree_meta(self.running_batch, self.fasttree_metadata)
            planned_for = len(self.running_batch.reqs)
        for step in range(burst):
            self.num_generated_tokens += len(self.running_batch.reqs)
            self.forward_decode_batch(self.running_batch)
            if enable_fasttree:
                if len(self.running_batch.reqs) < planned_for:
                    break                                   # a request finished: the schedule is stale
                if step < burst - 1:
                    fasttree_schedule.prepare_for_fasttree_step(self.running_batch, self.fasttree_metadata)
            if self.tp_rank == 0 and self.decode_forward_ct % 40 == 0:
                self.print_decode_stats()
            if self.running_batch.is_empty():
                self.running_batch = None
                break
            if self.out_pyobjs and self.running_batch.has_stream():
                break

    ModelTpServer.forward_step = forward_step


def _replace_fwd_batch_info():
    from sglang.srt.model_executor.forward_batch_info import InputMetadata

    if getattr(InputMetadata, "_fasttree_patched", False):
        return
    original = InputMetadata.from_schedule_batch.__func__

    def from_schedule_batch(cls, model_runner, batch, forward_mode):
        ret = original(cls, model_runner, batch, forward_mode)
        ret.fasttree = getattr(batch, "fasttree_metadata", None)
        return ret

    InputMetadata.from_schedule_batch = classmethod(from_schedule_batch)
    InputMetadata._fasttree_patched = True


def _delayed_load_fasttree_plugin(enable_fasttree=True, annotate_breakdown=False):
    _replace_tp_server_fwd(enable_fasttree, annotate_breakdown)
    if enable_fasttree:
        _replace_fwd_batch_info()
        _replace_radix_attn()


def _load_plugin_and_replace_tp_server_init(enable_fasttree=True, annotate_breakdown=False):
    from sglang.srt.managers.tp_worker import ModelTpServer

    original_init = ModelTpServer.__init__

    def patched_init(self, gpu_id, tp_rank, server_args, nccl_port, model_overide_args):
        # patch inside the worker process, after it exists (CUDA must not be touched before the fork/spawn)
        _delayed_load_fasttree_plugin(enable_fasttree, annotate_breakdown)
        # The reference switches CUDA graphs off because its grids depend on the schedule, which changes every
        # burst (plugin.py:209-211).  With FASTTREE_GRAPH_SAFE=1 the decode call takes its phase split from device
        # memory and runs one plan-independent persistent grid, so the host's graph setting is left alone.
        graph_safe = os.environ.get("FASTTREE_GRAPH_SAFE", "0") == "1"
        if enable_fasttree and not graph_safe:
            server_args.disable_cuda_graph = True
        original_init(self, gpu_id, tp_rank, server_args, nccl_port, model_overide_args)
        if enable_fasttree:
            cfg = self.model_config
            tp = max(1, int(getattr(server_args, "tp_size", 1) or 1))
            self.fasttree_metadata = FastTreeMetadata(
                max(1, cfg.num_attention_heads // tp), max(1, cfg.num_key_value_heads // tp), cfg.head_dim,
                torch.device("cuda", self.gpu_id), graph_safe=graph_safe)

    ModelTpServer.__init__ = patched_init


def load_fasttree_plugin(enable_fasttree=True, annotate_breakdown=False):
    if not enable_fasttree and not annotate_breakdown:
        print("[Warning] FastTree plugin is not enabled")
        return
    _load_plugin_and_replace_tp_server_init(enable_fasttree, annotate_breakdown)
