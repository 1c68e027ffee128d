"""``fasttree_decode`` of the plugin (reference:
fasttree_sglang_plugin_v0_2_13/attn_kernels.py:288-348): same signature, routed to
the sm_100a kernels through the C ABI.  ``vnode_to_kv_entries`` is SGLang's 2-D
``req_to_token`` table and ``vnode_to_kv_offs`` are flat offsets into it.  The
serving schedule never groups short nodes, so the call says outright that the
plan carries no per-row token ranges (no look-up behind ``vnode_to_q_entries``)."""
from ft_b200 import engine as _engine


def fasttree_decode(q, k_buffer, v_buffer, o, vnode_to_kv_entries, vnode_to_kv_offs, vnode_to_kv_lens,
                    vnode_to_q_entries, vnode_to_q_offs, vnode_to_q_lens, req_to_vnode_entries,
                    req_to_vnode_offs, req_to_vnode_lens, mid_o, mid_lse, phase_node_nums, phase_node_offsets,
                    phase_q_tile_sizes, phase_kv_tile_sizes, sm_scale, logit_cap=-1, phase_info=None):
    """``phase_info`` (beyond the reference's signature): a device copy of the phase split, see
    ``FastTreeMetadata.graph_safe``."""
    _engine.decode(q, k_buffer, v_buffer, o, vnode_to_kv_entries, vnode_to_kv_offs, vnode_to_kv_lens,
                   vnode_to_q_entries, vnode_to_q_offs, vnode_to_q_lens, req_to_vnode_entries,
                   req_to_vnode_offs, req_to_vnode_lens, mid_o, mid_lse, phase_node_nums, phase_node_offsets,
                   phase_q_tile_sizes, phase_kv_tile_sizes, sm_scale, logit_cap=logit_cap, row_ranges=None, phase_info=phase_info)
