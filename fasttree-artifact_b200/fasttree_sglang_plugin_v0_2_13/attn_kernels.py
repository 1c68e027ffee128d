"""``fasttree_decode`` of the plugin (reference:
fasttree_sglang_plugin_v0_2_13/attn_kernels.py:288-348): same signature, routed to
the sm_100a kernels through the C ABI.  ``vnode_to_kv_entries`` is SGLang's 2-D
``req_to_token`` table and ``vnode_to_kv_offs`` are flat offsets into it.  Per-row
token ranges and the auxiliary row-id table of grouped private tails
(``FastTreeMetadata.group_tails``) arrive as explicit keyword arguments; without
them the call says outright that the plan carries no ranges (no look-up behind
``vnode_to_q_entries``)."""
from ft_b200 import engine as _engine


def fasttree_decode(q, k_buffer, v_buffer, o, vnode_to_kv_entries, vnode_to_kv_offs, vnode_to_kv_lens,
                    vnode_to_q_entries, vnode_to_q_offs, vnode_to_q_lens, req_to_vnode_entries,
                    req_to_vnode_offs, req_to_vnode_lens, mid_o, mid_lse, phase_node_nums, phase_node_offsets,
                    phase_q_tile_sizes, phase_kv_tile_sizes, sm_scale, logit_cap=-1, phase_info=None,
                    row_ranges=None, kv_entries_aux=None):
    """Beyond the reference's signature: ``phase_info``, a device copy of the phase split (see
    ``FastTreeMetadata.graph_safe``); ``row_ranges`` / ``kv_entries_aux``, the per-row token ranges and the
    second row-id table of a plan with grouped tails."""
    _engine.decode(q, k_buffer, v_buffer, o, vnode_to_kv_entries, vnode_to_kv_offs, vnode_to_kv_lens,
                   vnode_to_q_entries, vnode_to_q_offs, vnode_to_q_lens, req_to_vnode_entries,
                   req_to_vnode_offs, req_to_vnode_lens, mid_o, mid_lse, phase_node_nums, phase_node_offsets,
                   phase_q_tile_sizes, phase_kv_tile_sizes, sm_scale, logit_cap=logit_cap, row_ranges=row_ranges, phase_info=phase_info,
                   kv_entries_aux=kv_entries_aux)
