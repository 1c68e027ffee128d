"""A stand-in for the slice of SGLang v0.2.13 that the FastTree plugin touches.

SGLang is not installed here, and its source is not reproduced: these classes
expose only the attributes and call signatures the plugin reads (listed in the
reference at fasttree_sglang_plugin_v0_2_13/plugin.py:10-51,67-152,158-226 and
schedule.py:6-35,79-85,156-157) with the simplest behaviour that satisfies
them.  ``install()`` registers them under the ``sglang.*`` module names the
plugin imports.

Conventions of the stand-in (the plugin's arithmetic is self-consistent under
them): a request holds ``origin_input_ids`` (P prompt tokens) and ``output_ids``
(n generated tokens); when a decode burst is planned the KV pool holds positions
0 .. P+n-1 of every request and the decode step writes position P+n.  The radix
cache holds prompt prefixes only; ``req_to_token[pool_idx, pos]`` gives the KV
pool slot of every position.
"""
import sys
import types

import torch


class TreeNode:
    def __init__(self):
        self.children = {}        # first token -> TreeNode
        self.parent = None
        self.key = []             # token ids of this edge
        self.value = None         # int32 tensor: KV pool slot per token


class RadixCache:
    """Prefix tree over token-id sequences; ``insert`` splits edges as needed."""

    def __init__(self):
        self.root_node = TreeNode()
        self.root_node.value = torch.zeros(0, dtype=torch.int32)

    def insert(self, tokens, slots):
        tokens = list(tokens)
        node, pos = self.root_node, 0
        while pos < len(tokens):
            child = node.children.get(tokens[pos])
            if child is None:
                new = TreeNode()
                new.parent, new.key, new.value = node, tokens[pos:], slots[pos:].clone()
                node.children[tokens[pos]] = new
                return
            common = 0
            while common < len(child.key) and pos + common < len(tokens) and child.key[common] == tokens[pos + common]:
                common += 1
            if common < len(child.key):               # split the edge
                upper = TreeNode()
                upper.parent, upper.key, upper.value = node, child.key[:common], child.value[:common].clone()
                child.key, child.value, child.parent = child.key[common:], child.value[common:].clone(), upper
                upper.children[child.key[0]] = child
                node.children[tokens[pos]] = upper
                child = upper
            node, pos = child, pos + common


class Req:
    def __init__(self, origin_input_ids, output_ids):
        self.origin_input_ids = list(origin_input_ids)
        self.output_ids = list(output_ids)


class ReqToTokenPool:
    def __init__(self, size, max_context_len, device):
        self.req_to_token = torch.zeros(size, max_context_len, dtype=torch.int32, device=device)


class TokenToKVPool:
    def __init__(self, size, num_layers, num_kv_heads, head_dim, dtype, device):
        self.k_buffer = [torch.zeros(size, num_kv_heads, head_dim, dtype=dtype, device=device)
                         for _ in range(num_layers)]
        self.v_buffer = [torch.zeros(size, num_kv_heads, head_dim, dtype=dtype, device=device)
                         for _ in range(num_layers)]

    def get_key_buffer(self, layer_id):
        return self.k_buffer[layer_id]

    def get_value_buffer(self, layer_id):
        return self.v_buffer[layer_id]


class ScheduleBatch:
    def __init__(self, reqs, tree_cache, req_pool_indices, req_to_token_pool, token_to_kv_pool=None):
        self.reqs = reqs
        self.tree_cache = tree_cache
        self.req_pool_indices = req_pool_indices
        self.req_to_token_pool = req_to_token_pool
        self.token_to_kv_pool = token_to_kv_pool
        self.out_cache_loc = None           # slots the current decode step writes, one per request

    def is_empty(self):
        return len(self.reqs) == 0

    def has_stream(self):
        return False

    def merge(self, other):
        self.reqs.extend(other.reqs)


class ForwardMode:
    DECODE = "decode"


class InputMetadata:
    def __init__(self, batch):
        self.token_to_kv_pool = batch.token_to_kv_pool
        self.req_to_token_pool = batch.req_to_token_pool
        self.out_cache_loc = batch.out_cache_loc

    @classmethod
    def from_schedule_batch(cls, model_runner, batch, forward_mode):
        return cls(batch)


class ModelRunner:
    pass


class RadixAttention:
    def __init__(self, num_heads, head_dim, scaling, num_kv_heads, layer_id, logit_cap=-1):
        self.tp_q_head_num = num_heads
        self.tp_k_head_num = num_kv_heads
        self.qk_head_dim = head_dim
        self.v_head_dim = head_dim
        self.scaling = scaling
        self.layer_id = layer_id
        self.logit_cap = logit_cap
        self.decode_forward = None

    def store_kv_cache(self, cache_k, cache_v, input_metadata):
        pool = input_metadata.token_to_kv_pool
        loc = input_metadata.out_cache_loc.long()
        pool.get_key_buffer(self.layer_id)[loc] = cache_k.view(-1, self.tp_k_head_num, self.qk_head_dim)
        pool.get_value_buffer(self.layer_id)[loc] = cache_v.view(-1, self.tp_k_head_num, self.v_head_dim)


class _GlobalConfig:
    num_continue_decode_steps = 4
    init_new_token_ratio = 0.7


global_config = _GlobalConfig()


class ServerArgs:
    def __init__(self):
        self.disable_cuda_graph = False


class _ModelConfig:
    def __init__(self, num_attention_heads, num_key_value_heads, head_dim):
        self.num_attention_heads = num_attention_heads
        self.num_key_value_heads = num_key_value_heads
        self.head_dim = head_dim


class ModelTpServer:
    """Only what the patched ``__init__`` / ``forward_step`` use.  ``decode_fn(batch)``
    stands for the model forward + sampling of one decode step."""

    def __init__(self, gpu_id, tp_rank, server_args, nccl_port, model_overide_args):
        self.gpu_id = gpu_id
        self.tp_rank = tp_rank
        self.server_args = server_args
        cfg = model_overide_args or {}
        self.model_config = _ModelConfig(cfg.get("num_attention_heads", 8), cfg.get("num_key_value_heads", 2),
                                         cfg.get("head_dim", 128))
        self.running_batch = None
        self.num_generated_tokens = 0
        self.decode_forward_ct = 0
        self.out_pyobjs = []
        self.new_token_ratio = 0.0
        self.decode_fn = cfg.get("decode_fn")
        self.prefill_queue = []
        self.memory_checks = 0

    def get_new_prefill_batch(self):
        return self.prefill_queue.pop(0) if self.prefill_queue else None

    def forward_prefill_batch(self, batch):
        pass

    def forward_decode_batch(self, batch):
        self.decode_forward_ct += 1
        if self.decode_fn is not None:
            self.decode_fn(batch)

    def print_decode_stats(self):
        pass

    def check_memory(self):
        self.memory_checks += 1

    def forward_step(self):
        raise NotImplementedError("replaced by the plugin")


def install():
    """Register the stand-in under the module names the plugin imports."""
    def mod(name, **attrs):
        m = sys.modules.get(name) or types.ModuleType(name)
        for k, v in attrs.items():
            setattr(m, k, v)
        sys.modules[name] = m
        return m

    mod("sglang")
    mod("sglang.srt")
    mod("sglang.srt.mem_cache")
    mod("sglang.srt.mem_cache.radix_cache", RadixCache=RadixCache, TreeNode=TreeNode)
    mod("sglang.srt.managers")
    mod("sglang.srt.managers.schedule_batch", ScheduleBatch=ScheduleBatch)
    mod("sglang.srt.managers.tp_worker", ModelTpServer=ModelTpServer, global_config=global_config,
        ServerArgs=ServerArgs)
    mod("sglang.srt.layers")
    mod("sglang.srt.layers.radix_attention", RadixAttention=RadixAttention)
    mod("sglang.srt.model_executor")
    mod("sglang.srt.model_executor.forward_batch_info", InputMetadata=InputMetadata, ForwardMode=ForwardMode)
    mod("sglang.srt.model_executor.model_runner", ModelRunner=ModelRunner)


def build_batch(tree_nodes, extra_prompt, generated, pool_size, num_kv_heads, head_dim, dtype, device, seed,
                num_layers=1, max_context_len=None, steps=1, slot_layout="scattered"):
    """A decode batch whose prompts share prefixes the way ``tree_nodes`` (a list of
    oracle/product tree nodes: parent, seqlen, num_children) does.  Each leaf is one
    request: prompt = tokens of its root->leaf path + ``extra_prompt`` private tokens
    that are NOT in the radix cache; ``generated[r]`` tokens already generated;
    pool slots are reserved for ``steps`` decode steps.
    ``slot_layout``: "scattered" - KV pool slots are a random permutation, the hardest case for the kernels'
    loaders (every row is fetched on its own); "prefill" - what a serving process produces: the tokens of a
    radix node and of a private prompt tail sit in consecutive slots (one prefill wrote them), generated tokens
    are interleaved across the requests (every decode step allocates one slot per request).
    Returns (batch, token lists per request)."""
    g = torch.Generator().manual_seed(seed)
    node_tokens, next_tok = [], 1000
    for nd in tree_nodes:
        node_tokens.append(list(range(next_tok, next_tok + nd.seqlen)))   # distinct ids -> distinct first tokens
        next_tok += nd.seqlen
    paths = []
    for nd in tree_nodes:
        if nd.num_children == 0:
            chain, cur = [], nd.id
            while cur != -1:
                chain.append(cur)
                cur = tree_nodes[cur].parent
            paths.append(chain[::-1])
    if slot_layout == "scattered":
        perm = torch.randperm(pool_size, generator=g).to(torch.int32)
    elif slot_layout == "prefill":
        perm = torch.arange(pool_size, dtype=torch.int32)
    else:
        raise ValueError("slot_layout must be 'scattered' or 'prefill'")
    used = 0
    node_slots = []
    for nd in tree_nodes:
        node_slots.append(perm[used:used + nd.seqlen])
        used += nd.seqlen
    cache = RadixCache()
    reqs, rows = [], []
    prompt_tail = []
    if slot_layout == "prefill":        # private prompt tails first, then one slot per request and decode step
        for r in range(len(paths)):
            prompt_tail.append(perm[used:used + extra_prompt])
            used += extra_prompt
        # step-major numbering: step i hands one slot to every request that still decodes at step i
        decode_slots_of = [[] for _ in paths]
        for i in range(max(generated, default=0) + steps):
            for r in range(len(paths)):
                if i < generated[r] + steps:
                    decode_slots_of[r].append(used)
                    used += 1
    for r, chain in enumerate(paths):
        shared = [t for n in chain for t in node_tokens[n]]
        shared_slots = torch.cat([node_slots[n] for n in chain]) if chain else perm[:0]
        cache.insert(shared, shared_slots)
        n_priv = extra_prompt + generated[r] + steps       # private prompt tail + generated + the tokens being decoded
        if slot_layout == "prefill":
            priv_slots = torch.cat([prompt_tail[r], perm[torch.tensor(decode_slots_of[r], dtype=torch.long)]])
        else:
            priv_slots = perm[used:used + n_priv]
            used += n_priv
        prompt = shared + list(range(next_tok, next_tok + extra_prompt))
        next_tok += extra_prompt
        outs = list(range(next_tok, next_tok + generated[r]))
        next_tok += generated[r]
        reqs.append(Req(prompt, outs))
        rows.append(torch.cat([shared_slots, priv_slots]))
    assert used <= pool_size, "KV pool too small for the stand-in batch"
    width = max_context_len or max(len(row) for row in rows) + 8
    r2t = ReqToTokenPool(len(reqs) + 3, width, device)
    pool_idx = torch.randperm(len(reqs) + 3, generator=g)[:len(reqs)].to(torch.int32)
    host = torch.zeros(len(reqs) + 3, width, dtype=torch.int32)
    for r, row in enumerate(rows):
        host[pool_idx[r], :len(row)] = row
    r2t.req_to_token.copy_(host)
    kv = TokenToKVPool(pool_size, num_layers, num_kv_heads, head_dim, dtype, device)
    for layer in range(num_layers):
        kv.k_buffer[layer].copy_(torch.randn(pool_size, num_kv_heads, head_dim, generator=g).to(dtype))
        kv.v_buffer[layer].copy_(torch.randn(pool_size, num_kv_heads, head_dim, generator=g).to(dtype))
    batch = ScheduleBatch(reqs, cache, pool_idx.to(device), r2t, kv)
    # slots written by the coming decode step: position P + n of each request
    batch.out_cache_loc = torch.stack([rows[r][len(reqs[r].origin_input_ids) + generated[r]]
                                       for r in range(len(reqs))]).to(device)
    return batch, rows
