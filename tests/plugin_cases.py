"""Stand-in decode batches shared by the plugin golden generator and the plugin tests."""
import torch

import sglang_standin
from oracle import ref_inputs

CASES = {
    # name: level sizes, level lens, generated tokens per request (cycled), hq, hkv
    "small_g4": ([1, 4], [40, 12], [3, 0, 5, 1], 8, 2),
    "three_level": ([1, 3, 9], [100, 30, 7], [0, 2, 9, 4, 1], 32, 8),
    "wide_mha": ([1, 40], [300, 20], [1, 0, 6], 32, 32),
    "long_tail": ([1, 4, 64], [2000, 300, 40], [5, 1100, 0, 17], 32, 8),
}


def build(name, device="cpu", dtype=torch.float16, extra_prompt=0, head_dim=128, steps=1):
    sizes, lens, gen, hq, hkv = CASES[name]
    nodes = ref_inputs.layered_tree(sizes, lens)
    batch_size = sum(1 for n in nodes if n.num_children == 0)
    generated = [gen[i % len(gen)] for i in range(batch_size)]
    total = sum(n.seqlen for n in nodes) + sum(g + steps + extra_prompt for g in generated)
    batch, rows = sglang_standin.build_batch(nodes, extra_prompt, generated, total + 64, hkv, head_dim, dtype,
                                             device, seed=len(name) * 7, steps=steps)
    return batch, rows, hq, hkv
