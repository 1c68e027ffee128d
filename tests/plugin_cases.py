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

# The four traffic shapes of the reference's serving benchmarks, as tree shapes only (synthetic token counts,
# no dataset content): shared system prompts with many questions each
# (sglang_bench/benchmarks/bench_multi_level_system.py:28-49), few-shot branches
# (bench_multi_few_shot.py:47-60), questions forked into reasoning chains
# (bench_multi_chain_reasoning.py:45-77), documents with several questions each
# (bench_multi_document.py:40-59).  Llama-3-8B head counts; not part of the reference-table goldens.
TRAFFIC_SHAPES = {
    "system_4x128": ([1, 4, 512], [24, 420, 36], [2, 0, 7, 1], 32, 8),
    "few_shot_8x16": ([1, 8, 128], [30, 900, 48], [0, 3, 1], 32, 8),
    "chains_32x4": ([1, 32, 128], [150, 60, 90], [5, 0, 11, 2], 32, 8),
    "documents_16x8": ([1, 16, 128], [12, 1500, 25], [1, 4, 0], 32, 8),
}


def build(name, device="cpu", dtype=torch.float16, extra_prompt=0, head_dim=128, steps=1, slot_layout="scattered"):
    sizes, lens, gen, hq, hkv = (CASES.get(name) or TRAFFIC_SHAPES[name])
    nodes = ref_inputs.layered_tree(sizes, lens)
    batch_size = sum(1 for n in nodes if n.num_children == 0)
    generated = [gen[i % len(gen)] for i in range(batch_size)]
    total = sum(n.seqlen for n in nodes) + sum(g + steps + extra_prompt for g in generated)
    batch, rows = sglang_standin.build_batch(nodes, extra_prompt, generated, total + 64, hkv, head_dim, dtype,
                                             device, seed=len(name) * 7, steps=steps, slot_layout=slot_layout)
    return batch, rows, hq, hkv
