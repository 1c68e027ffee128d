"""Writes a layered tree file: ``-n`` nodes per level, ``-l`` context length per level.

Same CLI and file format as the reference tool (kernel_bench/tree_generation.py):
child j of a level with ``size`` nodes hangs under parent ``(j * prev) // size``
of the previous level (:59); the file is ``<n>`` followed by
``parent id seqlen out_degree`` per node (:78-94).
"""
import argparse


def generate_tree(layer_sizes, layer_lengths):
    """Returns ``[[parent, id, seqlen, out_degree], ...]`` in id order."""
    if len(layer_sizes) != len(layer_lengths):
        raise ValueError("The length of layer_sizes must be equal to the length of layer_lengths.")
    rows = []
    above = []
    for depth, (count, seqlen) in enumerate(zip(layer_sizes, layer_lengths)):
        first = len(rows)
        for j in range(count):
            parent = -1 if depth == 0 else above[(j * len(above)) // count]
            rows.append([parent, first + j, seqlen, 0])
            if parent >= 0:
                rows[parent][3] += 1
        above = list(range(first, first + count))
    return rows


def generate_random_tree(levels, seed, max_children=32, lam=3.0, len_lo=16, len_hi=2048):
    """Irregular tree with ``levels`` node-levels in the same row format (no counterpart in the reference, whose
    generator is layered only).  Nodes get breadth-first ids; for each node in that order a context length
    ~ Uniform{len_lo..len_hi} is drawn and, unless it sits on the last level, a child count
    ``min(max_children, 1 + Poisson(lam))``, from ``numpy.random.default_rng(seed)``."""
    import numpy as np
    rng = np.random.default_rng(seed)
    rows, depth = [[-1, 0, 0, 0]], [0]
    head = 0
    while head < len(rows):
        rows[head][2] = int(rng.integers(len_lo, len_hi + 1))
        if depth[head] < levels - 1:
            kids = int(min(max_children, 1 + rng.poisson(lam)))
            rows[head][3] = kids
            for _ in range(kids):
                rows.append([head, len(rows), 0, 0])
                depth.append(depth[head] + 1)
        head += 1
    return rows


def save_tree(nodes, output_path):
    with open(output_path, "w", encoding="utf-8") as fh:
        fh.write(f"{len(nodes)}\n")
        fh.writelines(f"{p} {i} {s} {d}\n" for p, i, s, d in nodes)


def _csv_ints(text):
    return [int(x) for x in text.split(",")]


def main(argv=None):
    ap = argparse.ArgumentParser(description="Generate a tree based on layer sizes and sequence lengths.")
    ap.add_argument("-n", "--layer_sizes", type=str, help="node count per level, e.g. 1,2,4")
    ap.add_argument("-l", "--layer_lengths", type=str, help="context length per level, e.g. 128,64,64")
    ap.add_argument("-o", "--output_file", type=str, required=True)
    ap.add_argument("--random_levels", type=int, default=0, help="write a seeded irregular tree of this many levels instead")
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    if args.random_levels > 0:
        save_tree(generate_random_tree(args.random_levels, args.seed), args.output_file)
        return
    if not args.layer_sizes or not args.layer_lengths:
        ap.error("-n/--layer_sizes and -l/--layer_lengths are required for a layered tree")
    save_tree(generate_tree(_csv_ints(args.layer_sizes), _csv_ints(args.layer_lengths)), args.output_file)


if __name__ == "__main__":
    main()
