"""Tree model and tree-file reader of the micro-benchmark.

Same public surface as the reference module (kernel_bench/kv_tree_simple.py:4-10
node record, :50-64 reader): a node has ``parent`` (-1 for the root), ``id``,
``seqlen``, ``num_children`` and ``requests`` (ids of all requests whose path
contains the node).  Nodes are listed by id, node 0 is the root and parents
precede their children.
"""


class KVTreeNode:
    __slots__ = ("parent", "id", "seqlen", "num_children", "requests")

    def __init__(self, parent=-1, id=-1, seqlen=0, num_children=0):
        self.parent = parent
        self.id = id
        self.seqlen = seqlen
        self.num_children = num_children
        self.requests = []

    def __repr__(self):
        return (f"KVTreeNode(parent={self.parent}, id={self.id}, seqlen={self.seqlen}, "
                f"num_children={self.num_children}, requests={len(self.requests)})")


def retrive_from_file(filepath):
    """Read ``<n>`` then n lines ``parent id seqlen out_degree``.  (The name keeps
    the reference's spelling.)  Raises ValueError on a malformed file."""
    with open(filepath, "r", encoding="utf-8") as fh:
        tokens = fh.read().split()
    if not tokens:
        raise ValueError(f"{filepath}: empty tree file")
    count = int(tokens[0])
    if len(tokens) < 1 + 4 * count:
        raise ValueError(f"{filepath}: expected {count} node lines")
    nodes = []
    for i in range(count):
        par, nid, slen, deg = (int(t) for t in tokens[1 + 4 * i: 5 + 4 * i])
        nodes.append(KVTreeNode(par, nid, slen, deg))
    return nodes


def tree_from_rows(rows):
    """Nodes from ``[parent, id, seqlen, out_degree]`` rows (what tree_generation.generate_tree returns and
    what a tree file holds)."""
    return [KVTreeNode(int(p), int(i), int(s), int(d)) for p, i, s, d in rows]


def assign_requests(nodes):
    """Leaves, in id order, get request ids 0, 1, 2, ...; each id is recorded on the leaf and on all its
    ancestors (what the reference does while drawing the inputs, kernel_bench/flash_attn_wrap.py:24-33).
    Returns ``(batch_size, KV_ptrs)`` where node i owns rows ``[KV_ptrs[i], KV_ptrs[i+1])`` of the flat tree
    tensors (:13,22)."""
    for nd in nodes:
        nd.requests = []
    batch, ptrs = 0, [0]
    for nd in nodes:
        ptrs.append(ptrs[-1] + nd.seqlen)
        if nd.num_children == 0:
            cur = nd.id
            while cur != -1:
                nodes[cur].requests.append(batch)
                cur = nodes[cur].parent
            batch += 1
    return batch, ptrs


def validate_tree(nodes):
    """Checks the invariants the planner relies on; raises ValueError."""
    deg = [0] * len(nodes)
    for i, nd in enumerate(nodes):
        if nd.id != i:
            raise ValueError(f"node {i} carries id {nd.id}; nodes must be listed by id")
        if i == 0:
            if nd.parent != -1:
                raise ValueError("node 0 must be the root (parent -1)")
        else:
            if not 0 <= nd.parent < i:
                raise ValueError(f"node {i}: parent {nd.parent} must precede it")
            deg[nd.parent] += 1
        if nd.seqlen < 0:
            raise ValueError(f"node {i}: negative seqlen")
    for i, nd in enumerate(nodes):
        if deg[i] != nd.num_children:
            raise ValueError(f"node {i}: num_children {nd.num_children} but {deg[i]} nodes name it as parent")
