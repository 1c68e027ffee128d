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
