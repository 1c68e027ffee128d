"""B200-native tree-attention decode engine behind the FastTree artifact's entry points.

Sub-modules:
  build    nvcc recipe for libfasttree_b200.so (sm_100a)
  lib      ctypes binding of the C ABI (include/fasttree_b200.h)
  engine   torch-tensor glue for ft_decode / ft_stage1 / ft_stage2
  planner  tree -> vnode tables (reference-compatible and B200 splitters)
"""
from .lib import FastTreeError  # noqa: F401
