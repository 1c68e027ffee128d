"""CPU oracle for the FastTree tree-attention decode path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; it is used by the test-suite, by the smoke check and by the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark as the checker
and as the timed CPU baseline.  It restates, in plain Python / numpy / CPU
torch, what the reference computes on this path:

* ``ref_inputs``    - tree construction, tree-file format, request assignment
                      and the synthetic Q/K/V draw order
                      (kernel_bench/tree_generation.py, kv_tree_simple.py,
                      flash_attn_wrap.py::qkv_preparation).
* ``ref_planner``   - the cost model, the greedy split heuristic and the
                      vnode-table emission (kernel_bench/fasttree.py:30-296).
* ``ref_attention`` - fp32 per-leaf path-concatenated attention (ground
                      truth), the stage-1 per-vnode partial attention and the
                      stage-2 log-sum-exp merge
                      (kernel_bench/fasttree.py:299-546).

Parity pin: the restatements are checked against fixtures produced by the
reference's own code (imported on CPU under the Triton interpreter) by
``tests/golden/make_golden.py``; the fixtures are committed under
``tests/golden``.
"""
