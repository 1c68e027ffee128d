"""The micro-benchmark driver with the reference's command line runs end to end
on a GPU and prints the line the reference's result scraper looks for."""
import os
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KB = os.path.join(ROOT, "fasttree-artifact_b200", "kernel_bench")


@pytest.mark.parametrize("planner", ["b200", "reference"])
def test_benchmark_cli(tmp_path, planner):
    tree = tmp_path / "tree.txt"
    subprocess.run([sys.executable, os.path.join(KB, "tree_generation.py"), "-n", "1,4,16", "-l", "256,64,32",
                    "-o", str(tree)], check=True)
    plan_file = tmp_path / "plan.txt"
    res = subprocess.run(
        [sys.executable, os.path.join(KB, "benchmark.py"), "--load_file_path", str(tree), "--num_qo_heads", "32",
         "--num_kv_heads", "8", "--q_tile_size_per_phase", "16,4", "--choice", "fasttree", "--planner", planner,
         "--fasttree_heuristic_path", str(plan_file)],
        cwd=KB, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    m = re.search(r"fasttree attn time: ([0-9.eE+-]+)", res.stdout)
    assert m and 0 < float(m.group(1)) < 100
    assert plan_file.read_text().startswith("Node 0: parent -1, assignment")


def test_benchmark_cli_with_the_optional_baselines(tmp_path):
    """--choice all: flash-attn on the padded cache, FlashInfer paged decode and FlashInfer's multi-level cascade
    over the tree rows run beside the engine; whichever of them is available must agree with it under the
    reference's allclose check (kernel_bench/benchmark.py:216-220)."""
    tree = tmp_path / "tree.txt"
    subprocess.run([sys.executable, os.path.join(KB, "tree_generation.py"), "-n", "1,4,16", "-l", "256,64,32",
                    "-o", str(tree)], check=True)
    cmd = [sys.executable, os.path.join(KB, "benchmark.py"), "--load_file_path", str(tree), "--num_qo_heads", "32",
           "--num_kv_heads", "8", "--q_tile_size_per_phase", "16,4", "--choice", "all"]
    deft = os.path.join(ROOT, "oracle", "_ref", "kernel_bench", "DeFT.py")     # staged from a reference checkout, if any
    if os.path.isfile(deft):
        cmd += ["--deft_module", deft]
    res = subprocess.run(cmd, cwd=KB, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stderr[-2000:]
    assert "Check failed" not in res.stdout, res.stdout
    assert "fasttree attn time:" in res.stdout
    for name, verdict in (("DeFT attn time:", "fasttree vs DeFT Check passed!"),
                          ("flashinfer cascade time:", "fasttree vs cascade Check passed!"),
                          ("sglang flashinfer time:", "fasttree vs flashinfer Check passed!"),
                          ("flash attn time:", "fasttree attn Check passed!")):
        if name in res.stdout:
            assert verdict in res.stdout, res.stdout
