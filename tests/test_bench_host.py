"""Host-side logic of bench.py that needs no GPU: the tensor-parallel shard shapes of both
stacks and the algorithmic byte counts."""
import importlib.util
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
spec = importlib.util.spec_from_file_location("bench", os.path.join(ROOT, "bench.py"))
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)


@pytest.mark.parametrize("stack", ["decode", "tp5"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_shapes_partition_the_stack(stack, world):
    S = bench.STACKS[stack]
    full = {name: (k, n) for name, k, n, _ in bench.layer_linears(S)}
    got = [bench.layer_linears(S, r, world) for r in range(world)]
    for name, (k, n) in full.items():
        parts = [[s for s in layer if s[0] == name][0] for layer in got]
        if name in ("o", "down"):              # row-parallel: rows split, columns whole
            assert sum(p[1] for p in parts) == k and all(p[2] == n and p[3] == k for p in parts)
        else:                                  # column-parallel
            assert sum(p[2] for p in parts) == n and all(p[1] == k for p in parts)
        assert all(p[1] % 128 == 0 and p[2] % 128 == 0 for p in parts)
    for layer in got:                          # a rank's gate/up columns are its down rows
        d = {s[0]: s for s in layer}
        assert d["gate"][2] == d["up"][2] == d["down"][1] and d["q"][2] == d["o"][1]
    if S["vocab"]:
        heads = [bench.head_shape(S, r, world) for r in range(world)]
        assert sum(h[1] for h in heads) == S["vocab"] and all(h[1] % 128 == 0 for h in heads)
    else:
        assert bench.head_shape(S) is None


def test_tp5_mlp_shards_follow_the_largest_remainder_rule():
    S = bench.STACKS["tp5"]
    widths = [dict((s[0], s) for s in bench.layer_linears(S, r, 8))["gate"][2] for r in range(8)]
    assert widths == [3328] * 4 + [3072] * 4


def test_algorithmic_bytes_of_the_steps():
    # 32 x 7 linears at 4 bpw + lm_head at 6 bpw, with suh/svh and the batch-1 activations
    assert bench.algorithmic_bytes(bench.STACKS["decode"], 1) == 3894678528
    # 64 layers at 5 bpw: 291.5 M weights per layer
    S = bench.STACKS["tp5"]
    per_layer = sum(k * n for _, k, n, _ in bench.layer_linears(S))
    assert per_layer == 5120 * (6144 + 2 * 1024) + 6144 * 5120 + 3 * 5120 * 25600
    assert abs(bench.algorithmic_bytes(S, 1) - 64 * per_layer * 5 / 8) < 64 * 1e6
    # sharded: the ranks' weight bytes add up to the whole
    tot = sum(bench.algorithmic_bytes(S, 1, r, 8) for r in range(8))
    assert abs(tot - bench.algorithmic_bytes(S, 1)) < 0.01 * tot


def _run_bench(*args):
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    return subprocess.run([sys.executable, os.path.join(root, "bench.py")] + list(args), capture_output=True, text=True, env=env, timeout=300)


def test_secondary_workloads_refuse_to_run_without_a_gpu_and_check_their_arguments():
    """No CPU path: every GPU workload stops with a message instead of computing on the host; bad
    shapes and token counts are rejected before any device work."""
    for wl in ("moe-prefill", "gemm", "gemv", "moe", "prefill"):
        r = _run_bench("--workload", wl)
        assert r.returncode != 0 and "no CUDA device" in (r.stderr + r.stdout), (wl, r.stderr[-300:])
    r = _run_bench("--workload", "moe", "--tokens", "3")
    assert r.returncode != 0 and "--tokens 1, 4 or 16" in r.stderr
    r = _run_bench("--workload", "bogus")
    assert r.returncode != 0
