"""Host-side logic of bench.py that needs no GPU: the tensor-parallel shard shapes and the
algorithmic byte count."""
import importlib.util
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
spec = importlib.util.spec_from_file_location("bench", os.path.join(ROOT, "bench.py"))
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_shapes_partition_the_stack(world):
    full = {name: (k, n) for name, k, n in bench.LAYER_LINEARS}
    got = [bench.tp_shapes(r, world) for r in range(world)]
    for name, (k, n) in full.items():
        parts = [[s for s in layer if s[0] == name][0] for layer, _ in got]
        if name in ("o", "down"):              # row-parallel: rows split, columns whole
            assert sum(p[1] for p in parts) == k and all(p[2] == n and p[3] == k for p in parts)
        else:                                  # column-parallel
            assert sum(p[2] for p in parts) == n and all(p[1] == k for p in parts)
        assert all(p[1] % 128 == 0 and p[2] % 128 == 0 for p in parts)
    assert sum(h[1] for _, h in got) == bench.VOCAB and all(h[1] % 128 == 0 for _, h in got)


def test_algorithmic_bytes_of_the_step():
    # 32 x 7 linears at 4 bpw + lm_head at 6 bpw, with suh/svh and the batch-1 activations
    assert bench.algorithmic_bytes(1) == 3894678528
    assert bench.total_weights() == 32 * 218103808 + 4096 * 128256
