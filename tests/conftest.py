import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def make_linear(k, n, K, seed, m=1):
    """Seeded synthetic EXL3 linear: uniform random trellis words (every bit pattern is a valid
    stream), +-1 sign vectors, N(0,1) activations."""
    rng = np.random.default_rng(seed)
    trellis = rng.integers(0, 65536, size=(k // 16, n // 16, int(round(16 * K))), dtype=np.uint16)      # K may be 1.5 / 2.5 / 3.5
    suh = rng.choice(np.array([-1.0, 1.0], np.float16), size=k)
    svh = rng.choice(np.array([-1.0, 1.0], np.float16), size=n)
    x = rng.standard_normal((m, k)).astype(np.float16)
    return trellis, suh, svh, x


@pytest.fixture(scope="session")
def oracle():
    from oracle import exl3_oracle
    exl3_oracle.lib()
    return exl3_oracle


@pytest.fixture(autouse=True)
def _fp16_mul1_gemv_by_default():
    """The one-row GEMV of mul1 tensors takes the int8-activation form by default (as the
    reference). The parity tests compare the fp16 kernels against the fp32-accumulated oracle, so
    the switch is off unless a test turns it on (the int8 tests do, and compare against the int8
    restatement)."""
    try:
        from ampstein_b200 import _lib
        L = _lib.lib()
    except Exception:
        yield
        return
    old = L.amp_exl3_set_int8_gemv(0, 0)
    yield
    L.amp_exl3_set_int8_gemv(old, 0)
