"""amp_exl3_gemv_static: the decode GEMV whose scratch is a fixed array inside the library (no
device allocation at any call). Runs last in the suite on purpose: it must work on a device whose
other workspaces already exist, and -- in a fresh process -- as the very first GEMV call, before
the allocating entry point has created its workspace."""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import make_linear

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def amp():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import ampstein_b200
    return ampstein_b200


def dev(a):
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run(name, xx, t, s, v, m, k, n, K):
    from ampstein_b200 import _lib
    out = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    _lib.call(name, xx.data_ptr(), t.data_ptr(), out.data_ptr(), s.data_ptr(), v.data_ptr(),
              m, k, n, K, 0, 0, torch.cuda.current_stream().cuda_stream)
    return out


def test_static_scratch_matches_allocating_entry_point_twice_in_a_row(amp, oracle):
    # every column block of these shapes is shared between CTAs, so the scratch array is used
    cases = [make_linear(4096, 512, 4, seed=9100, m=1), make_linear(2048, 1024, 5, seed=9101, m=4)]
    for trellis, suh, svh, x in cases:
        m, k = x.shape
        n, K = trellis.shape[1] * 16, trellis.shape[2] // 16
        t, s, v, xx = dev(trellis), dev(suh), dev(svh), dev(x)
        ref = run("amp_exl3_gemv", xx, t, s, v, m, k, n, K)
        first = run("amp_exl3_gemv_static", xx, t, s, v, m, k, n, K)
        second = run("amp_exl3_gemv_static", xx, t, s, v, m, k, n, K)
        torch.cuda.synchronize()
        # the two entry points may cut the rows into different ranges (different fp32 summation
        # order), so they agree to fp16 rounding; the same entry point twice agrees bit for bit
        assert torch.equal(first, second)
        scale = ref.float().abs().max()
        assert float((first.float() - ref.float()).abs().max() / scale) < 2e-3
        want = oracle.linear(x, trellis, suh, svh, 0, fp32_out=True)
        err = np.max(np.abs(first.float().cpu().numpy() - want)) / np.max(np.abs(want))
        assert err < 1e-2                  # max relative error against the fp32-accumulated oracle


def test_static_scratch_refuses_sizes_beyond_its_array(amp):
    from ampstein_b200 import _lib
    L = _lib.lib()
    trellis, suh, svh, x = make_linear(128, 128, 4, seed=9102, m=5)
    t, s, v, xx = dev(trellis), dev(suh), dev(svh), dev(x)
    out = torch.empty((5, 128), dtype=torch.float16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    rc = L.amp_exl3_gemv_static(xx.data_ptr(), t.data_ptr(), out.data_ptr(), s.data_ptr(), v.data_ptr(), 5, 128, 128, 4, 0, 0, st)
    assert rc < 0 and "m must be 1..4" in _lib.last_error()
    n_big = 128 * 1025                      # one column block more than the array holds
    rc = L.amp_exl3_gemv_static(xx.data_ptr(), t.data_ptr(), out.data_ptr(), s.data_ptr(), v.data_ptr(), 1, 128, n_big, 4, 0, 0, st)
    assert rc < 0 and "131072" in _lib.last_error()
    torch.cuda.synchronize()


def test_static_scratch_allocates_no_device_memory(amp):
    """Free device memory, as the driver reports it, is the same before and after a series of
    calls (the allocating entry point's first call, by contrast, takes its 64 MB workspace)."""
    trellis, suh, svh, x = make_linear(2048, 1024, 4, seed=9103, m=2)
    t, s, v, xx = dev(trellis), dev(suh), dev(svh), dev(x)
    run("amp_exl3_gemv_static", xx, t, s, v, 2, 2048, 1024, 4)          # set-up call (symbol address, kernel attribute)
    out = torch.empty((2, 1024), dtype=torch.float16, device="cuda")
    from ampstein_b200 import _lib
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for _ in range(8):
        _lib.call("amp_exl3_gemv_static", xx.data_ptr(), t.data_ptr(), out.data_ptr(), s.data_ptr(), v.data_ptr(),
                  2, 2048, 1024, 4, 0, 0, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0


FIRST_CALL_SCRIPT = r"""
import sys
sys.path.insert(0, %r)
sys.path.insert(0, %r)
import numpy as np, torch
from conftest import make_linear
from ampstein_b200 import _lib
from oracle import exl3_oracle as oracle
trellis, suh, svh, x = make_linear(4096, 512, 4, seed=9104, m=1)
d = lambda a: torch.from_numpy(np.ascontiguousarray(a.view(np.int16) if a.dtype == np.uint16 else a)).cuda()
t, s, v, xx = d(trellis), d(suh), d(svh), d(x)
out = torch.full((1, 512), float("nan"), dtype=torch.float16, device="cuda")
torch.cuda.synchronize()
free0 = torch.cuda.mem_get_info()[0]
# the first GEMV call of this process: no workspace of the allocating entry point exists
for _ in range(3):
    _lib.call("amp_exl3_gemv_static", xx.data_ptr(), t.data_ptr(), out.data_ptr(), s.data_ptr(), v.data_ptr(),
              1, 4096, 512, 4, 0, 0, torch.cuda.current_stream().cuda_stream)
torch.cuda.synchronize()
# loading the kernel's module on first use may take device memory once; nothing may be taken per call
free1 = torch.cuda.mem_get_info()[0]
for _ in range(3):
    _lib.call("amp_exl3_gemv_static", xx.data_ptr(), t.data_ptr(), out.data_ptr(), s.data_ptr(), v.data_ptr(),
              1, 4096, 512, 4, 0, 0, torch.cuda.current_stream().cuda_stream)
torch.cuda.synchronize()
assert torch.cuda.mem_get_info()[0] == free1, "a later call allocated device memory"
want = oracle.linear(x, trellis, suh, svh, 0, fp32_out=True)
err = np.max(np.abs(out.float().cpu().numpy() - want)) / np.max(np.abs(want))
assert err < 1e-2, err
print("first-call ok", free0 - free1, err)
"""


def test_static_scratch_as_the_first_gemv_call_of_a_process():
    from conftest import ROOT
    script = FIRST_CALL_SCRIPT % (ROOT, os.path.join(ROOT, "tests"))
    r = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0 and "first-call ok" in r.stdout, r.stdout[-1500:] + r.stderr[-1500:]
