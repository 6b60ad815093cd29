"""amp_exl3_gemv_static: the decode GEMV whose scratch is a fixed array inside the library (no
device allocation at any call). Runs last in the suite on purpose: it must work on a device whose
other workspaces already exist, and alone."""
import ctypes

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
