"""GPU parity of the tensor-memory form of the decode GEMV (tcgen05.st of the decoded weights
into tensor memory, tcgen05.mma with the weights as the A operand), selected with
amp_exl3_set_gemv_tc(1), against the CPU oracle and against the default mma.sync kernel."""
import numpy as np
import pytest

from conftest import make_linear
from test_gpu_parity import check_close, dev, run_gemm

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture()
def amp_tmem():
    import ampstein_b200
    from ampstein_b200 import _lib
    old = _lib.lib().amp_exl3_set_gemv_tc(1)
    yield ampstein_b200
    _lib.lib().amp_exl3_set_gemv_tc(old)


@pytest.mark.parametrize("cb", [0, 1, 2])
@pytest.mark.parametrize("K", range(1, 9))
def test_all_bitrates(amp_tmem, oracle, K, cb):
    trellis, suh, svh, x = make_linear(512, 256, K, seed=3000 + 10 * K + cb, m=3)
    check_close(run_gemm(amp_tmem, trellis, suh, svh, x, cb), oracle.linear(x, trellis, suh, svh, cb, fp32_out=True))


@pytest.mark.parametrize("m", [1, 2, 5, 8])
def test_batch_sizes_and_output_types(amp_tmem, oracle, m):
    trellis, suh, svh, x = make_linear(1024, 384, 4, seed=4000 + m, m=m)
    ref = oracle.linear(x, trellis, suh, svh, 0, fp32_out=True)
    check_close(run_gemm(amp_tmem, trellis, suh, svh, x, 0), ref)
    check_close(run_gemm(amp_tmem, trellis, suh, svh, x, 0, fp32=True), ref)


@pytest.mark.parametrize("split", [1, 2, 3, 5, 8, 37, 72, 148])
def test_ranges_that_start_and_end_inside_a_block(amp_tmem, oracle, split):
    trellis, suh, svh, x = make_linear(2304, 256, 4, seed=5000, m=2)
    ref = oracle.linear(x, trellis, suh, svh, 0, fp32_out=True)
    check_close(run_gemm(amp_tmem, trellis, suh, svh, x, 0, split=split), ref)


@pytest.mark.parametrize("k,n,K", [(4096, 4096, 4), (4096, 14336, 4), (14336, 4096, 4), (4096, 2048, 6), (128, 128, 5)])
def test_layer_shapes_and_agreement_with_the_default_kernel(amp_tmem, oracle, k, n, K):
    from ampstein_b200 import _lib
    trellis, suh, svh, x = make_linear(k, n, K, seed=k + n + K, m=1)
    ref = oracle.linear(x, trellis, suh, svh, 0, fp32_out=True)
    got = run_gemm(amp_tmem, trellis, suh, svh, x, 0, fp32=True)
    check_close(got, ref)
    again = run_gemm(amp_tmem, trellis, suh, svh, x, 0, fp32=True)
    assert np.array_equal(got, again)                      # bitwise reproducible
    _lib.lib().amp_exl3_set_gemv_tc(0)
    check_close(run_gemm(amp_tmem, trellis, suh, svh, x, 0, fp32=True), got)
    _lib.lib().amp_exl3_set_gemv_tc(1)


def test_bundles(amp_tmem, oracle):
    from ampstein_b200.models import LinearEXL3, Multi, Sliced
    k, m = 1024, 3
    rng = np.random.default_rng(77)
    x = rng.standard_normal((m, k)).astype(np.float16)
    xd = dev(x).reshape(1, m, k)

    def lin(n, seed):
        trellis, suh, svh, _ = make_linear(k, n, 4, seed=seed)
        return (trellis, suh, svh), LinearEXL3(dev(trellis), dev(suh), dev(svh))

    (g_np, g), (u_np, u) = lin(768, 1), lin(768, 2)
    out = torch.full((2, m, 768), float("nan"), dtype=torch.float16, device="cuda")
    Multi([g, u], out).run(xd)
    torch.cuda.synchronize()
    for i, (t, su, sv) in enumerate((g_np, u_np)):
        check_close(out[i].cpu().numpy(), oracle.linear(x, t, su, sv, 0, fp32_out=True))
    (q_np, q), (k_np, kk), (v_np, v) = lin(1024, 3), lin(256, 4), lin(256, 5)
    outs = [torch.full((1, m, n), float("nan"), dtype=torch.float16, device="cuda") for n in (1024, 256, 256)]
    Sliced([q, kk, v], outs).run(xd)
    torch.cuda.synchronize()
    for o, (t, su, sv) in zip(outs, (q_np, k_np, v_np)):
        check_close(o[0].cpu().numpy(), oracle.linear(x, t, su, sv, 0, fp32_out=True))
