"""GPU parity of the half-integer bitrates 1.5 / 2.5 / 3.5 (mul1 codebook; trellis third dimension 16 KA
+ 8) through the C ABI: reconstruct and reconstruct_had bit for bit against the CPU oracle (which
the reference's own kernels pin through tests/golden/ref_reconstruct_K*5_cb2.npz), the decode kernel
and the many-rows operator within 1e-2 of the fp32-accumulated oracle, the shard cutters bit for bit."""
import numpy as np
import pytest

from conftest import make_linear

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def dev(a):
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(scope="module")
def amp():
    import ampstein_b200
    return ampstein_b200


@pytest.mark.parametrize("K", [1.5, 2.5, 3.5])
def test_reconstruct_bit_exact(amp, oracle, K):
    k, n = 256, 384
    trellis, suh, svh, _ = make_linear(k, n, K, seed=int(10 * K))
    assert trellis.shape[2] == 16 * int(K) + 8
    w = torch.empty((k, n), dtype=torch.float16, device="cuda")
    amp.exl3_reconstruct(w, dev(trellis), K, mul1=True)
    assert np.array_equal(w.cpu().numpy().view(np.uint16), oracle.reconstruct(trellis, 2).view(np.uint16))
    sc = np.random.default_rng(3).uniform(0.5, 2.0, n).astype(np.float16)
    wh = torch.empty((k, n), dtype=torch.float16, device="cuda")
    amp.exl3_reconstruct_had(wh, dev(trellis), dev(suh), dev(svh * sc), K, mul1=True)
    assert np.array_equal(wh.cpu().numpy().view(np.uint16), oracle.reconstruct_had(trellis, suh, svh * sc, 2).view(np.uint16))
    # a column slice, as the reference's reconstruct_had_slice takes it
    ws = torch.empty((k, 128), dtype=torch.float16, device="cuda")
    amp.exl3_reconstruct_had(ws, dev(trellis), dev(suh), dev((svh * sc)[256:]), K, mul1=True, n_offset=256)
    assert np.array_equal(ws.cpu().numpy().view(np.uint16), wh.cpu().numpy()[:, 256:].view(np.uint16))
    with pytest.raises(ValueError):
        amp.exl3_reconstruct(w, dev(trellis), K)                    # half-integer rates need mul1
    with pytest.raises(ValueError):
        amp.exl3_reconstruct(w, dev(trellis), int(K), mul1=True)    # K must match the trellis


@pytest.mark.parametrize("K,m,k,n", [(2.5, 1, 512, 256), (1.5, 3, 1024, 384), (3.5, 8, 2048, 128), (2.5, 16, 1536, 512), (3.5, 1, 4096, 1024)])
def test_decode_rows(amp, oracle, K, m, k, n):
    trellis, suh, svh, x = make_linear(k, n, K, seed=100 + m + n, m=m)
    svh = (svh.astype(np.float32) / (1.2437 * np.sqrt(k))).astype(np.float16)
    ref = oracle.linear(x, trellis, suh, svh, 2, fp32_out=True)
    for dt in (torch.float16, torch.float32):
        y = torch.full((m, n), float("nan"), dtype=dt, device="cuda")
        amp.exl3_gemm(dev(x), dev(trellis), y, dev(suh), dev(svh), mul1=True)
        torch.cuda.synchronize()
        got = y.float().cpu().numpy()
        assert np.all(np.isfinite(got))
        assert np.max(np.abs(got - ref)) / np.max(np.abs(ref)) < (2e-3 if dt == torch.float16 else 1e-3)


@pytest.mark.parametrize("K,rows", [(2.5, 40), (1.5, 300)])
def test_many_rows_reconstruct_once(amp, oracle, K, rows):
    """Above 16 rows the half-integer rates take the reference's own many-rows form: the weight
    decoded once into the original basis, then a library GEMM (exl3_gemm and exl3_gemm_recon alike)."""
    k, n = 512, 384
    trellis, suh, svh, x = make_linear(k, n, K, seed=200 + rows, m=rows)
    svh = (svh.astype(np.float32) / (1.2437 * np.sqrt(k))).astype(np.float16)
    ref = oracle.linear(x, trellis, suh, svh, 2, fp32_out=True)
    y = torch.empty((rows, n), dtype=torch.float16, device="cuda")
    amp.exl3_gemm(dev(x), dev(trellis), y, dev(suh), dev(svh), mul1=True)
    z = amp.exl3_gemm_recon(dev(x), dev(trellis), dev(suh), dev(svh), K, mul1=True)
    torch.cuda.synchronize()
    for got in (y, z):
        g = got.float().cpu().numpy()
        assert np.max(np.abs(g - ref)) / np.max(np.abs(ref)) < 1e-2


def test_shards_and_model_layer(amp, oracle):
    from ampstein_b200.models import LinearEXL3, cols, rows
    K, k, n = 2.5, 512, 512
    trellis, suh, svh, x = make_linear(k, n, K, seed=300, m=2)
    t, s, v = dev(trellis), dev(suh), dev(svh)
    tr, sv = amp.exl3_shard_cols(t, v, [(256, 128), (0, 128)])
    want = np.concatenate([trellis[:, 16:24], trellis[:, 0:8]], axis=1)
    assert tr.shape[2] == 40 and np.array_equal(tr.cpu().numpy().view(np.uint16), want.view(np.uint16))
    tr2, su2 = amp.exl3_shard_rows(t, s, 128, 256)
    assert np.array_equal(tr2.cpu().numpy().view(np.uint16), trellis[8:24].view(np.uint16))
    lin = LinearEXL3(t, s, v, mul1=True)
    full = lin.forward(dev(x)).float().cpu().numpy()
    part = cols(lin, [(256, 128), (0, 128)]).forward(dev(x)).float().cpu().numpy()
    assert np.max(np.abs(part - np.concatenate([full[:, 256:384], full[:, :128]], axis=1))) / np.max(np.abs(full)) < 2e-3
    ref = oracle.linear(x, trellis, suh, svh, 2, fp32_out=True)
    assert np.max(np.abs(full - ref)) / np.max(np.abs(ref)) < 1e-2
