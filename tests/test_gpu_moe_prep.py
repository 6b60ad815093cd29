"""GPU parity of the one-launch MoE dispatch (amp_moe_prep) through the C ABI: integer work, checked
bit for bit against a numpy stable sort, on the cases of the reference's own test
(tests/moe_prep.uc:7-68: same id / weight generators and sizes) plus the extremes of E."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def amp():
    import ampstein_b200
    return ampstein_b200


def expected(ids, ws, K, E, e0):
    A = ids.size
    loc = ids.reshape(-1) - e0
    fe = np.where((loc >= 0) & (loc < E), loc, E).astype(np.int64)
    order = np.argsort(fe, kind="stable").astype(np.int64)
    inv = np.empty(A, np.int64)
    inv[order] = np.arange(A)
    count = np.bincount(fe, minlength=E + 1).astype(np.int64)
    start = np.cumsum(count) - count
    return dict(fe=fe, order=order, tok=order // K, wts=ws.reshape(-1)[order].astype(np.float16), count=count,
                start=start, inv=inv, kind=(count[:E] > 0).astype(np.int64))


def run(amp, ids, ws, E, e0):
    r = amp.moe_prep(torch.from_numpy(ids).cuda(), torch.from_numpy(ws).cuda(), E, e0)
    torch.cuda.synchronize()
    return dict(zip(("fe", "order", "tok", "wts", "count", "start", "inv", "kind"), (t.cpu().numpy() for t in r)))


@pytest.mark.parametrize("T,K,E,e0,NE", [(5, 6, 384, 0, 384), (40, 6, 192, 192, 384), (300, 6, 192, 0, 384), (128, 3, 64, 64, 128),
                                         (4096, 10, 512, 0, 512), (1000, 10, 256, 100, 512), (33, 10, 512, 0, 512)])
def test_reference_cases(amp, T, K, E, e0, NE):
    a = np.arange(T * K, dtype=np.int64)
    ids = ((a * 37 + (a // K) * 11) % NE).reshape(T, K)
    ws = (0.01 * ((a % 17) + 1)).astype(np.float32).reshape(T, K)
    got, ref = run(amp, ids, ws, E, e0), expected(ids, ws, K, E, e0)
    for key in ref:
        if key == "wts":
            assert np.array_equal(got[key].view(np.uint16), ref[key].view(np.uint16)), key
        else:
            assert np.array_equal(got[key], ref[key]), key


@pytest.mark.parametrize("T,K,E,e0,NE", [(1, 1, 1, 0, 1), (1, 8, 4096, 0, 4096), (2048, 8, 128, 0, 128), (3000, 8, 4096, 17, 5000),
                                         (777, 5, 400, 0, 400), (777, 5, 401, 3, 500)])
def test_random_routing_and_the_extremes_of_e(amp, T, K, E, e0, NE):
    """One expert, the largest expert count (fewer sorting warps: the counters of 32 would not fit
    in shared memory), the benchmark's chunk, the widths either side of the 32-warp limit."""
    rng = np.random.default_rng(T + E)
    ids = rng.integers(0, NE, size=(T, K), dtype=np.int64)
    ws = rng.random((T, K), dtype=np.float32)
    got, ref = run(amp, ids, ws, E, e0), expected(ids, ws, K, E, e0)
    for key in ref:
        assert np.array_equal(got[key].view(np.uint16) if key == "wts" else got[key],
                              ref[key].view(np.uint16) if key == "wts" else ref[key]), key


def test_agrees_with_the_torch_built_dispatch_and_feeds_the_sorted_moe(amp):
    rng = np.random.default_rng(9)
    T, K, E = 300, 4, 16
    sel = torch.from_numpy(rng.integers(0, E, size=(T, K), dtype=np.int64)).cuda()
    w = torch.from_numpy(rng.random((T, K), dtype=np.float32)).cuda()
    fe, order, tok, wts, count, start, inv, kind = amp.moe_prep(sel, w, E, 0)
    c2, t2, w2, fe2, inv2, start2 = amp.moe_sort_routing(sel, w, E, 0, with_inverse=True)
    assert torch.equal(count, c2) and torch.equal(tok, t2) and torch.equal(wts, w2) and torch.equal(fe, fe2)
    assert torch.equal(inv, inv2) and torch.equal(start, start2)


def test_argument_errors(amp):
    idx = torch.zeros((4, 2), dtype=torch.int64, device="cuda")
    w = torch.zeros((4, 2), dtype=torch.float32, device="cuda")
    with pytest.raises(ValueError):
        amp.moe_prep(idx, w, 5000)
    with pytest.raises(ValueError):
        amp.moe_prep(idx, w.half(), 8)
    with pytest.raises(RuntimeError):
        amp.moe_prep(idx.cpu(), w, 8)
