"""The libtorch C++ layer (reference signatures over at::Tensor, ampstein_b200/_torch_glue.so):
it must load, throw on bad arguments like the reference's TORCH_CHECKs, and give the same bits as
the ctypes path (both end in the same C-ABI calls)."""
import numpy as np
import pytest
import torch

from conftest import make_linear


@pytest.fixture(scope="module")
def glue():
    from ampstein_b200 import build as amp_build
    amp_build.build_torch_glue()
    from ampstein_b200 import _torch_glue
    return _torch_glue


def test_glue_exports_reference_names(glue):
    for name in ("exl3_gemm", "exl3_mgemm", "reconstruct", "reconstruct_had_slice", "had_r_128", "exl3_moe_coop"):
        assert callable(getattr(glue, name))


def test_glue_rejects_cpu_tensors(glue):
    a = torch.zeros((1, 128), dtype=torch.float16)
    b = torch.zeros((8, 8, 64), dtype=torch.int16)
    c = torch.zeros((1, 128), dtype=torch.float16)
    s = torch.ones(128, dtype=torch.float16)
    with pytest.raises(RuntimeError):
        glue.exl3_gemm(a, b, c, s, None, s, 0, False, False, 0)
    with pytest.raises(RuntimeError):
        glue.reconstruct(torch.zeros((128, 128), dtype=torch.float16), b, 4.0, False, False)


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


@pytest.mark.gpu
@pytest.mark.parametrize("m", [1, 5, 64])
def test_glue_gemm_matches_ctypes_path(glue, amp, oracle, m):
    trellis, suh, svh, x = make_linear(512, 384, 4, seed=7100 + m, m=m)
    t, s, v, xx = dev(trellis), dev(suh), dev(svh), dev(x)
    c1 = torch.empty((m, 384), dtype=torch.float16, device="cuda")
    c2 = torch.empty_like(c1)
    idx = glue.exl3_gemm(xx, t, c1, s, torch.empty_like(xx), v, 0, False, False, 0)
    assert idx == (90 if m <= 16 else 100)
    amp.exl3_gemm(xx, t, c2, s, v)
    torch.cuda.synchronize()
    assert torch.equal(c1, c2)
    ref = oracle.linear(x, trellis, suh, svh, 0, fp32_out=True)
    err = np.max(np.abs(c1.float().cpu().numpy() - ref)) / np.max(np.abs(ref))
    assert err < 1e-2                      # max relative error against the fp32-accumulated oracle


@pytest.mark.gpu
def test_glue_reconstruct_and_hadamard_bit_exact(glue, oracle):
    trellis, suh, svh, x = make_linear(256, 256, 5, seed=7200, m=3)
    w = torch.empty((256, 256), dtype=torch.float16, device="cuda")
    glue.reconstruct(w, dev(trellis), 5.0, False, True)
    assert np.array_equal(w.cpu().numpy().view(np.uint16), oracle.reconstruct(trellis, 2).view(np.uint16))
    wh = torch.empty((256, 128), dtype=torch.float16, device="cuda")
    glue.reconstruct_had_slice(wh, dev(trellis), dev(suh), dev(svh[128:]), 5.0, False, False, 128)
    ref = oracle.reconstruct_had(trellis, suh, svh, 0)[:, 128:]
    assert np.array_equal(wh.cpu().numpy().view(np.uint16), ref.view(np.uint16))
    xx = dev(x)
    y = torch.empty_like(xx)
    glue.had_r_128(xx, y, dev(suh), None, 1.0)
    assert np.array_equal(y.cpu().numpy().view(np.uint16), oracle.had_hf(x, pre=suh).view(np.uint16))
    with pytest.raises(RuntimeError):
        glue.reconstruct(w, dev(trellis), 4.0, False, False)       # K does not match the trellis


@pytest.mark.gpu
def test_glue_mgemm_stacked(glue, amp, oracle):
    lins = [make_linear(512, 256, 4, seed=7300 + i, m=2) for i in range(2)]
    x = lins[0][3]
    keep = [(dev(t), dev(s), dev(v)) for t, s, v, _ in lins]
    B = amp.ptr_array([k[0].data_ptr() for k in keep])
    S = amp.ptr_array([k[1].data_ptr() for k in keep])
    V = amp.ptr_array([k[2].data_ptr() for k in keep])
    xx = dev(x).view(1, 2, 512)
    C = torch.empty((2, 2, 256), dtype=torch.float16, device="cuda")
    glue.exl3_mgemm(xx, B, C, S, torch.empty_like(xx), V, None, None, 4.0, 0, 0, 0, -1, -1, 0, 1, None, None, None, None, 0)
    torch.cuda.synchronize()
    for i, (t, s, v, _) in enumerate(lins):
        ref = oracle.linear(x, t, s, v, 0, fp32_out=True)
        err = np.max(np.abs(C[i].float().cpu().numpy() - ref)) / np.max(np.abs(ref))
        assert err < 1e-2
