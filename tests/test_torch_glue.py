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
    for name in ("exl3_gemm", "exl3_mgemm", "reconstruct", "reconstruct_had_slice", "had_r_128", "exl3_moe_coop",
                 "exl3_moe", "exl3_moe_gather", "exl3_moe_max_concurrency"):
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


@pytest.mark.gpu
def test_glue_sorted_moe_with_the_reference_call_sequence(glue, amp, oracle):
    """exl3_moe / exl3_moe_gather with the reference's argument lists, called the way its runtime calls
    them (src/ucode/ampstein/glm5.uc:1204-1230): three row tiers, once adding straight into the
    output and once through the per-assignment slots + gather. Experts with more rows than the
    reference's temps hold are left to the caller, as in the reference."""
    from test_gpu_moe import build_cfg, make_experts
    from test_gpu_moe_sorted import routing
    E, H, I, K, topk, T = 8, 256, 128, 4, 2, 120
    ex = make_experts(E, H, I, H, K, seed=7500)
    rng = np.random.default_rng(75)
    x = rng.standard_normal((T, H)).astype(np.float16)
    sel, rw = routing(rng, T, E, topk)
    cfg = build_cfg(amp, ex, H, I, H, H, K, 1, topk)
    xd = dev(x)
    count, tok, wts, fe, inv, start = amp.moe_sort_routing(dev(sel), dev(rw), E, 0, with_inverse=True)
    conc, cap = glue.exl3_moe_max_concurrency(0), 64
    assert conc == torch.cuda.get_device_properties(0).multi_processor_count // 8
    z = lambda *shape: torch.zeros(shape, dtype=torch.float16, device="cuda")
    temps = (z(conc, cap, H), z(conc, cap, H), z(conc, cap, I), z(conc, cap, I))
    tabs = [cfg[n] for n in ("g_trellis", "g_suh", "g_svh", "u_trellis", "u_suh", "u_svh", "d_trellis", "d_suh", "d_svh")]

    def fused(out, scratch=None, base=None):
        for lo, hi, mt in ((33, cap, 64), (17, 32, 32), (1, 16, 16)):
            glue.exl3_moe(xd, out, count, tok, wts, *temps, 0, float(K), float(K), float(K), *tabs,
                          False, False, False, False, False, False, 0.0, -1, scratch, base, lo, hi, mt, None, None, None)

    out = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    fused(out)
    torch.cuda.synchronize()
    ref = oracle.moe_coop(x, sel, rw, ex, gu_f16=True)
    got = out.cpu().numpy()
    err = np.max(np.abs(got - ref)) / np.max(np.abs(ref))
    assert err < 1e-2, err
    scratch = torch.zeros((T * topk, H), dtype=torch.float32, device="cuda")
    out2 = torch.zeros_like(out)
    fused(out2, scratch, start)
    assert not out2.any()
    kind = (count[:E] > 0).to(torch.int64)
    glue.exl3_moe_gather(out2, scratch, fe, inv, start[:E].contiguous(), start[:E].contiguous(), kind, wts)
    torch.cuda.synchronize()
    assert np.allclose(out2.cpu().numpy(), got, rtol=1e-5, atol=1e-6)
    # an expert above the temps' capacity is skipped (the caller's heavy tier handles it)
    small = tuple(t[:, :8].contiguous() for t in temps)
    out3 = torch.zeros_like(out)
    glue.exl3_moe(xd, out3, count, tok, wts, *small, 0, float(K), float(K), float(K), *tabs,
                  False, False, False, False, False, False, 0.0, -1, None, None, 1, 8, 16, None, None, None)
    torch.cuda.synchronize()
    light = [e for e in range(E) if 0 < int(count[e]) <= 8]
    assert bool(out3.any()) == bool(light)
    with pytest.raises(RuntimeError):
        glue.exl3_moe(xd, out3.half(), count, tok, wts, *temps, 0, float(K), float(K), float(K), *tabs,
                      False, False, False, False, False, False, 0.0, -1, None, None, 1, cap, 16, None, None, None)


@pytest.mark.gpu
def test_glue_half_integer_bitrates(glue, oracle):
    """The reference's float K at the C++ boundary (bits_from_K, vendor/exl3/exllamav3_ext/quant/bits_k.cuh:14-29):
    2.5 bits per weight through reconstruct, reconstruct_had_slice and exl3_gemm (decode kernel with the
    A_had scratch, reconstruct + library GEMM above 16 rows or without it)."""
    K, k, n = 2.5, 256, 256
    trellis, suh, svh, x = make_linear(k, n, K, seed=7700, m=20)
    t, su, sv = dev(trellis), dev(suh), dev(svh)
    w = torch.empty((k, n), dtype=torch.float16, device="cuda")
    glue.reconstruct(w, t, 2.5, False, True)
    assert np.array_equal(w.cpu().numpy().view(np.uint16), oracle.reconstruct(trellis, 2).view(np.uint16))
    glue.reconstruct_had_slice(w, t, su, sv, 2.5, False, True, 0)
    assert np.array_equal(w.cpu().numpy().view(np.uint16), oracle.reconstruct_had(trellis, suh, svh, 2).view(np.uint16))
    ref = oracle.linear(x, trellis, suh, svh, 2, fp32_out=True)
    for rows, scratch in ((1, True), (4, False), (20, True)):
        xx = dev(x[:rows])
        y = torch.empty((rows, n), dtype=torch.float16, device="cuda")
        fam = glue.exl3_gemm(xx, t, y, su, torch.empty_like(xx) if scratch else None, sv, 0, False, True, 0)
        torch.cuda.synchronize()
        assert fam == (90 if rows <= 16 and scratch else 100)
        err = np.max(np.abs(y.float().cpu().numpy() - ref[:rows])) / np.max(np.abs(ref[:rows]))
        assert err < 1e-2, (rows, err)
    with pytest.raises(RuntimeError):
        glue.reconstruct(w, t, 2.5, False, False)                   # mul1 only
    with pytest.raises(RuntimeError):
        glue.reconstruct(w, t, 2.0, False, True)                    # K must match the trellis
