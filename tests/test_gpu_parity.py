"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle on identical
seeded inputs. Decoded weights and Hadamard outputs must be bit-exact; linear outputs within
max relative error 1e-2 of the fp32-accumulated reference (the tolerance of the specification;
measured errors are ~5e-4, fp16 output rounding)."""
import ctypes

import numpy as np
import pytest

from conftest import make_linear

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

MAX_REL = 1e-2       # max |y - ref| / max |ref|
REL_RMS = 2e-3


def dev(a):
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host16(t):
    return t.cpu().numpy().view(np.uint16)


def check_close(got, ref):
    got, ref = got.astype(np.float64), ref.astype(np.float64)
    assert np.all(np.isfinite(got))
    max_rel = np.max(np.abs(got - ref)) / np.max(np.abs(ref))
    rms = np.sqrt(np.mean((got - ref) ** 2) / np.mean(ref ** 2))
    assert max_rel < MAX_REL and rms < REL_RMS, (max_rel, rms)
    return max_rel, rms


@pytest.fixture(scope="module")
def amp():
    import ampstein_b200
    from ampstein_b200 import _lib
    _lib.lib()
    return ampstein_b200


@pytest.mark.parametrize("cb", [0, 1, 2])
@pytest.mark.parametrize("K", range(1, 9))
def test_reconstruct_bit_exact(amp, oracle, K, cb):
    trellis, _, _, _ = make_linear(64, 256, K, seed=1000 + 10 * K + cb)
    out = torch.empty((64, 256), dtype=torch.float16, device="cuda")
    amp.exl3_reconstruct(out, dev(trellis), K, mul1=(cb == 2), mcg=(cb == 1))
    assert np.array_equal(host16(out), oracle.reconstruct(trellis, cb).view(np.uint16))


def test_reconstruct_4096_bit_exact_and_slices(amp, oracle):
    trellis, _, _, _ = make_linear(4096, 4096, 4, seed=0)
    t = dev(trellis)
    out = torch.empty((4096, 4096), dtype=torch.float16, device="cuda")
    amp.exl3_reconstruct(out, t, 4)
    ref = oracle.reconstruct(trellis, 0).view(np.uint16)
    assert np.array_equal(host16(out), ref)
    # column slice through the C ABI (reconstruct_slice semantics)
    from ampstein_b200 import _lib
    sl = torch.empty((4096, 256), dtype=torch.float16, device="cuda")
    _lib.call("amp_exl3_reconstruct", sl.data_ptr(), t.data_ptr(), 4096, 4096, 4, 0, 1024, 256,
              torch.cuda.current_stream().cuda_stream)
    assert np.array_equal(host16(sl), ref[:, 1024:1280])


@pytest.mark.parametrize("K,cb", [(2, 0), (4, 2), (5, 1)])
def test_reconstruct_batch_forms_bit_exact(amp, oracle, K, cb):
    """Three matrices of one shape in one launch, rotated and original basis, against the oracle."""
    mats = [make_linear(256, 384, K, seed=2500 + 7 * K + i) for i in range(3)]
    keep = [(dev(t), dev(su), dev(sv)) for t, su, sv, _ in mats]
    ptrs = [amp.ptr_array([k[i].data_ptr() for k in keep]) for i in range(3)]
    out = torch.full((3, 256, 384), float("nan"), dtype=torch.float16, device="cuda")
    amp.exl3_reconstruct_batch(out, ptrs[0], K, mul1=(cb == 2), mcg=(cb == 1))
    for i, (t, _, _, _) in enumerate(mats):
        assert np.array_equal(host16(out[i]), oracle.reconstruct(t, cb).view(np.uint16))
    out.fill_(float("nan"))
    amp.exl3_reconstruct_batch(out, ptrs[0], K, mul1=(cb == 2), mcg=(cb == 1), suh_ptrs=ptrs[1], svh_ptrs=ptrs[2])
    for i, (t, su, sv, _) in enumerate(mats):
        assert np.array_equal(host16(out[i]), oracle.reconstruct_had(t, su, sv, cb).view(np.uint16))


@pytest.mark.parametrize("K,cb", [(1, 0), (3, 2), (4, 0), (5, 1), (6, 0), (8, 2)])
def test_reconstruct_had_bit_exact(amp, oracle, K, cb):
    trellis, suh, svh, _ = make_linear(256, 384, K, seed=2000 + K)
    rng = np.random.default_rng(K)
    suh = (suh.astype(np.float32) * rng.uniform(0.5, 2.0, suh.shape)).astype(np.float16)
    out = torch.empty((256, 384), dtype=torch.float16, device="cuda")
    amp.exl3_reconstruct_had(out, dev(trellis), dev(suh), dev(svh), K, mul1=(cb == 2), mcg=(cb == 1))
    ref = oracle.reconstruct_had(trellis, suh, svh, cb).view(np.uint16)
    assert np.array_equal(host16(out), ref)
    # slice: columns 128..383 with the slice's own svh
    sl = torch.empty((256, 256), dtype=torch.float16, device="cuda")
    amp.exl3_reconstruct_had(sl, dev(trellis), dev(suh), dev(svh[128:]), K, mul1=(cb == 2), mcg=(cb == 1), n_offset=128)
    assert np.array_equal(host16(sl), ref[:, 128:])


def test_had_r_128_bit_exact(amp, oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((37, 512)).astype(np.float16)
    pre = rng.choice(np.array([-1.0, 1.0], np.float16), 512)
    post = (rng.uniform(0.5, 2, 512)).astype(np.float16)
    for kw in ({"pre": pre}, {"post": post}, {}, {"pre": pre, "post": post}):
        out = torch.empty((37, 512), dtype=torch.float16, device="cuda")
        amp.had_r_128(dev(x), out, dev(kw["pre"]) if "pre" in kw else None,
                      dev(kw["post"]) if "post" in kw else None)
        assert np.array_equal(host16(out), oracle.had_hf(x, **kw).view(np.uint16)), kw
    xf = rng.standard_normal((5, 256)).astype(np.float32)
    outf = torch.empty((5, 256), dtype=torch.float32, device="cuda")
    amp.had_r_128(dev(xf), outf, None, dev(post[:256]))
    assert np.array_equal(outf.cpu().numpy(), oracle.had_ff(xf, post=post[:256]))
    # fp32 in, fp16 out: transform in fp32, one rounding, fp16 post-scale
    outh = torch.empty((5, 256), dtype=torch.float16, device="cuda")
    amp.had_r_128(dev(xf), outh, None, dev(post[:256]))
    assert np.array_equal(host16(outh), oracle.had_fh(xf, post=post[:256]).view(np.uint16))
    amp.had_r_128(dev(xf), outh)
    assert np.array_equal(host16(outh), oracle.had_fh(xf).view(np.uint16))
    # in place
    t = dev(x)
    amp.had_r_128(t, t, dev(pre), None)
    assert np.array_equal(host16(t), oracle.had_hf(x, pre=pre).view(np.uint16))


def run_gemm(amp, trellis, suh, svh, x, cb, fp32=False, split=0, xgroups=0):
    from ampstein_b200 import _lib
    m, k = x.shape
    n = trellis.shape[1] * 16
    K = trellis.shape[2] // 16
    out = torch.full((m, n), float("nan"), dtype=torch.float32 if fp32 else torch.float16, device="cuda")
    t, s, v, xx = dev(trellis), dev(suh), dev(svh), dev(x)
    if split or xgroups:
        _lib.call("amp_exl3_gemv_cfg", xx.data_ptr(), t.data_ptr(), out.data_ptr(), s.data_ptr(), v.data_ptr(),
                  m, k, n, K, cb, int(fp32), split, xgroups, torch.cuda.current_stream().cuda_stream)
    else:
        amp.exl3_gemm(xx, t, out, s, v, mul1=(cb == 2), mcg=(cb == 1))
    torch.cuda.synchronize()
    st = ctypes.c_int(-1)
    _lib.call("amp_exl3_gemv_status", ctypes.byref(st))
    assert st.value == 0, "a bounded wait ran out inside the kernel"
    return out.cpu().numpy()


@pytest.mark.parametrize("cb", [0, 1, 2])
@pytest.mark.parametrize("K", range(1, 9))
def test_gemv_all_bitrates(amp, oracle, K, cb):
    trellis, suh, svh, x = make_linear(512, 256, K, seed=3000 + 10 * K + cb, m=3)
    got = run_gemm(amp, trellis, suh, svh, x, cb)
    check_close(got, oracle.linear(x, trellis, suh, svh, cb, fp32_out=True))


@pytest.mark.parametrize("m", [1, 2, 7, 8, 9, 16])
def test_gemv_batch_sizes(amp, oracle, m):
    trellis, suh, svh, x = make_linear(1024, 384, 4, seed=4000 + m, m=m)
    ref = oracle.linear(x, trellis, suh, svh, 0, fp32_out=True)
    check_close(run_gemm(amp, trellis, suh, svh, x, 0), ref)
    check_close(run_gemm(amp, trellis, suh, svh, x, 0, fp32=True), ref)


@pytest.mark.parametrize("split,xgroups", [(1, 0), (1, 4), (2, 8), (3, 0), (5, 4), (8, 12), (8, 0), (37, 4), (72, 0), (148, 4)])
def test_gemv_splits_and_chunk_sizes(amp, oracle, split, xgroups):
    # k = 2304 = 36 groups x 2 column blocks = 72 units: one CTA walking both blocks, ragged
    # ranges that start and end inside a block, one unit per CTA, more CTAs than units
    trellis, suh, svh, x = make_linear(2304, 256, 4, seed=5000, m=2)
    ref = oracle.linear(x, trellis, suh, svh, 0, fp32_out=True)
    check_close(run_gemm(amp, trellis, suh, svh, x, 0, split=split, xgroups=xgroups), ref)


def test_gemv_split_larger_than_blocks(amp, oracle):
    trellis, suh, svh, x = make_linear(256, 128, 5, seed=5100, m=1)
    ref = oracle.linear(x, trellis, suh, svh, 0, fp32_out=True)
    check_close(run_gemm(amp, trellis, suh, svh, x, 0, split=8, xgroups=4), ref)


def test_config1_single_layer_4096(amp, oracle):
    """in = out = 4096, K = 4, batch 1, +-1 sign vectors (the reference's CPU-runnable case)."""
    trellis, suh, svh, x = make_linear(4096, 4096, 4, seed=0, m=1)
    ref = oracle.linear(x, trellis, suh, svh, 0, fp32_out=True)
    check_close(run_gemm(amp, trellis, suh, svh, x, 0), ref)


@pytest.mark.parametrize("k,n,K", [(4096, 1024, 4), (4096, 14336, 4), (14336, 4096, 4), (4096, 2048, 6), (5120, 6144, 5),
                                   # shards of the tensor-parallel stack (8 and 4 ways): short k, narrow n
                                   (512, 4096, 4), (1792, 4096, 4), (4096, 768, 4), (3584, 4096, 4), (1024, 4096, 4)])
def test_llama_shapes(amp, oracle, k, n, K):
    trellis, suh, svh, x = make_linear(k, n, K, seed=k + n + K, m=1)
    ref = oracle.linear(x, trellis, suh, svh, 0, fp32_out=True)
    check_close(run_gemm(amp, trellis, suh, svh, x, 0), ref)


@pytest.mark.parametrize("m", [1, 4, 12])
def test_shared_blocks_large_batch_chunks(amp, oracle, m):
    """k large enough that x~ does not fit in one chunk at m = 12 and every block is shared by
    several CTAs."""
    trellis, suh, svh, x = make_linear(6144, 384, 4, seed=5200 + m, m=m)
    ref = oracle.linear(x, trellis, suh, svh, 0, fp32_out=True)
    check_close(run_gemm(amp, trellis, suh, svh, x, 0), ref)
    check_close(run_gemm(amp, trellis, suh, svh, x, 0, split=11, xgroups=4), ref)


def test_mgemm_multi_and_sliced(amp, oracle):
    """Bundles (models.uc multi / sliced): gate|up stacked, q|k|v sliced by the gcd of the widths,
    each slice with its own suh source; results equal the separate linears'."""
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
    sl = Sliced([q, kk, v], outs)
    assert sl.width == 256 and sl.slices == 6
    sl.run(xd)
    torch.cuda.synchronize()
    for o, (t, su, sv) in zip(outs, (q_np, k_np, v_np)):
        check_close(o[0].cpu().numpy(), oracle.linear(x, t, su, sv, 0, fp32_out=True))


@pytest.mark.parametrize("m,bf16", [(40, False), (300, False), (130, True)])
def test_mgemm_bundles_above_16_rows(amp, oracle, m, bf16):
    """The same bundles at prefill row counts: one tensor-core grid over all slices (pair form
    for widths that are multiples of 256, single-CTA form for 128). Checked against the oracle and,
    bit for bit, against separate exl3_gemm calls (same rotation, same tiles)."""
    from ampstein_b200.models import LinearEXL3, Multi, Sliced
    k = 512
    rng = np.random.default_rng(78 + m)
    x = rng.standard_normal((m, k)).astype(np.float32)
    xt = torch.from_numpy(x).cuda().to(torch.bfloat16 if bf16 else torch.float16)
    x = xt.float().cpu().numpy().astype(np.float16)   # what the kernel sees (bf16 values are exact in fp16 here)
    xd = xt.reshape(1, m, k)

    def lin(n, seed, K=4):
        trellis, suh, svh, _ = make_linear(k, n, K, seed=seed)
        return (trellis, suh, svh), LinearEXL3(dev(trellis), dev(suh), dev(svh))

    def separate(w, n):
        y = torch.empty((m, n), dtype=torch.float16, device="cuda")
        amp.exl3_gemm(xt, w.trellis, y, w.suh, w.svh)
        return y

    (g_np, g), (u_np, u) = lin(768, 11, 3), lin(768, 12, 3)
    out = torch.full((2, m, 768), float("nan"), dtype=torch.float16, device="cuda")
    Multi([g, u], out).run(xd)
    torch.cuda.synchronize()
    for i, ((t, su, sv), w) in enumerate(((g_np, g), (u_np, u))):
        check_close(out[i].cpu().numpy(), oracle.linear(x, t, su, sv, 0, fp32_out=True))
        assert torch.equal(out[i], separate(w, 768))

    for widths in ((1024, 256, 256), (384, 128, 128)):
        parts = [lin(n, 20 + i + n) for i, n in enumerate(widths)]
        outs = [torch.full((1, m, n), float("nan"), dtype=torch.float16, device="cuda") for n in widths]
        sl = Sliced([p[1] for p in parts], outs)
        assert sl.width == min(widths)
        sl.run(xd)
        torch.cuda.synchronize()
        for o, ((t, su, sv), w), n in zip(outs, parts, widths):
            check_close(o[0].cpu().numpy(), oracle.linear(x, t, su, sv, 0, fp32_out=True))
            assert torch.equal(o[0], separate(w, n))
    assert gemm_status() == 0


@pytest.mark.parametrize("m,K,cb", [(5, 4, 0), (8, 5, 0), (8, 3, 2), (13, 4, 1), (16, 6, 0)])
def test_rows_5_to_16_with_and_without_the_rotation_scratch(amp, oracle, m, K, cb):
    """From five rows on, exl3_gemm with A_had rotates the input once in a launch of its own; without
    A_had every CTA rotates its rows. Same arithmetic: the results must agree bit for bit, for a
    single matrix and for a sliced bundle, and match the oracle."""
    from ampstein_b200 import _lib
    from ampstein_b200.models import LinearEXL3, Sliced
    k, n = 1536, 1024
    trellis, suh, svh, x = make_linear(k, n, K, seed=6100 + m + K, m=m)
    t, su, sv, xx = dev(trellis), dev(suh), dev(svh), dev(x)
    st = torch.cuda.current_stream().cuda_stream
    outs = []
    for scratch in (None, torch.empty((m, k), dtype=torch.float16, device="cuda")):
        y = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        _lib.call("amp_exl3_gemm", xx.data_ptr(), t.data_ptr(), y.data_ptr(), su.data_ptr(),
                  scratch.data_ptr() if scratch is not None else None, sv.data_ptr(), m, k, n, K, cb, 0, st)
        outs.append(y)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])
    check_close(outs[1].cpu().numpy(), oracle.linear(x, trellis, suh, svh, cb, fp32_out=True))

    widths = (512, 256, 256)
    parts = []
    for i, w in enumerate(widths):
        tr, s_u, s_v, _ = make_linear(k, w, K, seed=6200 + i + m)
        parts.append(((tr, s_u, s_v), LinearEXL3(dev(tr), dev(s_u), dev(s_v), mul1=(cb == 2), mcg=(cb == 1))))
    xd = xx.reshape(1, m, k)
    res = []
    for scratch in (False, True):
        o = [torch.full((1, m, w), float("nan"), dtype=torch.float16, device="cuda") for w in widths]
        sl = Sliced([p[1] for p in parts], o)
        a = sl.linears[0]
        amp.mgemm(xd, sl.B, sl.carrier, sl.suh, torch.empty((3, m, k), dtype=torch.float16, device="cuda") if scratch else None,
                  sl.svh, a.K, a.mcg, a.mul1, sl.opts)
        res.append(o)
    torch.cuda.synchronize()
    for o0, o1, ((tr, s_u, s_v), _) in zip(res[0], res[1], parts):
        assert torch.equal(o0, o1)
        check_close(o1[0].cpu().numpy(), oracle.linear(x, tr, s_u, s_v, cb, fp32_out=True))


@pytest.mark.parametrize("k,n,K", [(256, 128, 4), (1024, 768, 3), (4096, 1024, 4), (1536, 512, 5), (2048, 256, 6), (512, 384, 1),
                                   (14336, 512, 4)])
def test_int8_activation_gemv_mul1(amp, oracle, k, n, K):
    """One row, mul1 codebook, int8 switch on: the kernel quantises the rotated input per 128 rows of
    k and sums bytesum * code exactly, so it must agree closely with the CPU restatement of that
    arithmetic (1e-4 of the largest output: fp32 summation order is all that differs) and stay
    within the reference's figure for this form against the fp32-accumulated linear (relative
    rms < 1e-2; src/torch/amp_torch.cpp:12974-12981 quotes ~8e-3). Bit widths above the limit, two
    rows and the switch set to 0 take the fp16 kernel."""
    from ampstein_b200 import _lib
    trellis, suh, svh, x = make_linear(k, n, K, seed=9300 + K + n, m=2)
    t, su, sv = dev(trellis), dev(suh), dev(svh)
    x1 = x[:1]
    ref8 = oracle.linear_int8(x1, trellis, suh, svh, fp32_out=True)
    ref = oracle.linear(x1, trellis, suh, svh, 2, fp32_out=True)

    def run(xx, mode, max_k=6):
        old = _lib.lib().amp_exl3_set_int8_gemv(mode, max_k)
        try:
            y = torch.full((xx.shape[0], n), float("nan"), dtype=torch.float32, device="cuda")
            amp.exl3_gemm(dev(xx), t, y, su, sv, mul1=True)
            torch.cuda.synchronize()
            return y.cpu().numpy()
        finally:
            _lib.lib().amp_exl3_set_int8_gemv(old, 6)

    got = run(x1, 2)
    assert np.all(np.isfinite(got))
    assert np.max(np.abs(got - ref8)) / np.max(np.abs(ref8)) < 1e-4
    rms = np.sqrt(np.mean((got.astype(np.float64) - ref) ** 2) / np.mean(ref.astype(np.float64) ** 2))
    assert 1e-4 < rms < 1e-2, rms                                  # really the int8 form, and within its figure
    fp = run(x1, 0)
    check_close(fp, ref)                                           # switch off: the fp16 kernel
    # mode 1, the error-feedback form: agrees with its own CPU restatement and is far closer to
    # the fp32-accumulated linear than the plain int8 form (about 15 bits of activation precision)
    ref8r = oracle.linear_int8(x1, trellis, suh, svh, fp32_out=True, residual=True)
    got_r = run(x1, 1)
    assert np.all(np.isfinite(got_r))
    assert np.max(np.abs(got_r - ref8r)) / np.max(np.abs(ref8r)) < 1e-4
    rms_r = np.sqrt(np.mean((got_r.astype(np.float64) - ref) ** 2) / np.mean(ref.astype(np.float64) ** 2))
    assert rms_r < 1e-3 and rms_r < rms / 4, (rms_r, rms)
    assert np.array_equal(run(x1, 2, max_k=K - 1), fp) if K > 1 else True    # above the bit-width limit
    both = run(x, 2)                                               # two rows: fp16 kernel
    check_close(both, oracle.linear(x, trellis, suh, svh, 2, fp32_out=True))
    if k == 1024:
        # a sliced bundle of mul1 linears at one row takes the int8 form too
        from ampstein_b200.models import LinearEXL3, Sliced
        parts = []
        for i, w in enumerate((512, 256, 256)):
            tr, s_u, s_v, _ = make_linear(k, w, K, seed=9400 + i)
            parts.append(((tr, s_u, s_v), LinearEXL3(dev(tr), dev(s_u), dev(s_v), mul1=True)))
        outs = [torch.full((1, 1, w), float("nan"), dtype=torch.float16, device="cuda") for w in (512, 256, 256)]
        old = _lib.lib().amp_exl3_set_int8_gemv(2, 6)
        try:
            Sliced([p[1] for p in parts], outs).run(dev(x1).reshape(1, 1, k))
            torch.cuda.synchronize()
        finally:
            _lib.lib().amp_exl3_set_int8_gemv(old, 6)
        for o, ((tr, s_u, s_v), _) in zip(outs, parts):
            r8 = oracle.linear_int8(x1, tr, s_u, s_v, fp32_out=True)
            assert np.max(np.abs(o[0].float().cpu().numpy() - r8)) / np.max(np.abs(r8)) < 1e-3      # fp16 output rounding


def test_gemm_more_than_16_rows(amp, oracle):
    trellis, suh, svh, x = make_linear(256, 256, 3, seed=6000, m=37)
    ref = oracle.linear(x, trellis, suh, svh, 1, fp32_out=True)
    check_close(run_gemm(amp, trellis, suh, svh, x, 1), ref)
    # the many-rows operator of the reference (exl3_gemm_recon) returns a new tensor
    y = amp.exl3_gemm_recon(dev(x), dev(trellis), dev(suh), dev(svh), 3, mcg=True)
    check_close(y.cpu().numpy(), ref)


@pytest.mark.parametrize("m,k,n,K,cb", [(1, 1024, 512, 4, 0), (3, 2048, 256, 5, 1), (8, 768, 384, 3, 2), (12, 512, 256, 6, 0),
                                        (1, 14336, 1024, 4, 0)])
def test_down_projection_with_the_activation_in_its_prologue(amp, oracle, m, k, n, K, cb):
    """exl3_gemm_silu_mul(gate, up, ...) against the two-step sequence it replaces: the oracle's
    silu_mul then linear, and this library's exl3_gemm on an activation formed by torch (fp32 math,
    rounded to fp16): same rounding points, so the bound is the linear's own."""
    trellis, suh, svh, g = make_linear(k, n, K, seed=9500 + m + K, m=m)
    u = np.random.default_rng(95 + m).standard_normal((m, k)).astype(np.float16)
    t, su, sv, gd, ud = dev(trellis), dev(suh), dev(svh), dev(g), dev(u)
    y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    amp.exl3_gemm_silu_mul(gd, ud, t, y, su, sv, mul1=(cb == 2), mcg=(cb == 1))
    a = (torch.nn.functional.silu(gd.float()) * ud.float()).to(torch.float16)
    y2 = torch.empty_like(y)
    amp.exl3_gemm(a, t, y2, su, sv, mul1=(cb == 2), mcg=(cb == 1))
    torch.cuda.synchronize()
    ref = oracle.linear(oracle.silu_mul(g, u), trellis, suh, svh, cb, fp32_out=True)
    check_close(y.cpu().numpy(), ref)
    check_close(y.cpu().numpy(), y2.cpu().numpy())


@pytest.mark.parametrize("m,k,K,cb", [(1, 1024, 4, 0), (2, 4096, 4, 0), (5, 512, 5, 2), (9, 768, 3, 1)])
def test_linears_with_the_residual_norm_in_their_prologue(amp, oracle, m, k, K, cb):
    """exl3_gemm_rms_norm_res and the bundle form against the two-step sequence they replace (the
    oracle's rms_norm_res, then linear): y bit-exact, the linears within their own bound (the scale may
    differ in its last fp32 bit: the sum of squares is added in another order)."""
    from ampstein_b200.models import LinearEXL3, Multi, Sliced
    n = 512
    trellis, suh, svh, x = make_linear(k, n, K, seed=9600 + m + K, m=m)
    rng = np.random.default_rng(96 + m)
    res = (rng.standard_normal((m, k)) * 0.5).astype(np.float16)
    w = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float16)
    eps = 1e-5
    y_ref, n_ref = oracle.rms_norm_res(x, res, w, eps)
    t, su, sv, xd, rd, wd = dev(trellis), dev(suh), dev(svh), dev(x), dev(res), dev(w)
    y = torch.full((m, k), float("nan"), dtype=torch.float16, device="cuda")
    c = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    amp.exl3_gemm_rms_norm_res(xd, rd, wd, eps, y, t, c, su, sv, mul1=(cb == 2), mcg=(cb == 1))
    torch.cuda.synchronize()
    assert np.array_equal(host16(y), y_ref.view(np.uint16))
    check_close(c.cpu().numpy(), oracle.linear(n_ref, trellis, suh, svh, cb, fp32_out=True))
    with pytest.raises(ValueError):
        amp.exl3_gemm_rms_norm_res(xd, rd, wd, eps, xd, t, c, su, sv)

    # bundles: stacked pair and a sliced triple behind the same norm
    parts = []
    for i, wd_ in enumerate((512, 256, 256, 384, 384)):
        tr, s_u, s_v, _ = make_linear(k, wd_, K, seed=9700 + i + m)
        parts.append(((tr, s_u, s_v), LinearEXL3(dev(tr), dev(s_u), dev(s_v), mul1=(cb == 2), mcg=(cb == 1))))
    x3, r3 = xd.reshape(1, m, k), rd.reshape(1, m, k)
    outs = [torch.full((1, m, wd_), float("nan"), dtype=torch.float16, device="cuda") for wd_ in (512, 256, 256)]
    y.fill_(float("nan"))
    Sliced([p[1] for p in parts[:3]], outs).run_norm(x3, r3, wd, eps, y.reshape(1, m, k))
    gu = torch.full((2, m, 384), float("nan"), dtype=torch.float16, device="cuda")
    y2 = torch.full((1, m, k), float("nan"), dtype=torch.float16, device="cuda")
    Multi([p[1] for p in parts[3:]], gu).run_norm(x3, r3, wd, eps, y2)
    torch.cuda.synchronize()
    assert np.array_equal(host16(y), y_ref.view(np.uint16)) and np.array_equal(host16(y2[0]), y_ref.view(np.uint16))
    for o, ((tr, s_u, s_v), _) in zip([o[0] for o in outs] + [gu[0], gu[1]], parts):
        check_close(o.float().cpu().numpy(), oracle.linear(n_ref, tr, s_u, s_v, cb, fp32_out=True))


@pytest.mark.parametrize("m,K,cb", [(1, 4, 0), (3, 5, 2), (8, 3, 1)])
def test_residual_norm_split_between_producer_and_consumer(amp, oracle, m, K, cb):
    """exl3_gemm_add_res (the producing linear adds its output to the residual stream and leaves block
    sums of squares) followed by exl3_gemm_normed / the bundle form (the consumer scales): against the
    oracle's sequence linear -> rms_norm_res -> linear. y bit-exact given the producer's own fp16
    output; the block sums within fp32 rounding of numpy's; the consumers within their bound."""
    from ampstein_b200.models import LinearEXL3, Multi
    k0, H, n = 768, 1024, 512
    tr0, su0, sv0, x = make_linear(k0, H, K, seed=9950 + m, m=m)
    sv0 = (sv0.astype(np.float32) / (1.2437 * np.sqrt(k0))).astype(np.float16)
    tr1, su1, sv1, _ = make_linear(H, n, K, seed=9960 + m)
    rng = np.random.default_rng(995 + m)
    h = rng.standard_normal((m, H)).astype(np.float16)
    w = (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float16)
    eps = 1e-5
    mul1, mcg = cb == 2, cb == 1
    xd, hd = dev(x), dev(h)
    # the producer's own fp16 output, from the plain entry (same kernel arithmetic)
    o = torch.empty((m, H), dtype=torch.float16, device="cuda")
    amp.exl3_gemm(xd, dev(tr0), o, dev(su0), dev(sv0), mul1=mul1, mcg=mcg)
    y = torch.full((m, H), float("nan"), dtype=torch.float16, device="cuda")
    ssq = torch.full((m, H // 128), float("nan"), dtype=torch.float32, device="cuda")
    amp.exl3_gemm_add_res(xd, dev(tr0), dev(su0), dev(sv0), hd, y, ssq, mul1=mul1, mcg=mcg)
    torch.cuda.synchronize()
    y_ref, n_ref = oracle.rms_norm_res(h, o.cpu().numpy(), w, eps)
    assert np.array_equal(host16(y), y_ref.view(np.uint16))
    want = (y_ref.astype(np.float64) ** 2).reshape(m, H // 128, 128).sum(axis=2)
    assert np.allclose(ssq.cpu().numpy(), want, rtol=1e-5)
    c = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    amp.exl3_gemm_normed(y, ssq, dev(w), eps, dev(tr1), c, dev(su1), dev(sv1), mul1=mul1, mcg=mcg)
    torch.cuda.synchronize()
    check_close(c.cpu().numpy(), oracle.linear(n_ref, tr1, su1, sv1, cb, fp32_out=True))
    # bundle form
    parts = []
    for i in range(2):
        tr, s_u, s_v, _ = make_linear(H, 384, K, seed=9970 + i + m)
        parts.append(((tr, s_u, s_v), LinearEXL3(dev(tr), dev(s_u), dev(s_v), mul1=mul1, mcg=mcg)))
    gu = torch.full((2, m, 384), float("nan"), dtype=torch.float16, device="cuda")
    Multi([p[1] for p in parts], gu).run_normed(y.reshape(1, m, H), ssq, dev(w), eps)
    torch.cuda.synchronize()
    for i, ((tr, s_u, s_v), _) in enumerate(parts):
        check_close(gu[i].float().cpu().numpy(), oracle.linear(n_ref, tr, s_u, s_v, cb, fp32_out=True))


def test_stand_alone_neighbour_kernels(amp, oracle):
    """The stand-alone residual norm, gated activation and greedy pick against the oracle / numpy, and
    the fused sequence against the unfused one built from them: same logits bits, same pick."""
    k, I, n, K = 1024, 2048, 2048, 4
    rng = np.random.default_rng(99)
    x = rng.standard_normal((2, k)).astype(np.float16)
    res = (0.5 * rng.standard_normal((2, k))).astype(np.float16)
    w = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float16)
    y, nn = amp.rms_norm_res(dev(x), dev(res), dev(w), 1e-5)
    y_ref, n_ref = oracle.rms_norm_res(x, res, w, 1e-5)
    assert np.array_equal(host16(y), y_ref.view(np.uint16))
    d = np.abs(nn.float().cpu().numpy() - n_ref.astype(np.float32))
    assert np.max(d) <= 2e-3 * np.max(np.abs(n_ref.astype(np.float32))) and np.mean(d > 0) < 0.01     # scale may differ in its last bit
    g = rng.standard_normal((2, I)).astype(np.float16)
    u = rng.standard_normal((2, I)).astype(np.float16)
    a = amp.silu_mul(dev(g), dev(u))
    d = np.abs(a.float().cpu().numpy() - oracle.silu_mul(g, u).astype(np.float32))
    assert np.max(d) <= 2e-3 and np.mean(d > 0) < 0.01                                                 # __expf against exp
    # unfused tail (norm, lm_head, pick) against the fused launch: identical logits and pick
    trellis, suh, svh, _ = make_linear(k, n, K, seed=9900)
    t, su, sv = dev(trellis), dev(suh), dev(svh)
    mk = lambda v: torch.tensor([v], dtype=torch.int64, device="cuda")
    ids1, pos1, ids2, pos2 = mk(3), mk(5), mk(3), mk(5)
    log1 = torch.zeros(8, dtype=torch.int64, device="cuda"); log2 = torch.zeros(8, dtype=torch.int64, device="cuda")
    ws1 = torch.zeros(4, dtype=torch.int32, device="cuda"); ws2 = torch.zeros(4, dtype=torch.int32, device="cuda")
    x1, r1 = dev(x[:1]), dev(res[:1])
    _, n1 = amp.rms_norm_res(x1, r1, dev(w), 1e-5)
    lg1 = torch.empty((1, n), dtype=torch.float16, device="cuda")
    amp.exl3_gemm(n1, t, lg1, su, sv)
    amp.argmax_advance(lg1, ids1, pos1, log1, ws1)
    lg2 = torch.empty((1, n), dtype=torch.float16, device="cuda")
    y2 = torch.empty((1, k), dtype=torch.float16, device="cuda")
    amp.lm_head_argmax(x1, r1, dev(w), 1e-5, y2, t, lg2, su, sv, ids2, pos2, log2, ws2)
    torch.cuda.synchronize()
    assert int(ids1.item()) == int(np.argmax(lg1.float().cpu().numpy()[0]))
    assert int(ids2.item()) == int(np.argmax(lg2.float().cpu().numpy()[0]))
    assert torch.equal(log1, log2) and int(pos1.item()) == int(pos2.item()) == 6
    check_close(lg2.cpu().numpy(), lg1.float().cpu().numpy())


def test_lm_head_with_norm_argmax_and_state_advance(amp, oracle):
    """The end of a greedy decode step in one launch against the oracle's sequence (rms_norm_res,
    linear, argmax with ties to the lowest index): three steps in a row on one state (the key and the
    block counter in ws reset themselves), a vocabulary shorter than the padded width, a log too short
    for the last position."""
    k, n, K, vocab = 1024, 4096, 6, 4000
    trellis, suh, svh, _ = make_linear(k, n, K, seed=9800)
    rng = np.random.default_rng(98)
    w = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float16)
    t, su, sv, wd = dev(trellis), dev(suh), dev(svh), dev(w)
    ids = torch.tensor([7], dtype=torch.int64, device="cuda")
    pos = torch.tensor([0], dtype=torch.int64, device="cuda")
    log = torch.full((2,), -1, dtype=torch.int64, device="cuda")
    ws = torch.zeros(4, dtype=torch.int32, device="cuda")
    logits = torch.empty((1, n), dtype=torch.float16, device="cuda")
    y = torch.empty((1, k), dtype=torch.float16, device="cuda")
    prev, want_log = 7, []
    for step in range(3):
        x = rng.standard_normal((1, k)).astype(np.float16)
        res = (0.5 * rng.standard_normal((1, k))).astype(np.float16)
        amp.lm_head_argmax(dev(x), dev(res), wd, 1e-5, y, t, logits, su, sv, ids, pos, log, ws, vocab=vocab)
        torch.cuda.synchronize()
        y_ref, n_ref = oracle.rms_norm_res(x, res, w, 1e-5)
        assert np.array_equal(host16(y), y_ref.view(np.uint16))
        got = logits.cpu().numpy()
        check_close(got, oracle.linear(n_ref, trellis, suh, svh, 0, fp32_out=True))
        valid = got[0, :vocab].astype(np.float32)
        assert int(ids.item()) == int(np.argmax(valid))            # numpy: first occurrence of the maximum
        assert int(pos.item()) == step + 1
        want_log.append(prev)
        prev = int(ids.item())
        assert ws.cpu().tolist() == [0, 0, 0, 0]
    assert log.cpu().tolist() == want_log[:2]                      # the third write fell outside the log
    # ties: equal logits resolve to the lowest index (svh = 0 makes every logit +0)
    amp.lm_head_argmax(dev(x), dev(res), wd, 1e-5, y, t, logits, su, torch.zeros_like(sv), ids, pos, log, ws, vocab=vocab)
    torch.cuda.synchronize()
    assert int(ids.item()) == 0 and int(pos.item()) == 4


def test_gemm_recon_takes_the_trellis_gemm_for_wide_weights(amp, oracle):
    """Above RECON_MM_MAX_N columns the many-rows operator is the tensor-core trellis GEMM (same bits
    as exl3_gemm); at or below it the weight is reconstructed once and multiplied by a library GEMM."""
    from ampstein_b200 import exl3
    k, n, K, rows = 256, exl3.RECON_MM_MAX_N + 256, 4, 150
    trellis, suh, svh, x = make_linear(k, n, K, seed=6250, m=rows)
    t, su, sv, xx = dev(trellis), dev(suh), dev(svh), dev(x)
    y = torch.empty((rows, n), dtype=torch.float16, device="cuda")
    amp.exl3_gemm(xx, t, y, su, sv)
    z = amp.exl3_gemm_recon(xx, t, su, sv, K)
    torch.cuda.synchronize()
    assert torch.equal(y, z)
    check_close(z.float().cpu().numpy(), oracle.linear(x, trellis, suh, svh, 0, fp32_out=True))


@pytest.mark.parametrize("rows", [200, 1100])
def test_gemm_recon_next_to_gemm(amp, oracle, rows):
    """The many-rows operator against the in-place operator on the same input, at the two row
    counts the reference's test uses for its two sub-paths (tests/exl3_recon.uc:38-52: within
    relative rms 5e-3 of each other), and both against the oracle."""
    k, n, K = 512, 768, 4
    trellis, suh, svh, x = make_linear(k, n, K, seed=6300 + rows, m=rows)
    t, su, sv, xx = dev(trellis), dev(suh), dev(svh), dev(x)
    y = torch.empty((rows, n), dtype=torch.float16, device="cuda")
    amp.exl3_gemm(xx, t, y, su, sv)
    z = amp.exl3_gemm_recon(xx, t, su, sv, K)
    torch.cuda.synchronize()
    assert gemm_status() == 0
    a, b = y.float().cpu().numpy().astype(np.float64), z.float().cpu().numpy().astype(np.float64)
    assert np.sqrt(np.mean((a - b) ** 2) / np.mean(a ** 2)) < 5e-3
    check_close(b, oracle.linear(x, trellis, suh, svh, 0, fp32_out=True))


@pytest.mark.parametrize("m", [1, 3])
def test_chain_of_layers_against_the_oracle_chain(amp, oracle, m):
    """Four layers of q|k|v (sliced bundle) -> o -> gate|up (stacked bundle) -> down, every output
    feeding the next linear as in the decode graph (the reference's tests/exl3_stack.uc chains 16
    layers of 7 linears). The oracle runs the same chain on its own intermediates; rounding
    differences pass through eight linears per path, so the bound is 1e-2 relative rms at the end and
    per layer."""
    from ampstein_b200.models import LinearEXL3, Multi, Sliced
    H, KV, I, K, layers = 512, 128, 1024, 4, 4
    rng = np.random.default_rng(64 + m)
    x = rng.standard_normal((m, H)).astype(np.float16)

    def lin(k, n, seed):
        tr, su, sv, _ = make_linear(k, n, K, seed=seed)
        sv = (sv.astype(np.float32) / (1.2437 * np.sqrt(k))).astype(np.float16)      # keep activations O(1)
        return (tr, su, sv), LinearEXL3(dev(tr), dev(su), dev(sv))

    h_ref, h = x, dev(x).reshape(1, m, H)
    for layer in range(layers):
        s0 = 7000 + 10 * layer
        (q_np, q), (k_np, kk), (v_np, v) = lin(H, H, s0), lin(H, KV, s0 + 1), lin(H, KV, s0 + 2)
        (o_np, o), (g_np, g), (u_np, u), (d_np, d) = lin(H, H, s0 + 3), lin(H, I, s0 + 4), lin(H, I, s0 + 5), lin(I, H, s0 + 6)
        outs = [torch.empty((1, m, n), dtype=torch.float16, device="cuda") for n in (H, KV, KV)]
        Sliced([q, kk, v], outs).run(h)
        a = o.forward(outs[0][0])                                   # attention stands in as the identity on q
        gu = torch.empty((2, m, I), dtype=torch.float16, device="cuda")
        Multi([g, u], gu).run(a.reshape(1, m, H))
        h = d.forward(gu[0]).reshape(1, m, H)                        # (the activation is not part of this path)
        r = oracle.linear(h_ref, *q_np, 0)
        r = oracle.linear(r, *o_np, 0)
        r = oracle.linear(r, *g_np, 0)
        h_ref = oracle.linear(r, *d_np, 0)
        torch.cuda.synchronize()
        got, ref = h[0].float().cpu().numpy().astype(np.float64), h_ref.astype(np.float64)
        assert np.all(np.isfinite(got))
        assert np.sqrt(np.mean((got - ref) ** 2) / np.mean(ref ** 2)) < 1e-2, layer


def gemm_status():
    from ampstein_b200 import _lib
    st = ctypes.c_int(-1)
    _lib.call("amp_exl3_gemm_status", ctypes.byref(st))
    return st.value


@pytest.mark.parametrize("m,k,n,K,cb", [(17, 128, 128, 4, 0), (200, 256, 256, 4, 0), (512, 512, 384, 3, 0),
                                        (1100, 1024, 256, 5, 0), (130, 256, 128, 2, 1), (96, 384, 256, 6, 2),
                                        (640, 256, 256, 8, 0), (300, 128, 256, 1, 0)])
def test_prefill_gemm_tensor_core(amp, oracle, m, k, n, K, cb):
    """More than 16 rows: x~ by the Hadamard kernel, weights decoded into shared memory, tcgen05
    MMA with fp32 accumulators in tensor memory; ragged row counts included."""
    trellis, suh, svh, x = make_linear(k, n, K, seed=7000 + m + K, m=m)
    svh = (svh.astype(np.float32) / (1.2437 * np.sqrt(k))).astype(np.float16)
    ref = oracle.linear(x, trellis, suh, svh, cb, fp32_out=True)
    got = run_gemm(amp, trellis, suh, svh, x, cb)
    assert gemm_status() == 0
    check_close(got, ref)
    got32 = run_gemm(amp, trellis, suh, svh, x, cb, fp32=True)
    assert gemm_status() == 0
    check_close(got32, ref)


@pytest.mark.parametrize("mode", [2, 3])
@pytest.mark.parametrize("m,k,n,K,cb", [(600, 256, 256, 4, 0), (257, 512, 512, 3, 0), (1024, 384, 256, 5, 1),
                                        (100, 128, 256, 6, 2), (513, 256, 512, 8, 0), (129, 1024, 256, 7, 0)])
def test_prefill_gemm_cta_pairs(amp, oracle, m, k, n, K, cb, mode):
    """The pair form (two CTAs per 512 or 256 tokens x 256 columns, tcgen05 cta_group::2), forced
    for small shapes: ragged token counts, a second CTA with few or no rows, several k steps,
    three- and four-stage pipelines (bit widths above and below 6)."""
    from ampstein_b200 import _lib
    trellis, suh, svh, x = make_linear(k, n, K, seed=7400 + m + K, m=m)
    svh = (svh.astype(np.float32) / (1.2437 * np.sqrt(k))).astype(np.float16)
    ref = oracle.linear(x, trellis, suh, svh, cb, fp32_out=True)
    old = _lib.lib().amp_exl3_set_gemm_pair(mode)
    try:
        got = run_gemm(amp, trellis, suh, svh, x, cb)
        assert gemm_status() == 0
        check_close(got, ref)
        got32 = run_gemm(amp, trellis, suh, svh, x, cb, fp32=True)
        assert gemm_status() == 0
        check_close(got32, ref)
    finally:
        _lib.lib().amp_exl3_set_gemm_pair(old)


@pytest.mark.parametrize("k,n,K", [(4096, 4096, 5), (14336, 4096, 4), (4096, 14336, 3)])
def test_prefill_gemm_bench_shapes_repeatable(amp, k, n, K):
    """The benchmark's prefill shapes (2048 tokens) through the default dispatch, i.e. the pair
    form: twelve launches must agree bit for bit (the two CTAs of a pair hand stages to each other
    through shared-memory barriers; a hand-off that came too early would show as a difference
    between launches), the single-CTA form must agree within rounding, and both must agree with
    "reconstruct, then an fp32 matmul of the rotated input" computed by other kernels."""
    from ampstein_b200 import _lib
    m = 2048
    g = torch.Generator(device="cuda").manual_seed(9100 + K)
    t = torch.randint(-32768, 32767, (k // 16, n // 16, 16 * K), dtype=torch.int16, device="cuda", generator=g)
    suh = (torch.randint(0, 2, (k,), device="cuda", generator=g) * 2 - 1).to(torch.float16)
    svh = ((torch.randint(0, 2, (n,), device="cuda", generator=g) * 2 - 1) / (1.2437 * np.sqrt(k))).to(torch.float16)
    x = torch.randn((m, k), device="cuda", generator=g).to(torch.float16)
    outs = []
    for _ in range(12):
        y = torch.empty((m, n), dtype=torch.float16, device="cuda")
        amp.exl3_gemm(x, t, y, suh, svh)
        outs.append(y)
    torch.cuda.synchronize()
    assert gemm_status() == 0
    for y in outs[1:]:
        assert torch.equal(y, outs[0])
    # the releasing form of the pair's remote arrival must give the same bits as the relaxed default
    prev = _lib.lib().amp_exl3_set_gemm_relay_release(1)
    try:
        for _ in range(12):
            y = torch.empty((m, n), dtype=torch.float16, device="cuda")
            amp.exl3_gemm(x, t, y, suh, svh)
            assert torch.equal(y, outs[0])
    finally:
        _lib.lib().amp_exl3_set_gemm_relay_release(prev)
    assert gemm_status() == 0
    old = _lib.lib().amp_exl3_set_gemm_pair(0)
    try:
        y1 = torch.empty((m, n), dtype=torch.float16, device="cuda")
        amp.exl3_gemm(x, t, y1, suh, svh)
        torch.cuda.synchronize()
    finally:
        _lib.lib().amp_exl3_set_gemm_pair(old)
    assert gemm_status() == 0
    # other kernels: rotation of the input, reconstruct of the weight, fp32 matmul, rotation of the output
    xt = torch.empty_like(x)
    amp.had_r_128(x, xt, pre_scale=suh)
    w = torch.empty((k, n), dtype=torch.float16, device="cuda")
    amp.exl3_reconstruct(w, t, K)
    acc = xt.float() @ w.float()
    ref = torch.empty_like(acc)
    amp.had_r_128(acc, ref, post_scale=svh)
    ref = ref.cpu().numpy()
    check_close(outs[0].float().cpu().numpy(), ref)
    check_close(y1.float().cpu().numpy(), ref)
    check_close(y1.float().cpu().numpy(), outs[0].float().cpu().numpy())


def test_prefill_gemm_bf16_activations(amp, oracle):
    """bf16 activations (the prefill configuration): the oracle consumes the bf16 values exactly,
    with the fp32 input scale the bf16 form uses."""
    k, n, K, m = 512, 256, 4, 257
    trellis, suh, svh, _ = make_linear(k, n, K, seed=7100)
    svh = (svh.astype(np.float32) / (1.2437 * np.sqrt(k))).astype(np.float16)
    xb = torch.randn((m, k), generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    x32 = xb.float().numpy()
    # oracle: rotate in fp32 (bf16 is a subset of fp32), then the usual chain on the rotated input
    xt = oracle.had_ff(x32 * suh.astype(np.float32)[None, :]).astype(np.float16)
    what = oracle.reconstruct(trellis, 0)
    acc = oracle.matmul_f32(xt, what)
    ref = oracle.had_ff(acc, post=svh)
    out = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    amp.exl3_gemm(xb.cuda(), dev(trellis), out, dev(suh), dev(svh))
    torch.cuda.synchronize()
    assert gemm_status() == 0
    check_close(out.cpu().numpy(), ref)


def test_linearity_and_determinism_at_full_size(amp):
    """Size-independent properties at the benchmark's shapes: exact scaling by two, bitwise
    reproducibility across launches."""
    trellis, suh, svh, x = make_linear(4096, 14336, 4, seed=77, m=4)
    a = run_gemm(amp, trellis, suh, svh, x, 0, fp32=True)
    b = run_gemm(amp, trellis, suh, svh, x, 0, fp32=True)
    assert np.array_equal(a, b)
    c = run_gemm(amp, trellis, suh, svh, (x * np.float16(2)), 0, fp32=True)
    assert np.array_equal(c, 2.0 * a)


def test_reference_kernels_agree_when_built(amp, oracle):
    """When the reference's own reconstruct / Hadamard kernels were compiled (oracle/_ref), run
    them on the same inputs: bit-exact three ways (reference, oracle, this library)."""
    import os
    from conftest import ROOT
    so = os.path.join(ROOT, "oracle", "_ref", "libexl3_ref.so")
    if not os.path.exists(so):
        pytest.skip("reference kernels not built")
    R = ctypes.CDLL(so)
    for K, cb in [(2, 1), (4, 0), (6, 2)]:
        trellis, suh, svh, x = make_linear(256, 256, K, seed=8000 + K, m=4)
        t = dev(trellis)
        ref = torch.empty((256, 256), dtype=torch.float16, device="cuda")
        assert R.ref_reconstruct(ctypes.c_void_p(ref.data_ptr()), ctypes.c_void_p(t.data_ptr()), 256, 256, K, cb, 0) == 0
        mine = torch.empty_like(ref)
        amp.exl3_reconstruct(mine, t, K, mul1=(cb == 2), mcg=(cb == 1))
        torch.cuda.synchronize()
        assert np.array_equal(host16(ref), host16(mine))
        assert np.array_equal(host16(ref), oracle.reconstruct(trellis, cb).view(np.uint16))
        refh = torch.empty_like(ref)
        assert R.ref_reconstruct_had(ctypes.c_void_p(refh.data_ptr()), ctypes.c_void_p(t.data_ptr()),
                                     ctypes.c_void_p(dev(suh).data_ptr()), ctypes.c_void_p(dev(svh).data_ptr()),
                                     256, 256, K, cb, 0) == 0
        mineh = torch.empty_like(ref)
        amp.exl3_reconstruct_had(mineh, t, dev(suh), dev(svh), K, mul1=(cb == 2), mcg=(cb == 1))
        torch.cuda.synchronize()
        assert np.array_equal(host16(refh), host16(mineh))


@pytest.mark.parametrize("K", [3, 4, 5])
def test_shards_cut_on_the_device_are_the_host_slices(K):
    """amp_exl3_shard_cols / amp_exl3_shard_rows (load path): byte moves, bit for bit the narrow + cat
    of the reference's sub_columns / rows (src/ucode/ampstein/models.uc:440-562), several ranges in
    one launch, and the sharded linears still give the full product's columns / partial sums."""
    import ampstein_b200 as amp
    from ampstein_b200.models import LinearEXL3, cols, rows
    k, n = 512, 1024
    trellis, suh, svh, x = make_linear(k, n, K, seed=9100 + K, m=2)
    t, s, v = dev(trellis), dev(suh), dev(svh)
    ranges = [(256, 128), (0, 256), (768, 256)]
    tr, sv = amp.exl3_shard_cols(t, v, ranges)
    torch.cuda.synchronize()
    want_t = np.concatenate([trellis[:, a // 16:(a + ln) // 16] for a, ln in ranges], axis=1)
    want_v = np.concatenate([svh[a:a + ln] for a, ln in ranges])
    assert np.array_equal(tr.cpu().numpy().view(np.uint16), want_t.view(np.uint16))
    assert np.array_equal(sv.cpu().numpy().view(np.uint16), want_v.view(np.uint16))
    tr2, su2 = amp.exl3_shard_rows(t, s, 128, 256)
    torch.cuda.synchronize()
    assert np.array_equal(tr2.cpu().numpy().view(np.uint16), trellis[8:24].view(np.uint16))
    assert np.array_equal(su2.cpu().numpy().view(np.uint16), suh[128:384].view(np.uint16))
    # through the model layer: column shards give the columns, row shards sum to the whole
    lin = LinearEXL3(t, s, v)
    xd = dev(x)
    full = lin.forward(xd).float().cpu().numpy()
    part = cols(lin, ranges).forward(xd).float().cpu().numpy()
    want = np.concatenate([full[:, a:a + ln] for a, ln in ranges], axis=1)
    assert np.max(np.abs(part - want)) / np.max(np.abs(full)) < 2e-3       # (the k split of the launch may differ)
    halves = sum(rows(lin, k0, 256).forward(xd[:, k0:k0 + 256].contiguous()).float().cpu().numpy() for k0 in (0, 256))
    assert np.max(np.abs(halves - full)) / np.max(np.abs(full)) < 1e-2
    for bad in ([(64, 128)], [(0, 100)], [(1024, 128)], []):
        with pytest.raises(ValueError):
            amp.exl3_shard_cols(t, v, bad)
    with pytest.raises(ValueError):
        amp.exl3_shard_rows(t, s, 64, 128)
