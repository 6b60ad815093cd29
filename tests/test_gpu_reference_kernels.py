"""The reference's own GPU kernels (exl3_gemm dispatch with its GEMV and block-pipelined GEMM
kernels, exl3_mgemm, exl3_moe_coop), compiled unmodified for sm_100a into oracle/_ref, run next
to this library on identical inputs: a second oracle (outputs within 1e-2 of the fp32-accumulated
CPU oracle and of each other; the fused MoE within the 0.02 of the reference's own
tests/moe_mixed.uc) and the bar for the timing table (`-s` prints it; with AMP_RESULTS_DIR set it is
also written there as ref_kernel_timing.json). Skipped when the reference library was not built."""
import ctypes
import json
import os

import numpy as np
import pytest

from conftest import ROOT, make_linear
import ref_kernels

torch = pytest.importorskip("torch")
pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_kernels.available(), reason="reference kernels not built")]


def dev(a):
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel(got, ref):
    got, ref = got.astype(np.float64), ref.astype(np.float64)
    return np.max(np.abs(got - ref)) / np.max(np.abs(ref))


@pytest.fixture(scope="module")
def amp():
    import ampstein_b200
    return ampstein_b200


@pytest.mark.parametrize("k,n,K,m", [(4096, 4096, 4, 1), (4096, 1024, 4, 3), (14336, 4096, 4, 1), (4096, 2048, 6, 1),
                                     (5120, 6144, 5, 8), (1024, 768, 3, 16), (512, 256, 8, 2),
                                     (1024, 512, 4, 64), (512, 768, 5, 200)])
def test_gemm_dispatch_agrees(amp, oracle, k, n, K, m):
    trellis, suh, svh, x = make_linear(k, n, K, seed=k + n + K + m, m=m)
    svh = (svh.astype(np.float32) / (1.2437 * np.sqrt(k))).astype(np.float16)
    t, su, sv, xx = dev(trellis), dev(suh), dev(svh), dev(x)
    ref_out = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    a_had = torch.empty_like(xx)
    shape_idx = ref_kernels.gemm(xx, t, ref_out, su, sv, a_had)
    mine = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    amp.exl3_gemm(xx, t, mine, su, sv)
    torch.cuda.synchronize()
    cpu = oracle.linear(x, trellis, suh, svh, 0, fp32_out=True)
    e_ref, e_mine, e_pair = rel(ref_out.cpu().numpy(), cpu), rel(mine.cpu().numpy(), cpu), rel(mine.cpu().numpy(), ref_out.cpu().numpy())
    assert e_ref < 1e-2 and e_mine < 1e-2 and e_pair < 1e-2, (shape_idx, e_ref, e_mine, e_pair)


@pytest.mark.parametrize("k,n,K", [(4096, 4096, 4), (4096, 1024, 3), (14336, 4096, 4), (2048, 1024, 6)])
def test_int8_gemv_next_to_the_reference_int8_kernel(amp, oracle, k, n, K):
    """mul1 codebook, one row: the reference's dispatcher takes its int8-activation GEMV by default
    (exl3_gemm.cu:188-196); so does this library. Both quantise the activations (with different
    scale granularity), so they are compared through the fp32-accumulated oracle: each within
    relative rms 1e-2 of it, and of each other."""
    from ampstein_b200 import _lib
    trellis, suh, svh, x = make_linear(k, n, K, seed=3 * k + n + K, m=1)
    svh = (svh.astype(np.float32) / np.sqrt(k)).astype(np.float16)
    t, su, sv, xx = dev(trellis), dev(suh), dev(svh), dev(x)
    ref_out = torch.full((1, n), float("nan"), dtype=torch.float16, device="cuda")
    a_had = torch.empty_like(xx)
    ref_kernels.gemm(xx, t, ref_out, su, sv, a_had, cb=2)
    mine = torch.full((1, n), float("nan"), dtype=torch.float16, device="cuda")
    old = _lib.lib().amp_exl3_set_int8_gemv(2, 6)
    try:
        amp.exl3_gemm(xx, t, mine, su, sv, mul1=True)
        torch.cuda.synchronize()
    finally:
        _lib.lib().amp_exl3_set_int8_gemv(old, 6)
    cpu = oracle.linear(x, trellis, suh, svh, 2, fp32_out=True).astype(np.float64)

    def rms(a, b):
        return np.sqrt(np.mean((a.astype(np.float64) - b) ** 2) / np.mean(b ** 2))

    e_ref, e_mine = rms(ref_out.cpu().numpy(), cpu), rms(mine.cpu().numpy(), cpu)
    e_pair = rms(mine.cpu().numpy(), ref_out.cpu().numpy().astype(np.float64))
    assert e_ref < 1.2e-2 and e_mine < 1e-2 and e_pair < 1.6e-2, (e_ref, e_mine, e_pair)


def moe_case(T, E, Hi, I, Ho, K, topk, seed):
    from test_gpu_moe import make_experts
    ex = make_experts(E, Hi, I, Ho, K, seed=seed)
    rng = np.random.default_rng(T + seed)
    x = rng.standard_normal((T, Hi)).astype(np.float16)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    sel = np.argsort(-logits, axis=1)[:, :topk].astype(np.int64)
    w = np.take_along_axis(logits, sel, axis=1)
    w = np.exp(w - w.max(axis=1, keepdims=True))
    rw = (w / w.sum(axis=1, keepdims=True)).astype(np.float16)
    return ex, x, sel, rw


def ref_moe(amp, ex, x, sel, rw, Hi, I, Ho, K, rows_max=16):
    """The reference's exl3_moe_coop on device copies of the experts; returns (out, call)."""
    T, topk = sel.shape
    keep = []

    def table(name, idx):
        ptrs = []
        for e in ex:
            t = dev(e[name][idx])
            keep.append(t)
            ptrs.append(t.data_ptr())
        return amp.ptr_array(ptrs)

    tabs = [table(n, i) for n in ("gate", "up", "down") for i in (0, 1, 2)]
    slots = rows_max * topk
    z = lambda shape, dt: torch.zeros(shape, dtype=dt, device="cuda")
    sc = dict(had_g=z((slots, Hi), torch.float16), had_u=z((slots, Hi), torch.float16), gu_g=z((slots, I), torch.float16),
              gu_u=z((slots, I), torch.float16), act_out=z((slots, I), torch.float16), d_out=z((slots, Ho), torch.float32))
    ctr_len = slots * (I // 128) + rows_max * (Ho // 128) + 2 + (slots + 1) + slots
    ctr = z((ctr_len,), torch.int32)
    out = torch.full((rows_max, Hi), float("nan"), dtype=torch.float32, device="cuda")
    xd, seld, rwd = dev(x), dev(sel), dev(rw)
    a = ref_kernels.RefMoeArgs()
    a.x, a.bsz, a.H, a.x_stride = xd.data_ptr(), T, Hi, Hi
    a.sel, a.rw, a.topk = seld.data_ptr(), rwd.data_ptr(), topk
    a.experts, a.Hi, a.I, a.Ho = len(ex), Hi, I, Ho
    for i, t in enumerate(tabs):
        a.tables[i] = t.data_ptr()
    a.K, a.cb, a.act, a.act_limit, a.gated = K, 0, 0, 0.0, 1
    for key, t in sc.items():
        setattr(a, key, t.data_ptr())
    a.slots_max, a.rows_max, a.ctr, a.ctr_len, a.out, a.H_out = slots, rows_max, ctr.data_ptr(), ctr_len, out.data_ptr(), Hi
    keep += [tabs, sc, ctr, xd, seld, rwd]

    def call():
        assert ref_kernels.lib().ref_exl3_moe_coop(ctypes.byref(a), 0) == 0

    return out, call, keep


@pytest.mark.parametrize("T,E,Hi,I,Ho,K,topk", [(1, 16, 256, 256, 256, 3, 4), (3, 16, 256, 256, 256, 3, 4), (8, 16, 256, 256, 256, 4, 4),
                                                (16, 24, 512, 256, 512, 3, 8), (4, 128, 2048, 768, 2048, 3, 8)])
def test_fused_moe_agrees(amp, oracle, T, E, Hi, I, Ho, K, topk):
    """Pins the CPU restatement of the fused MoE to the reference's kernels (tolerance of the
    reference's own test, tests/moe_mixed.uc:59-133: 0.02) and this library to both."""
    from test_gpu_moe import build_cfg
    ex, x, sel, rw = moe_case(T, E, Hi, I, Ho, K, topk, seed=4000 + E)
    out_ref, call, keep = ref_moe(amp, ex, x, sel, rw, Hi, I, Ho, K)
    call()
    cfg = build_cfg(amp, ex, Hi, I, Ho, Hi, K, 16, topk)
    amp.moe_coop(dev(x), dev(sel), dev(rw), cfg)
    torch.cuda.synchronize()
    cpu = oracle.moe_coop(x, sel, rw, ex)
    r, mine = out_ref[:T].cpu().numpy(), cfg["out"][:T].cpu().numpy()
    assert rel(r, cpu) < 2e-2 and rel(mine, cpu) < 1e-2 and rel(mine, r) < 2e-2, (rel(r, cpu), rel(mine, cpu), rel(mine, r))


def graph_time_us(fn_list, reps=20):
    """Average time of one call when the calls of fn_list run back to back inside one CUDA graph."""
    g, s = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(s):
        for f in fn_list:
            f()
    torch.cuda.synchronize()
    with torch.cuda.stream(s), torch.cuda.graph(g, stream=s):
        for f in fn_list:
            f()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * len(fn_list))


@pytest.mark.timeout(600)
def test_timing_table(amp):
    """This library next to the reference's kernels on the same GPU: the decode step's launches
    (single matrices through exl3_gemm, the q|k|v and gate|up bundles through exl3_mgemm), the
    5-bit stack's shapes, and the fused MoE at 1 / 4 / 16 tokens. Weights rotate through more than
    the L2 holds. Asserts only that both ran; the numbers are printed and saved."""
    from ampstein_b200.models import LinearEXL3, Multi, Sliced
    rows = []
    g = torch.Generator(device="cuda").manual_seed(5)

    def lin(k, n, K):
        t = torch.randint(-32768, 32767, (k // 16, n // 16, 16 * K), dtype=torch.int16, device="cuda", generator=g)
        sg = lambda c: (torch.randint(0, 2, (c,), device="cuda", generator=g) * 2 - 1).to(torch.float16)
        return LinearEXL3(t, sg(k), (sg(n) / (1.2437 * np.sqrt(k))).to(torch.float16))

    for name, k, n, K, m in [("o 4096x4096 K4", 4096, 4096, 4, 1), ("down 14336x4096 K4", 14336, 4096, 4, 1),
                             ("lm_head 4096x128256 K6", 4096, 128256, 6, 1), ("tp5 o 6144x5120 K5", 6144, 5120, 5, 1),
                             ("tp5 down 25600x5120 K5", 25600, 5120, 5, 1), ("tp5 down 25600x5120 K5 m8", 25600, 5120, 5, 8)]:
        nset = 2 if k * n > 2e8 else max(2, int(3e8 // (k * n * K // 8)))
        ls = [lin(k, n, K) for _ in range(nset)]
        x = torch.randn((m, k), device="cuda", generator=g).to(torch.float16)
        y = torch.empty((m, n), dtype=torch.float16, device="cuda")
        a_had = torch.empty_like(x)
        ours = graph_time_us([lambda L=L: amp.exl3_gemm(x, L.trellis, y, L.suh, L.svh) for L in ls])
        idx = ref_kernels.gemm(x, ls[0].trellis, y, ls[0].suh, ls[0].svh, a_had)
        ref = graph_time_us([lambda L=L: ref_kernels.gemm(x, L.trellis, y, L.suh, L.svh, a_had) for L in ls])
        rows.append(dict(case=name, ours_us=round(ours, 2), reference_us=round(ref, 2), reference_kernel=idx,
                         weight_mb=round(k * n * K / 8e6, 1)))
        del ls
        torch.cuda.empty_cache()

    # mul1 codebook, one row: both libraries take their int8-activation GEMV
    from ampstein_b200 import _lib as _amp_lib
    old_i8 = _amp_lib.lib().amp_exl3_set_int8_gemv(2, 6)
    try:
        for name, k, n, K in [("o 4096x4096 K4 mul1 (int8 activations)", 4096, 4096, 4), ("down 14336x4096 K4 mul1 (int8 activations)", 14336, 4096, 4),
                              ("lm_head 4096x128256 K6 mul1 (int8 activations)", 4096, 128256, 6)]:
            nset = 2 if k * n > 2e8 else max(2, int(3e8 // (k * n * K // 8)))
            ls = [lin(k, n, K) for _ in range(nset)]
            x = torch.randn((1, k), device="cuda", generator=g).to(torch.float16)
            y = torch.empty((1, n), dtype=torch.float16, device="cuda")
            a_had = torch.empty_like(x)
            ours = graph_time_us([lambda L=L: amp.exl3_gemm(x, L.trellis, y, L.suh, L.svh, mul1=True) for L in ls])
            idx = ref_kernels.gemm(x, ls[0].trellis, y, ls[0].suh, ls[0].svh, a_had, cb=2)
            ref = graph_time_us([lambda L=L: ref_kernels.gemm(x, L.trellis, y, L.suh, L.svh, a_had, cb=2) for L in ls])
            rows.append(dict(case=name, ours_us=round(ours, 2), reference_us=round(ref, 2), reference_kernel=idx,
                             weight_mb=round(k * n * K / 8e6, 1)))
            del ls
            torch.cuda.empty_cache()
    finally:
        _amp_lib.lib().amp_exl3_set_int8_gemv(old_i8, 6)

    # prefill: the layer's four shapes at 2048 fp16 tokens. At this row count the reference does not
    # run its trellis GEMM but reconstructs the original-basis weight (its reconstruct_had kernel)
    # and multiplies with cuBLAS accumulating in fp16 (torch_exl3_gemm_recon, rows >= 2048:
    # src/torch/amp_torch.cpp:11211-11214, recon_mm :11096-11125); its GEMM kernel is not timed
    # here: without a tuning cache it first benchmarks every tile shape on 2..125 SMs.
    so = os.path.join(ROOT, "oracle", "_ref", "libexl3_ref.so")
    if os.path.exists(so):
        import ctypes
        R = ctypes.CDLL(so)
        M = 2048
        vp = ctypes.c_void_p
        acc16 = torch.backends.cuda.matmul.allow_fp16_accumulation
        torch.backends.cuda.matmul.allow_fp16_accumulation = True
        try:
            for name, k, n, K in [("prefill 2048 x (4096x4096 K5)", 4096, 4096, 5), ("prefill 2048 x (4096x1024 K5)", 4096, 1024, 5),
                                  ("prefill 2048 x (4096x14336 K3)", 4096, 14336, 3), ("prefill 2048 x (14336x4096 K4)", 14336, 4096, 4)]:
                ls = [lin(k, n, K) for _ in range(2)]
                x = torch.randn((M, k), device="cuda", generator=g).to(torch.float16)
                y = torch.empty((M, n), dtype=torch.float16, device="cuda")
                w = torch.empty((k, n), dtype=torch.float16, device="cuda")
                w2 = torch.empty((k, n), dtype=torch.float16, device="cuda")
                a_had = torch.empty_like(x)
                from ampstein_b200 import _lib

                def ours_call(L):
                    # the operator of this row count (reference: torch.exl3_gemm_recon): the tensor-core trellis
                    # GEMM, or reconstruct_had + a library GEMM for narrow weights
                    amp.exl3_gemm_recon(x, L.trellis, L.suh, L.svh, K, out=y, scratch=w2)

                def ref_call(L):
                    # (the reference kernels run on the legacy default stream, so they are timed eagerly)
                    assert R.ref_reconstruct_had(vp(w.data_ptr()), vp(L.trellis.data_ptr()), vp(L.suh.data_ptr()), vp(L.svh.data_ptr()),
                                                 k, n, K, 0, 0) == 0
                    torch.mm(x, w, out=y)

                def eager_us(fn, reps=10):
                    for L in ls:
                        fn(L)
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(reps):
                        for L in ls:
                            fn(L)
                    e1.record()
                    torch.cuda.synchronize()
                    return e0.elapsed_time(e1) * 1e3 / (reps * len(ls))

                # ours inside a CUDA graph (at ~30 us per call the Python wrapper's checks, not the GPU, set the
                # pace of eager calls); the reference's shim launches on the legacy default stream and stays eager
                ours, ref = graph_time_us([lambda L=L: ours_call(L) for L in ls]), eager_us(ref_call)
                rows.append(dict(case=name, ours_us=round(ours, 2), reference_us=round(ref, 2), reference_kernel="reconstruct_had + cuBLAS (fp16 accumulate)",
                                 tflops_ours=round(2.0 * M * k * n / ours / 1e6, 1), tflops_reference=round(2.0 * M * k * n / ref / 1e6, 1)))
                del ls
                torch.cuda.empty_cache()
        finally:
            torch.backends.cuda.matmul.allow_fp16_accumulation = acc16

    # bundles: q|k|v sliced (4096 -> 4096, 1024, 1024) and gate|up stacked (4096 -> 14336 x 2), K = 4
    m, k = 1, 4096
    x3 = torch.randn((1, m, k), device="cuda", generator=g).to(torch.float16)
    for name, widths in (("q|k|v 4096x6144 K4 (sliced bundle)", (4096, 1024, 1024)), ("gate|up 4096x28672 K4 (stacked bundle)", (14336, 14336))):
        nset = 6 if sum(widths) < 10000 else 3
        sets = []
        for _ in range(nset):
            ls = [lin(k, w, 4) for w in widths]
            if len(set(widths)) == 1:
                out = torch.empty((len(ls), m, widths[0]), dtype=torch.float16, device="cuda")
                b = Multi(ls, out)
                a_had = torch.zeros((len(ls), m, k), dtype=torch.float16, device="cuda")
                rf = lambda b=b, out=out, a_had=a_had, n=len(ls), w=widths[0]: ref_kernels.mgemm(
                    x3, b.B, out, b.suh, a_had, b.svh, n, n, m, k, w, 4)
            else:
                outs = [torch.empty((1, m, w), dtype=torch.float16, device="cuda") for w in widths]
                b = Sliced(ls, outs)
                a_had = torch.zeros((len(ls), m, k), dtype=torch.float16, device="cuda")
                rf = lambda b=b, a_had=a_had, n=len(ls): ref_kernels.mgemm(
                    x3, b.B, b.carrier, b.suh, a_had, b.svh, b.slices, n, m, k, b.width, 4, opts=b.opts)
            sets.append((b, rf, ls))
        ours = graph_time_us([lambda b=b: b.run(x3) for b, _, _ in sets])
        ref = graph_time_us([rf for _, rf, _ in sets])
        rows.append(dict(case=name, ours_us=round(ours, 2), reference_us=round(ref, 2), weight_mb=round(k * sum(widths) * 4 / 8e6, 1)))
        del sets
        torch.cuda.empty_cache()

    # fused MoE, 128 experts 2048 -> 768 -> 2048 K3 top-8
    from test_gpu_moe import build_cfg
    E, Hi, I, Ho, K, topk = 128, 2048, 768, 2048, 3, 8
    ex, _, _, _ = moe_case(1, E, Hi, I, Ho, K, topk, seed=777)
    cfg = build_cfg(amp, ex, Hi, I, Ho, Hi, K, 16, topk)
    for T in (1, 4, 16):
        routes = [moe_case(T, 1, 128, 128, 128, 1, 1, seed=s) for s in ()]  # (no extra experts)
        calls_ours, calls_ref, keep = [], [], []
        for s in range(8):
            rng = np.random.default_rng(100 * T + s)
            x = rng.standard_normal((T, Hi)).astype(np.float16)
            logits = rng.standard_normal((T, E)).astype(np.float32)
            sel = np.argsort(-logits, axis=1)[:, :topk].astype(np.int64)
            w = np.take_along_axis(logits, sel, axis=1)
            rw = (np.exp(w) / np.exp(w).sum(axis=1, keepdims=True)).astype(np.float16)
            xd, sd, rd = dev(x), dev(sel), dev(rw)
            keep.append((xd, sd, rd))
            calls_ours.append(lambda xd=xd, sd=sd, rd=rd: amp.moe_coop(xd, sd, rd, cfg))
            _, call, kp = ref_moe(amp, ex, x, sel, rw, Hi, I, Ho, K)
            keep.append(kp)
            calls_ref.append(call)
        ours = graph_time_us(calls_ours)
        ref = graph_time_us(calls_ref)
        rows.append(dict(case="fused MoE 128 experts top-8 K3, %d token(s)" % T, ours_us=round(ours, 2), reference_us=round(ref, 2)))
        del keep, calls_ref
        torch.cuda.empty_cache()

    for r in rows:
        print(r)
    out_dir = os.environ.get("AMP_RESULTS_DIR")
    if out_dir and os.path.isdir(out_dir):
        json.dump(rows, open(os.path.join(out_dir, "ref_kernel_timing.json"), "w"), indent=1)
    assert all(r["ours_us"] > 0 and r["reference_us"] > 0 for r in rows)


@pytest.mark.skipif(not ref_kernels.moe_available(), reason="reference prefill MoE not built")
@pytest.mark.timeout(300)
@pytest.mark.parametrize("cbname,T", [("mcg", 512), ("mul1", 512), ("mul1", 2048)])
def test_sorted_moe_next_to_the_reference_kernel(amp, cbname, T):
    """The reference's token-sorted prefill MoE kernel (exl3_moe, instantiated for the mcg and mul1
    codebooks only) and this library's moe_fused on the same routing: 128 experts 2048 -> 768 ->
    2048 at K = 3, top-8. Outputs within 2e-2 of each other (the tolerance of the reference's fused-MoE
    tests); both timed with CUDA events. The reference is called as its own caller does
    (src/ucode/ampstein/glm5.uc:1212-1230): three row tiers for mul1, one 16-row tier for mcg, experts
    up to 256 rows, atomic accumulation (its faster mode)."""
    from test_gpu_moe import build_cfg
    E, H, I, K, topk = 128, 2048, 768, 3, 8
    cb = {"mcg": 1, "mul1": 2}[cbname]
    ex, _, _, _ = moe_case(1, E, H, I, H, K, topk, seed=888)
    rng = np.random.default_rng(T)
    x = rng.standard_normal((T, H)).astype(np.float16)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    sel = np.argsort(-logits, axis=1)[:, :topk].astype(np.int64)
    w = np.take_along_axis(logits, sel, axis=1)
    rw = (np.exp(w) / np.exp(w).sum(axis=1, keepdims=True)).astype(np.float16)
    cfg = build_cfg(amp, ex, H, I, H, H, K, 1, topk, **{cbname: True})
    cfg["I"] = I
    xd = dev(x)
    count, tok, wts = amp.moe_sort_routing(dev(sel), dev(rw), E)
    assert int(count[:E].max()) <= 256
    mine = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    ours_call = lambda: amp.moe_fused(xd, mine, count, tok, wts, cfg)
    ours_call()
    torch.cuda.synchronize()
    assert amp.moe_fused_status(cfg) == 0

    L = ref_kernels.moe_lib()
    conc = L.ref_exl3_moe_concurrency(0)
    assert conc > 0
    cap = 256
    z = lambda shape: torch.zeros(shape, dtype=torch.float16, device="cuda")
    temps = [z((conc, cap, H)), z((conc, cap, H)), z((conc, cap, I)), z((conc, cap, I))]
    ref_out = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    a = ref_kernels.RefMoeSortedArgs()
    a.y, a.out, a.count, a.tok, a.w = xd.data_ptr(), ref_out.data_ptr(), count.data_ptr(), tok.data_ptr(), wts.data_ptr()
    a.T, a.H, a.I, a.E, a.A = T, H, I, E, tok.numel()
    for i, n in enumerate(("g_trellis", "g_suh", "g_svh", "u_trellis", "u_suh", "u_svh", "d_trellis", "d_suh", "d_svh")):
        a.tables[i] = cfg[n].data_ptr()
    a.K, a.cb, a.act, a.act_limit = K, cb, 0, 0.0
    a.ts_g, a.ts_u, a.ti_g, a.ti_u = (t.data_ptr() for t in temps)
    a.conc, a.cap, a.num_active = conc, cap, -1
    tiers = [(33, cap, 64), (17, 32, 32), (1, 16, 16)] if cbname == "mul1" else [(1, cap, 16)]

    def ref_call():
        for lo, hi, mt in tiers:
            a.lo, a.hi, a.m_tile = lo, hi, mt
            assert L.ref_exl3_moe_sorted(ctypes.byref(a), 0) == 0

    torch.cuda.synchronize()
    ref_call()
    torch.cuda.synchronize()
    r, m = ref_out.cpu().numpy(), mine.cpu().numpy()
    assert np.all(np.isfinite(r)) and rel(m, r) < 2e-2, rel(m, r)

    def time_us(fn, reps=5):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    row = dict(case="token-sorted MoE 128 experts top-8 K3 %s, %d tokens" % (cbname, T),
               ours_us=round(time_us(ours_call), 1), reference_us=round(time_us(ref_call), 1), max_rel_diff=float(rel(m, r)))
    print(row)
    out_dir = os.environ.get("AMP_RESULTS_DIR")
    if out_dir and os.path.isdir(out_dir):
        with open(os.path.join(out_dir, "ref_moe_sorted_timing.jsonl"), "a") as f:
            f.write(json.dumps(row) + "\n")
