"""GPU parity at the sizes the benchmark configurations name, against the CPU oracle
(reconstruct, then an fp32-accumulated product): the 6-bit lm_head at its full width, the
tensor-parallel stack's shapes and their 2/4/8-way column / row shards (sharded by the
reference's rules, src/ucode/ampstein/qwen35_tp.uc:40-79, models.uc:527-562), the prefill GEMM
at 2048 bf16 tokens for each bit width, and the fused decode MoE at 128 experts / top-8.
Tolerance as everywhere: max |y - ref| / max |ref| < 1e-2."""
import ctypes

import numpy as np
import pytest

from conftest import make_linear

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

MAX_REL = 1e-2


def dev(a):
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def check_close(got, ref, tol=MAX_REL):
    got, ref = got.astype(np.float64), ref.astype(np.float64)
    assert np.all(np.isfinite(got))
    err = np.max(np.abs(got - ref)) / np.max(np.abs(ref))
    assert err < tol, err
    return err


@pytest.fixture(scope="module")
def amp():
    import ampstein_b200
    return ampstein_b200


def gemv(amp, trellis, suh, svh, x):
    from ampstein_b200 import _lib
    out = torch.full((x.shape[0], trellis.shape[1] * 16), float("nan"), dtype=torch.float16, device="cuda")
    amp.exl3_gemm(dev(x), dev(trellis), out, dev(suh), dev(svh))
    torch.cuda.synchronize()
    st = ctypes.c_int(-1)
    _lib.call("amp_exl3_gemv_status", ctypes.byref(st))
    assert st.value == 0
    return out.cpu().numpy()


def scaled(svh, k):
    return (svh.astype(np.float32) / (1.2437 * np.sqrt(k))).astype(np.float16)


@pytest.mark.parametrize("m", [1, 8])
def test_lm_head_full_width(amp, oracle, m):
    """4096 -> 128256 at 6 bits per weight: the largest launch of the decode step."""
    k, n, K = 4096, 128256, 6
    trellis, suh, svh, x = make_linear(k, n, K, seed=60 + m, m=m)
    svh = scaled(svh, k)
    ref = oracle.linear(x, trellis, suh, svh, 0, fp32_out=True)
    check_close(gemv(amp, trellis, suh, svh, x), ref)


@pytest.mark.parametrize("m", [1, 8])
@pytest.mark.parametrize("k,n", [(5120, 25600), (25600, 5120), (5120, 6144), (6144, 5120), (5120, 1024)])
def test_tp_stack_shapes_unsharded(amp, oracle, k, n, m):
    """The 5-bit tensor-parallel stack (hidden 5120, q 6144, k/v 1024, MLP 25600) on one GPU."""
    trellis, suh, svh, x = make_linear(k, n, 5, seed=k + n + m, m=m)
    svh = scaled(svh, k)
    check_close(gemv(amp, trellis, suh, svh, x), oracle.linear(x, trellis, suh, svh, 0, fp32_out=True))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_mlp_shards_sum_to_the_full_layer(amp, oracle, world):
    """gate (column-parallel) and down (row-parallel) of the 5-bit stack, cut by the reference's
    rules: every rank's gate shard equals the matching columns of the full product, and the ranks'
    down partials, all-reduced in fp32 in rank order and rounded once (the all-reduce's
    arithmetic), equal the full down product; batch 1 and 8."""
    from ampstein_b200.models import LinearEXL3, cols, rows, split_n
    hidden, ffn, K = 5120, 25600, 5
    ranges = split_n(ffn, 256, [1] * world)
    assert sum(w for _, w in ranges) == ffn and all(n0 % 256 == 0 and w % 256 == 0 for n0, w in ranges)
    for m in (1, 8):
        gt, gsu, gsv, x = make_linear(hidden, ffn, K, seed=700 + world + m, m=m)
        gsv = scaled(gsv, hidden)
        dt, dsu, dsv, xd = make_linear(ffn, hidden, K, seed=800 + world + m, m=m)
        dsv = scaled(dsv, ffn)
        gate = LinearEXL3(dev(gt), dev(gsu), dev(gsv))
        down = LinearEXL3(dev(dt), dev(dsu), dev(dsv))
        ref_g = oracle.linear(x, gt, gsu, gsv, 0, fp32_out=True)
        ref_d = oracle.linear(xd, dt, dsu, dsv, 0, fp32_out=True)
        parts = []
        for n0, w in ranges:
            g = cols(gate, [(n0, w)])
            assert g.out_features == w
            yg = torch.empty((m, w), dtype=torch.float16, device="cuda")
            amp.exl3_gemm(dev(x), g.trellis, yg, g.suh, g.svh)
            check_close(yg.cpu().numpy(), ref_g[:, n0:n0 + w])
            d = rows(down, n0, w)
            yd = torch.empty((m, hidden), dtype=torch.float16, device="cuda")
            amp.exl3_gemm(dev(xd[:, n0:n0 + w]), d.trellis, yd, d.suh, d.svh)
            parts.append(yd.cpu().numpy())
        torch.cuda.synchronize()
        total = oracle.allreduce_fp16(np.stack([p.reshape(-1) for p in parts])).reshape(m, hidden)
        check_close(total, ref_d)


@pytest.mark.parametrize("k,n,K", [(4096, 4096, 5), (4096, 1024, 5), (4096, 14336, 3), (14336, 4096, 4)])
def test_prefill_2048_bf16_tokens_against_the_oracle(amp, oracle, k, n, K):
    """The prefill configuration: 2048 bf16 tokens, attention linears at 5 bits, gate/up at 3,
    down at 4. The full launch runs; a sample of token rows and of whole 128-column blocks (the
    output rotation mixes a block's columns) is compared with the oracle, which consumes the bf16
    values exactly (bf16 is a subset of fp32; the bf16 form scales in fp32)."""
    from test_gpu_parity import gemm_status
    M = 2048
    trellis, suh, svh, _ = make_linear(k, n, K, seed=k + n + K)
    svh = scaled(svh, k)
    xb = torch.randn((M, k), generator=torch.Generator().manual_seed(K)).to(torch.bfloat16)
    out = torch.full((M, n), float("nan"), dtype=torch.float16, device="cuda")
    amp.exl3_gemm(xb.cuda(), dev(trellis), out, dev(suh), dev(svh))
    torch.cuda.synchronize()
    assert gemm_status() == 0
    got = out.cpu().numpy()
    assert np.all(np.isfinite(got))
    rng = np.random.default_rng(K)
    rows_s = np.sort(rng.choice(M, 48, replace=False))
    rows_s[0], rows_s[-1] = 0, M - 1
    blocks = sorted(set([0, n // 128 - 1] + list(rng.choice(n // 128, 3, replace=False))))
    xt = oracle.had_ff(xb.float().numpy()[rows_s] * suh.astype(np.float32)[None, :]).astype(np.float16)
    for b in blocks:
        sub = np.ascontiguousarray(trellis[:, b * 8:(b + 1) * 8])
        acc = oracle.matmul_f32(xt, oracle.reconstruct(sub, 0))
        ref = oracle.had_ff(acc, post=svh[b * 128:(b + 1) * 128])
        check_close(got[rows_s][:, b * 128:(b + 1) * 128], ref)


@pytest.mark.parametrize("T", [4, 16])
def test_moe_128_experts_top8(amp, oracle, T):
    """The MoE configuration at its own size: 128 experts 2048 -> 768 -> 2048 at 3 bits, top-8
    routing from seeded fp32 router logits ~ N(0,1), softmax over the selected eight."""
    from test_gpu_moe import build_cfg, make_experts
    E, Hi, I, Ho, K, topk = 128, 2048, 768, 2048, 3, 8
    ex = make_experts(E, Hi, I, Ho, K, seed=12000)
    rng = np.random.default_rng(T)
    x = rng.standard_normal((T, Hi)).astype(np.float16)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    sel = np.argsort(-logits, axis=1)[:, :topk].astype(np.int64)
    w = np.take_along_axis(logits, sel, axis=1)
    w = np.exp(w - w.max(axis=1, keepdims=True))
    rw = (w / w.sum(axis=1, keepdims=True)).astype(np.float16)
    cfg = build_cfg(amp, ex, Hi, I, Ho, Hi, K, 16, topk)
    amp.moe_coop(dev(x), dev(sel), dev(rw), cfg)
    torch.cuda.synchronize()
    ref = oracle.moe_coop(x, sel, rw, ex)
    check_close(cfg["out"][:T].cpu().numpy(), ref)


def test_sorted_moe_128_experts_2048_tokens(amp, oracle):
    """The token-sorted prefill MoE at the MoE configuration's size (128 experts 2048 -> 768 -> 2048,
    3 bits, top-8) on a 2048-token chunk. The oracle checks the first 48 tokens' rows (their picks
    land anywhere in the 16384-row sorted list); the whole chunk is checked through properties that
    hold bit for bit: doubling every routing weight doubles every output (fp16 doubling and fp32
    doubling are exact), and reversing the token order reverses the outputs (a row's result does
    not depend on where in an expert's tile it sits, and a token's sum runs in expert order)."""
    from test_gpu_moe import build_cfg, make_experts
    E, H, I, K, topk, T = 128, 2048, 768, 3, 8, 2048
    ex = make_experts(E, H, I, H, K, seed=12000)
    rng = np.random.default_rng(2048)
    x = rng.standard_normal((T, H)).astype(np.float16)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    sel = np.argsort(-logits, axis=1)[:, :topk].astype(np.int64)
    w = np.take_along_axis(logits, sel, axis=1)
    w = np.exp(w - w.max(axis=1, keepdims=True))
    rw = (w / w.sum(axis=1, keepdims=True)).astype(np.float16)
    cfg = build_cfg(amp, ex, H, I, H, H, K, 1, topk)
    cfg["I"] = I

    def run(xa, sa, wa):
        count, tok, wts = amp.moe_sort_routing(dev(sa), dev(wa), E)
        out = torch.zeros((T, H), dtype=torch.float32, device="cuda")
        amp.moe_fused(dev(xa), out, count, tok, wts, cfg)
        torch.cuda.synchronize()
        assert amp.moe_fused_status(cfg) == 0
        return out.cpu().numpy()

    got = run(x, sel, rw)
    n = 48
    check_close(got[:n], oracle.moe_coop(x[:n], sel[:n], rw[:n], ex, gu_f16=True))
    assert np.array_equal(run(x, sel, (rw.astype(np.float32) * 2).astype(np.float16)), got * np.float32(2))
    assert np.array_equal(run(x[::-1].copy(), sel[::-1].copy(), rw[::-1].copy()), got[::-1])
