"""GPU parity of the fused decode MoE (grouped expert GEMV) against the CPU oracle, through the
C ABI (amp_exl3_moe_coop). Tolerance: max |y - ref| / max |ref| < 1e-2 (the specification's
bound for GEMV outputs); measured errors are ~1e-3 (two fp16 roundings on the way)."""
import numpy as np
import pytest

from conftest import make_linear

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def dev(a):
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make_experts(E, Hi, I, Ho, K, seed):
    ex = []
    for e in range(E):
        def one(k, n, s):
            t, su, sv, _ = make_linear(k, n, K, seed=seed + s)
            sv = (sv.astype(np.float32) / (1.2437 * np.sqrt(k))).astype(np.float16)   # keep values O(1)
            return (t, su, sv)
        ex.append({"gate": one(Hi, I, 3 * e), "up": one(Hi, I, 3 * e + 1), "down": one(I, Ho, 3 * e + 2)})
    return ex


def build_cfg(amp, ex, Hi, I, Ho, H, K, rows_max, topk, gu_dtype=torch.float32, gated=True, **extra):
    keep = []

    def table(name, idx):
        ptrs = []
        for e in ex:
            t = dev(e[name][idx])
            keep.append(t)
            ptrs.append(t.data_ptr())
        return amp.ptr_array(ptrs)

    slots = rows_max * topk
    z = lambda shape, dt: torch.zeros(shape, dtype=dt, device="cuda")
    cfg = {
        "g_trellis": table("gate", 0), "g_suh": table("gate", 1), "g_svh": table("gate", 2),
        "u_trellis": table("up", 0), "u_suh": table("up", 1), "u_svh": table("up", 2),
        "d_trellis": table("down", 0), "d_suh": table("down", 1), "d_svh": table("down", 2),
        "gu_g": z((slots, I), gu_dtype), "gu_u": z((slots, I), gu_dtype),
        "d_out": z((slots, Ho), torch.float32),
        "ctr": z((amp.moe_coop_ctr_len(slots),), torch.int32),
        "out": torch.full((rows_max, H), float("nan"), dtype=torch.float32, device="cuda"),
        "Hi": Hi, "Kg": K, "Ku": K, "Kd": K, "mcg": False, "mul1": False, "act": 0, "act_limit": 0.0,
        "gated": gated, "_keep": keep,
    }
    cfg.update(extra)
    return cfg


def check(got, ref, tol=1e-2):
    got, ref = got.astype(np.float64), ref.astype(np.float64)
    assert np.all(np.isfinite(got))
    err = np.max(np.abs(got - ref)) / max(np.max(np.abs(ref)), 1e-6)
    assert err < tol, err
    return err


@pytest.fixture(scope="module")
def amp():
    import ampstein_b200
    return ampstein_b200


@pytest.mark.parametrize("T", [1, 4, 16])
def test_moe_decode_tokens(amp, oracle, T):
    """config-4 structure at reduced width: top-4 of 16 experts, K = 3, softmax routing weights."""
    E, Hi, I, Ho, K, topk = 16, 256, 256, 256, 3, 4
    ex = make_experts(E, Hi, I, Ho, K, seed=100)
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
    check(cfg["out"][:T].cpu().numpy(), ref)
    # second call on the same scratch (the run table and counters are reused)
    cfg["out"].fill_(float("nan"))
    amp.moe_coop(dev(x), dev(sel), dev(rw), cfg)
    torch.cuda.synchronize()
    check(cfg["out"][:T].cpu().numpy(), ref)


def test_moe_runs_longer_than_eight_rows(amp, oracle):
    """16 tokens all picking the same two experts: runs are cut at eight rows."""
    E, Hi, I, Ho, K, topk = 3, 128, 128, 256, 4, 2
    ex = make_experts(E, Hi, I, Ho, K, seed=300)
    rng = np.random.default_rng(5)
    T = 16
    x = rng.standard_normal((T, Hi)).astype(np.float16)
    sel = np.tile(np.array([[2, 0]], np.int64), (T, 1))
    rw = rng.uniform(0.2, 0.8, (T, topk)).astype(np.float16)
    cfg = build_cfg(amp, ex, Hi, I, Ho, Hi, K, 16, topk)
    amp.moe_coop(dev(x), dev(sel), dev(rw), cfg)
    torch.cuda.synchronize()
    check(cfg["out"].cpu().numpy(), oracle.moe_coop(x, sel, rw, ex))


def test_moe_expert_range_zero_weights_padding_and_shared_expert(amp, oracle):
    """Expert-parallel shard [2, 6) of 8 experts, a zero routing weight, a token with no local
    pick, H < Hi (zero padded input), fp16 gate/up scratch, sigmoid-gated shared expert."""
    E, Hi, I, Ho, K, topk = 8, 256, 128, 256, 3, 3
    H = 200
    ex_all = make_experts(E, Hi, I, Ho, K, seed=500)
    local = ex_all[2:6]
    rng = np.random.default_rng(9)
    T = 5
    x = rng.standard_normal((T, H)).astype(np.float16)
    sel = np.array([[2, 7, 3], [0, 1, 7], [5, 4, 2], [3, 3, 6], [4, 0, 5]], np.int64)
    rw = rng.uniform(0.1, 0.6, (T, topk)).astype(np.float16)
    rw[2, 1] = 0.0
    sh_out = rng.standard_normal((T, H)).astype(np.float32)
    sh_gate = (rng.standard_normal(H) * 0.05).astype(np.float16)
    cfg = build_cfg(amp, local, Hi, I, Ho, H, K, 8, topk, gu_dtype=torch.float16,
                    min_expert=2, max_expert=6, sh_gate_w=dev(sh_gate))
    amp.moe_coop(dev(x), dev(sel), dev(rw), cfg, dev(sh_out))
    torch.cuda.synchronize()
    ref = oracle.moe_coop(x, sel, rw, local, min_expert=2, max_expert=6, sh_out=sh_out, sh_gate_w=sh_gate,
                          gu_f16=True, H_out=H)
    check(cfg["out"][:T].cpu().numpy(), ref)


@pytest.mark.parametrize("act,gated,limit", [(1, True, 0.0), (2, True, 0.0), (3, True, 7.0), (0, False, 0.0)])
def test_moe_activations(amp, oracle, act, gated, limit):
    E, Hi, I, Ho, K, topk = 4, 128, 128, 128, 4, 2
    ex = make_experts(E, Hi, I, Ho, K, seed=700 + act)
    rng = np.random.default_rng(act)
    x = rng.standard_normal((3, Hi)).astype(np.float16)
    sel = np.array([[0, 1], [2, 3], [1, 2]], np.int64)
    rw = np.full((3, topk), 0.5, np.float16)
    cfg = build_cfg(amp, ex, Hi, I, Ho, Hi, K, 4, topk, gated=gated, act=act, act_limit=limit)
    amp.moe_coop(dev(x), dev(sel), dev(rw), cfg)
    torch.cuda.synchronize()
    ref = oracle.moe_coop(x, sel, rw, ex, act=act, act_limit=limit, gated=gated)
    check(cfg["out"][:3].cpu().numpy(), ref)


def test_moe_config4_shapes_one_token(amp, oracle):
    """The benchmark's expert shapes (2048 -> 768 -> 2048, K = 3), 8 experts, top-8, one token."""
    E, Hi, I, Ho, K, topk = 8, 2048, 768, 2048, 3, 8
    ex = make_experts(E, Hi, I, Ho, K, seed=900)
    rng = np.random.default_rng(4)
    x = rng.standard_normal((1, Hi)).astype(np.float16)
    sel = rng.permutation(E)[None, :topk].astype(np.int64)
    rw = np.full((1, topk), 1.0 / topk, np.float16)
    cfg = build_cfg(amp, ex, Hi, I, Ho, Hi, K, 16, topk)
    amp.moe_coop(dev(x), dev(sel), dev(rw), cfg)
    torch.cuda.synchronize()
    check(cfg["out"][:1].cpu().numpy(), oracle.moe_coop(x, sel, rw, ex))


@pytest.mark.parametrize("T", [1, 5])
def test_moe_experts_of_different_bit_widths(amp, oracle, T):
    """Mixed packs (the reference's g_bits / u_bits / d_bits tables, exl3_moe_coop.cuh:46-50): every
    expert's gate|up and down have their own bit width; one pair of launches per width that occurs,
    each working on the runs of its width. One token (tables built in the kernel, cluster form) and
    several; a token whose picks all fall on one width; the second call reuses the cached masks."""
    E, Hi, I, Ho, topk = 8, 256, 256, 256, 3
    kgu = [3, 4, 4, 3, 5, 4, 3, 5]
    kd = [4, 4, 2, 2, 4, 6, 6, 2]
    ex = []
    for e in range(E):
        def one(k, n, K, s):
            t, su, sv, _ = make_linear(k, n, K, seed=1500 + s)
            sv = (sv.astype(np.float32) / (1.2437 * np.sqrt(k))).astype(np.float16)
            return (t, su, sv)
        ex.append({"gate": one(Hi, I, kgu[e], 3 * e), "up": one(Hi, I, kgu[e], 3 * e + 1), "down": one(I, Ho, kd[e], 3 * e + 2)})
    rng = np.random.default_rng(15 + T)
    x = rng.standard_normal((T, Hi)).astype(np.float16)
    sel = np.stack([rng.permutation(E)[:topk] for _ in range(T)]).astype(np.int64)
    sel[0] = [1, 2, 5]                                   # gate|up all 4 bits
    rw = rng.uniform(0.2, 0.6, (T, topk)).astype(np.float16)
    bits = lambda v: torch.tensor(v, dtype=torch.uint8, device="cuda")
    cfg = build_cfg(amp, ex, Hi, I, Ho, Hi, 0, 8, topk, g_bits=bits(kgu), u_bits=bits(kgu), d_bits=bits(kd))
    ref = oracle.moe_coop(x, sel, rw, ex)
    for _ in range(2):
        cfg["out"].fill_(float("nan"))
        amp.moe_coop(dev(x), dev(sel), dev(rw), cfg)
        torch.cuda.synchronize()
        check(cfg["out"][:T].cpu().numpy(), ref)
    assert cfg["_kmask"] == (0b11100, 0b101010)


def test_moe_and_a_plain_gemv_on_two_streams_at_once(amp, oracle):
    """The reference runs the shared expert's linears on a side stream while moe_coop runs
    (src/ucode/ampstein/glm5.uc:970,998): launches that overlap on the GPU must not share arrival
    counters. Many rounds of a fused MoE on one stream and plain GEMVs (shapes whose column blocks
    are shared between CTAs) on another, all results checked."""
    from test_gpu_parity import check_close
    E, Hi, I, Ho, K, topk, T = 16, 512, 256, 512, 3, 4, 4
    ex = make_experts(E, Hi, I, Ho, K, seed=1300)
    rng = np.random.default_rng(13)
    x = rng.standard_normal((T, Hi)).astype(np.float16)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    sel = np.argsort(-logits, axis=1)[:, :topk].astype(np.int64)
    rw = np.full((T, topk), 1.0 / topk, np.float16)
    cfg = build_cfg(amp, ex, Hi, I, Ho, Hi, K, 16, topk)
    ref_moe = oracle.moe_coop(x, sel, rw, ex)
    trellis, suh, svh, xg = make_linear(4096, 1024, 4, seed=1301, m=2)
    ref_lin = oracle.linear(xg, trellis, suh, svh, 0, fp32_out=True)
    t, su, sv, xgd = dev(trellis), dev(suh), dev(svh), dev(xg)
    xd, seld, rwd = dev(x), dev(sel), dev(rw)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    outs = [torch.empty((2, 1024), dtype=torch.float16, device="cuda") for _ in range(24)]
    moe_outs = []
    torch.cuda.synchronize()
    for i in range(24):
        with torch.cuda.stream(s1):
            amp.moe_coop(xd, seld, rwd, cfg)
            if i % 6 == 5:
                moe_outs.append(cfg["out"][:T].clone())
        with torch.cuda.stream(s2):
            amp.exl3_gemm(xgd, t, outs[i], su, sv)
    torch.cuda.synchronize()
    for o in outs:
        check_close(o.cpu().numpy(), ref_lin)
    for o in moe_outs:
        check(o.cpu().numpy(), ref_moe)
