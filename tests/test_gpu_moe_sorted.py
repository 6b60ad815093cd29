"""GPU parity of the token-sorted prefill MoE (amp_exl3_moe_sorted: expert-grouped tcgen05 GEMMs)
against the CPU oracle's per-slot MoE and against the decode-shaped fused MoE of this library, through
the C ABI. Tolerance: max |y - ref| / max |ref| < 1e-2 (the bound for fp16 linears); measured errors
are ~1e-3. The reference's own check of this path compares it with its composite path at 3.4-4.3e-3
relative RMS (tests/glm5_moe.uc)."""
import numpy as np
import pytest

from conftest import make_linear
from test_gpu_moe import build_cfg, check, dev, make_experts

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def amp():
    import ampstein_b200
    return ampstein_b200


def routing(rng, T, E, topk):
    logits = rng.standard_normal((T, E)).astype(np.float32)
    sel = np.argsort(-logits, axis=1)[:, :topk].astype(np.int64)
    w = np.take_along_axis(logits, sel, axis=1)
    w = np.exp(w - w.max(axis=1, keepdims=True))
    return sel, (w / w.sum(axis=1, keepdims=True)).astype(np.float16)


def run_sorted(amp, cfg, x, sel, rw, E, e0=0, tiers=None):
    xd = dev(x)
    count, tok, wts = amp.moe_sort_routing(dev(sel), dev(rw), E, e0)
    out = torch.zeros((x.shape[0], x.shape[1]), dtype=torch.float32, device="cuda")
    for lo, hi in (tiers or [(1, 0)]):
        amp.moe_fused(xd, out, count, tok, wts, cfg, -1, lo, hi, 16)
    torch.cuda.synchronize()
    assert amp.moe_fused_status(cfg) == 0
    from test_gpu_parity import gemm_status
    assert gemm_status() == 0                       # no bounded wait of the tensor-core kernel ran out
    return out.cpu().numpy(), count.cpu().numpy()


@pytest.mark.parametrize("T,E,topk,K", [(300, 16, 4, 3), (1200, 4, 2, 4), (7, 16, 4, 3)])
def test_sorted_moe_against_the_oracle(amp, oracle, T, E, topk, K):
    """Random routing: experts with a handful of rows, with hundreds (more than one 512-row tile at
    T = 1200), and with none (T = 7)."""
    H, I = 256, 256
    ex = make_experts(E, H, I, H, K, seed=2100 + T)
    rng = np.random.default_rng(T)
    x = rng.standard_normal((T, H)).astype(np.float16)
    sel, rw = routing(rng, T, E, topk)
    cfg = build_cfg(amp, ex, H, I, H, H, K, 1, topk)
    cfg["I"] = I
    got, count = run_sorted(amp, cfg, x, sel, rw, E)
    assert count[:E].sum() == T * topk
    ref = oracle.moe_coop(x, sel, rw, ex, gu_f16=True)
    check(got, ref)
    # a second call on the same workspace adds the same sum again, bit for bit
    got2, _ = run_sorted(amp, cfg, x, sel, rw, E)
    assert np.array_equal(got, got2)


def test_sorted_moe_row_tiers_shard_range_and_accumulation(amp, oracle):
    """The reference's three tiered calls (rows 33+, 17-32, 1-16) add up to the single call; picks
    outside the expert-parallel shard [2, 6) land in the sentinel bin and contribute nothing; out
    is accumulated into, not overwritten."""
    E_all, H, I, K, topk, T = 8, 256, 128, 3, 3, 90
    ex_all = make_experts(E_all, H, I, H, K, seed=2300)
    local = ex_all[2:6]
    rng = np.random.default_rng(11)
    x = rng.standard_normal((T, H)).astype(np.float16)
    sel, rw = routing(rng, T, E_all, topk)
    sel[:40, 0] = 3                                      # one heavy expert, several light ones
    sel[:40, 1] = np.where(sel[:40, 1] == 3, 4, sel[:40, 1])
    sel[:40, 2] = np.where(sel[:40, 2] == 3, 5, sel[:40, 2])
    for r in range(40):                                  # keep a token's picks distinct
        if len(set(sel[r])) < topk:
            sel[r] = [3, 4, 5]
    cfg = build_cfg(amp, local, H, I, H, H, K, 1, topk)
    cfg["I"] = I
    one, count = run_sorted(amp, cfg, x, sel, rw, 4, e0=2)
    assert count[4] > 0 and count[:4].max() > 32 and count[:4].min() <= 32
    tiers, _ = run_sorted(amp, cfg, x, sel, rw, 4, e0=2, tiers=[(33, 0), (17, 32), (1, 16)])
    # (a token's sum is split over the calls, so the fp32 additions associate differently)
    assert np.allclose(one, tiers, rtol=1e-5, atol=1e-6)
    ref = oracle.moe_coop(x, sel, rw, local, min_expert=2, max_expert=6, gu_f16=True)
    check(one, ref)
    # accumulation: a second pass over a non-zero output adds to it
    xd = dev(x)
    cnt, tok, wts = amp.moe_sort_routing(dev(sel), dev(rw), 4, 2)
    out = torch.full((T, H), 1.5, dtype=torch.float32, device="cuda")
    amp.moe_fused(xd, out, cnt, tok, wts, cfg)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), one + np.float32(1.5))


@pytest.mark.parametrize("act,gated,limit,cbname", [(1, True, 0.0, None), (3, True, 7.0, "mcg"), (0, False, 0.0, "mul1")])
def test_sorted_moe_activations_codebooks_and_no_gate(amp, oracle, act, gated, limit, cbname):
    E, H, I, K, topk, T = 4, 128, 256, 4, 2, 150
    ex = make_experts(E, H, I, H, K, seed=2500 + act)
    rng = np.random.default_rng(20 + act)
    x = rng.standard_normal((T, H)).astype(np.float16)
    sel, rw = routing(rng, T, E, topk)
    extra = {cbname: True} if cbname else {}
    cfg = build_cfg(amp, ex, H, I, H, H, K, 1, topk, gated=gated, act=act, act_limit=limit, **extra)
    cfg["I"] = I
    got, _ = run_sorted(amp, cfg, x, sel, rw, E)
    cb = {"mcg": 1, "mul1": 2}.get(cbname, 0)
    ref = oracle.moe_coop(x, sel, rw, ex, act=act, act_limit=limit, gated=gated, cb=cb, gu_f16=True)
    check(got, ref)


def test_sorted_moe_deferred_slots_and_gather(amp, oracle):
    """The reference's reproducible mode: moe_fused stores weight * result of every assignment in its
    slot (slot = sorted position, as src/ucode/ampstein/glm5.uc:1204-1221 sets it up) and leaves out
    alone; moe_gather adds every token's slots in pick order. Also slots of kind 2 (unweighted rows
    of another tier, weighted by the gather)."""
    E, H, I, K, topk, T = 8, 256, 128, 3, 3, 70
    ex = make_experts(E, H, I, H, K, seed=3500)
    rng = np.random.default_rng(61)
    x = rng.standard_normal((T, H)).astype(np.float16)
    sel, rw = routing(rng, T, E, topk)
    cfg = build_cfg(amp, ex, H, I, H, H, K, 1, topk)
    cfg["I"] = I
    direct, _ = run_sorted(amp, cfg, x, sel, rw, E)
    xd = dev(x)
    count, tok, wts, fe, inv, start = amp.moe_sort_routing(dev(sel), dev(rw), E, 0, with_inverse=True)
    A = T * topk
    scratch = torch.full((A, H), float("nan"), dtype=torch.float32, device="cuda")
    out = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    amp.moe_fused(xd, out, count, tok, wts, cfg, -1, 1, 0, 16, scratch, start)
    torch.cuda.synchronize()
    assert amp.moe_fused_status(cfg) == 0
    assert not out.any() and torch.isfinite(scratch).all()
    kind = (count[:E] > 0).to(torch.int64)
    amp.moe_gather(out, scratch, fe, inv, start[:E].contiguous(), start[:E].contiguous(), kind, wts)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert np.allclose(got, direct, rtol=1e-5, atol=1e-6)          # same terms, pick order instead of expert order
    check(got, oracle.moe_coop(x, sel, rw, ex, gu_f16=True))
    # kind 2: the same rows unweighted, the gather applies the weights
    unweighted = (scratch / wts.float()[:, None]).contiguous()
    out2 = torch.zeros_like(out)
    amp.moe_gather(out2, unweighted, fe, inv, start[:E].contiguous(), start[:E].contiguous(), kind * 2, wts)
    torch.cuda.synchronize()
    assert np.allclose(out2.cpu().numpy(), got, rtol=1e-4, atol=1e-5)
    # a slot scratch that is too short is reported, not overrun
    short = torch.zeros((A // 2, H), dtype=torch.float32, device="cuda")
    amp.moe_fused(xd, out, count, tok, wts, cfg, -1, 1, 0, 16, short, start)
    assert amp.moe_fused_status(cfg) & 16


def test_sorted_moe_gate_and_up_of_different_widths(amp, oracle):
    """Kg != Ku: gate and up run as two grouped launches instead of one."""
    E, H, I, topk, T = 4, 256, 128, 2, 64
    ex = []
    for e in range(E):
        def one(k, n, K, s):
            t, su, sv, _ = make_linear(k, n, K, seed=2700 + s)
            sv = (sv.astype(np.float32) / (1.2437 * np.sqrt(k))).astype(np.float16)
            return (t, su, sv)
        ex.append({"gate": one(H, I, 3, 3 * e), "up": one(H, I, 5, 3 * e + 1), "down": one(I, H, 4, 3 * e + 2)})
    rng = np.random.default_rng(31)
    x = rng.standard_normal((T, H)).astype(np.float16)
    sel, rw = routing(rng, T, E, topk)
    cfg = build_cfg(amp, ex, H, I, H, H, 0, 1, topk)
    cfg.update({"Kg": 3, "Ku": 5, "Kd": 4, "I": I})
    got, _ = run_sorted(amp, cfg, x, sel, rw, E)
    check(got, oracle.moe_coop(x, sel, rw, ex, gu_f16=True))


def test_sorted_moe_experts_of_different_bit_widths(amp, oracle):
    """Mixed packs (the reference's bits_g / bits_u / bits_d tables of exl3_moe, exl3_moe.cuh:50-52):
    every expert's gate|up and down have their own bit width; one grouped GEMM launch per width that
    occurs, each serving the tiles of its width. Default codebook (the reference: mul1 only)."""
    E, H, I, topk, T = 8, 256, 256, 3, 200
    kgu = [3, 4, 4, 3, 5, 4, 3, 5]
    kd = [4, 4, 2, 2, 4, 6, 6, 2]
    ex = []
    for e in range(E):
        def one(k, n, K, s):
            t, su, sv, _ = make_linear(k, n, K, seed=3700 + s)
            sv = (sv.astype(np.float32) / (1.2437 * np.sqrt(k))).astype(np.float16)
            return (t, su, sv)
        ex.append({"gate": one(H, I, kgu[e], 3 * e), "up": one(H, I, kgu[e], 3 * e + 1), "down": one(I, H, kd[e], 3 * e + 2)})
    rng = np.random.default_rng(71)
    x = rng.standard_normal((T, H)).astype(np.float16)
    sel, rw = routing(rng, T, E, topk)
    bits = lambda v: torch.tensor(v, dtype=torch.uint8, device="cuda")
    cfg = build_cfg(amp, ex, H, I, H, H, 0, 1, topk, g_bits=bits(kgu), u_bits=bits(kgu), d_bits=bits(kd))
    cfg["I"] = I
    ref = oracle.moe_coop(x, sel, rw, ex, gu_f16=True)
    for _ in range(2):                                   # the second call reuses the cached masks
        got, _ = run_sorted(amp, cfg, x, sel, rw, E)
        check(got, ref)
    assert cfg["_kmask"] == (0b11100, 0b101010)


def test_sorted_moe_agrees_with_the_decode_moe(amp):
    """16 tokens through both fused forms of this library (grouped GEMV and grouped tensor-core
    GEMM): same element arithmetic, different summation order inside the dot products."""
    E, H, I, K, topk, T = 16, 256, 256, 3, 4, 16
    ex = make_experts(E, H, I, H, K, seed=2900)
    rng = np.random.default_rng(41)
    x = rng.standard_normal((T, H)).astype(np.float16)
    sel, rw = routing(rng, T, E, topk)
    cfg = build_cfg(amp, ex, H, I, H, H, K, 16, topk, gu_dtype=torch.float16)
    cfg["I"] = I
    amp.moe_coop(dev(x), dev(sel), dev(rw), cfg)
    torch.cuda.synchronize()
    dec = cfg["out"][:T].cpu().numpy()
    got, _ = run_sorted(amp, cfg, x, sel, rw, E)
    check(got, dec, tol=5e-3)


def test_sorted_moe_replays_from_a_cuda_graph_with_new_routing(amp, oracle):
    """Nothing in the call depends on the routing's values on the host: captured once in a CUDA graph,
    the six launches serve a different routing (other counts, other tiles) written into the same
    device tensors before a replay."""
    E, H, I, K, topk, T = 8, 256, 128, 3, 2, 96
    ex = make_experts(E, H, I, H, K, seed=3900)
    cfg = build_cfg(amp, ex, H, I, H, H, K, 1, topk)
    cfg["I"] = I
    rng = np.random.default_rng(81)
    cases = []
    for i in range(2):
        x = rng.standard_normal((T, H)).astype(np.float16)
        sel, rw = routing(rng, T, E, topk)
        if i == 1:
            sel[:60, 0] = 5                              # a heavy expert and two empty ones
            sel[:, 1] = np.where(np.isin(sel[:, 1], (0, 5, 7)), 3, sel[:, 1])
            sel[:, 0] = np.where(np.isin(sel[:, 0], (0, 7)), 2, sel[:, 0])
            sel[:, 1] = np.where(sel[:, 1] == sel[:, 0], (sel[:, 0] + 1) % 7 + (sel[:, 0] + 1) // 7, sel[:, 1])
        cases.append((x, sel, rw))
    xd = dev(cases[0][0])
    count, tok, wts = amp.moe_sort_routing(dev(cases[0][1]), dev(cases[0][2]), E)
    out = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    st, gr = torch.cuda.Stream(), torch.cuda.CUDAGraph()
    with torch.cuda.stream(st):
        amp.moe_fused(xd, out, count, tok, wts, cfg)    # warm-up: workspace and kernel attributes exist before capture
    torch.cuda.synchronize()
    with torch.cuda.stream(st), torch.cuda.graph(gr, stream=st):
        amp.moe_fused(xd, out, count, tok, wts, cfg)
    for x, sel, rw in cases[::-1]:
        c2, t2, w2 = amp.moe_sort_routing(dev(sel), dev(rw), E)
        xd.copy_(dev(x)); count.copy_(c2); tok.copy_(t2); wts.copy_(w2)
        out.zero_()
        torch.cuda.synchronize()
        gr.replay()
        torch.cuda.synchronize()
        assert amp.moe_fused_status(cfg) == 0
        check(out.cpu().numpy(), oracle.moe_coop(x, sel, rw, ex, gu_f16=True))


def test_sorted_moe_reports_bad_routing_without_touching_memory(amp):
    """A token index outside [0, T) and counts that describe more rows than the list holds set the
    status word; the entries in error are left out."""
    E, H, I, K, topk, T = 4, 128, 128, 3, 2, 12
    ex = make_experts(E, H, I, H, K, seed=3100)
    rng = np.random.default_rng(51)
    x = rng.standard_normal((T, H)).astype(np.float16)
    sel, rw = routing(rng, T, E, topk)
    cfg = build_cfg(amp, ex, H, I, H, H, K, 1, topk)
    cfg["I"] = I
    xd = dev(x)
    count, tok, wts = amp.moe_sort_routing(dev(sel), dev(rw), E)
    bad_tok = tok.clone()
    bad_tok[3] = T + 5
    out = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    amp.moe_fused(xd, out, count, bad_tok, wts, cfg)
    assert amp.moe_fused_status(cfg) & 4
    assert torch.isfinite(out).all()
    bad_count = count.clone()
    bad_count[1] += 1000
    out.zero_()
    amp.moe_fused(xd, out, bad_count, tok, wts, cfg)
    assert amp.moe_fused_status(cfg) & 3
    assert torch.isfinite(out).all()
    # and a clean call afterwards is clean
    out.zero_()
    amp.moe_fused(xd, out, count, tok, wts, cfg)
    assert amp.moe_fused_status(cfg) == 0


def test_sorted_moe_argument_errors(amp):
    E, H, I, K, topk, T = 2, 128, 128, 3, 1, 4
    ex = make_experts(E, H, I, H, K, seed=3300)
    cfg = build_cfg(amp, ex, H, I, H, H, K, 1, topk)
    cfg["I"] = I
    x = torch.zeros((T, H), dtype=torch.float16, device="cuda")
    out = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    count = torch.tensor([2, 2, 0], dtype=torch.int64, device="cuda")
    tok = torch.tensor([0, 1, 2, 3], dtype=torch.int64, device="cuda")
    w = torch.ones(4, dtype=torch.float16, device="cuda")
    with pytest.raises(TypeError):
        amp.moe_fused(x, out.half(), count, tok, w, cfg)
    with pytest.raises(RuntimeError):
        amp.moe_fused(x, out, count, tok[:3].contiguous(), w[:3].contiguous(), cfg)     # 3 picks for 4 tokens
    with pytest.raises(RuntimeError):
        amp.moe_fused(x.cpu(), out, count, tok, w, cfg)
