"""CPU tests of the oracle (the C restatement of the reference's EXL3 arithmetic): pins it
against the reference's packer, against an independent numpy restatement, against float64
linear algebra and against fixtures written by the reference's own kernels."""
import glob
import os

import numpy as np
import pytest

from conftest import make_linear

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_half_conversion_matches_numpy(oracle):
    L = oracle.lib()
    rng = np.random.default_rng(0)
    vals = np.concatenate([
        rng.standard_normal(20000) * rng.choice([1e-7, 1e-5, 1e-3, 1.0, 100.0, 3e4], 20000),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, 6e-8, 2.9802322387695312e-8, 2.98e-8, 3e-8]),
    ])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([L.exl3o_d2h(float(v)) for v in vals], np.uint16)
    assert np.array_equal(got, want)
    hs = rng.integers(0, 65536, 5000).astype(np.uint16)
    hs = hs[(hs & 0x7c00) != 0x7c00]
    back = np.array([L.exl3o_h2f(int(h)) for h in hs], np.float32)
    assert np.array_equal(back, hs.view(np.float16).astype(np.float32))


# ---- independent numpy restatement of the format (written from the format description, not
# from the C code): bits MSB-first in little-endian uint32 words, window ends at (t+1)K --------

def np_states(tile_u16, K):
    w32 = tile_u16.astype(np.uint32)
    words = w32[0::2] | (w32[1::2] << 16)
    bits = ((words[:, None] >> np.arange(31, -1, -1, dtype=np.uint32)[None, :]) & 1).reshape(-1)
    ring = 256 * K
    t = np.arange(256)
    idx = ((t[:, None] + 1) * K - 16 + np.arange(16)[None, :]) % ring
    wbits = bits[idx].astype(np.uint32)
    return (wbits << np.arange(15, -1, -1, dtype=np.uint32)[None, :]).sum(axis=1).astype(np.uint16)


def np_decode(states, cb):
    s = states.astype(np.uint64)
    if cb == 2:
        x = (s * 0x83DCD12D) & 0xFFFFFFFF
        bs = (x & 0xff) + ((x >> 8) & 0xff) + ((x >> 16) & 0xff) + (x >> 24)
        h = (0x6400 + bs).astype(np.uint16).view(np.float16).astype(np.float64)
        kinv = np.array([0x1eee], np.uint16).view(np.float16).astype(np.float64)[0]
        kbias = np.array([0xc931], np.uint16).view(np.float16).astype(np.float64)[0]
        return (h * kinv + kbias).astype(np.float16)
    x = (s * 89226354 + 64248484) & 0xFFFFFFFF if cb == 0 else (s * 0xCBAC1FED) & 0xFFFFFFFF
    x = (x & 0x8fff8fff) ^ 0x3b603b60
    lo = (x & 0xffff).astype(np.uint16).view(np.float16).astype(np.float64)
    hi = (x >> 16).astype(np.uint16).view(np.float16).astype(np.float64)
    return (lo + hi).astype(np.float16)


def np_reconstruct(trellis, cb):
    tk, tn, w = trellis.shape
    K = w // 16
    out = np.zeros((tk * 16, tn * 16), np.float16)
    t = np.arange(256)
    lane, j = t // 8, t % 8
    row = 2 * (lane % 4) + (j & 1) + 8 * ((j >> 1) & 1)
    col = lane // 4 + 8 * (j >> 2)
    for a in range(tk):
        for b in range(tn):
            vals = np_decode(np_states(trellis[a, b], K), cb)
            out[a * 16 + row, b * 16 + col] = vals
    return out


@pytest.mark.parametrize("K", range(1, 9))
def test_states_match_numpy_and_packer(oracle, K):
    rng = np.random.default_rng(K)
    tile = rng.integers(0, 65536, 16 * K, dtype=np.uint16)
    st = oracle.tile_states(tile, K)
    assert np.array_equal(st, np_states(tile, K))
    # reference packer (pack.cu): the low K bits of code t are the last K bits of window t, and
    # consecutive windows overlap by 16-K bits (tail-biting ring)
    codes = rng.integers(0, 65536, 256, dtype=np.uint16)
    packed = oracle.pack_tile(codes, K)
    st = oracle.tile_states(packed, K).astype(np.uint32)
    mask = (1 << K) - 1
    assert np.array_equal(st & mask, codes.astype(np.uint32) & mask)
    prev = np.roll(st, 1)
    assert np.array_equal(st >> K, prev & ((1 << (16 - K)) - 1))


@pytest.mark.parametrize("cb", [0, 1, 2])
def test_codebook_matches_numpy(oracle, cb):
    table = oracle.decode_table(cb)
    want = np_decode(np.arange(65536, dtype=np.uint32), cb)
    assert np.array_equal(table.view(np.uint16), want.view(np.uint16))
    t64 = table.astype(np.float64)
    assert abs(t64.mean()) < 5e-3 and np.abs(t64).max() < 4.0
    assert abs(t64.std() - (1.0 if cb == 2 else 1.244)) < 2e-3


def test_tile_permutation_is_mma_fragment_order(oracle):
    seen = set()
    for t in range(256):
        r, c = oracle.tile_pos(t)
        lane, j = t // 8, t % 8
        assert r == 2 * (lane % 4) + (j & 1) + 8 * ((j >> 1) & 1)
        assert c == lane // 4 + 8 * (j >> 2)
        seen.add((r, c))
    assert len(seen) == 256


@pytest.mark.parametrize("K,cb", [(1, 0), (2, 1), (3, 2), (4, 0), (5, 0), (6, 2), (7, 1), (8, 0)])
def test_reconstruct_matches_numpy(oracle, K, cb):
    trellis, _, _, _ = make_linear(32, 128, K, seed=100 + K)
    got = oracle.reconstruct(trellis, cb)
    assert np.array_equal(got.view(np.uint16), np_reconstruct(trellis, cb).view(np.uint16))


def sylvester(n):
    H = np.array([[1.0]])
    while H.shape[0] < n:
        H = np.block([[H, H], [H, -H]])
    return H


def test_hadamard_is_sylvester_and_involutive(oracle):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 256)).astype(np.float32)
    y = oracle.had_ff(x)
    H = sylvester(128) / np.sqrt(128.0)
    want = np.concatenate([x[:, :128].astype(np.float64) @ H, x[:, 128:].astype(np.float64) @ H], axis=1)
    assert np.allclose(y, want, rtol=0, atol=2e-6)
    assert np.allclose(oracle.had_ff(y), x, rtol=0, atol=4e-6)
    # fp16 form: pre-scale multiply in fp16, one rounding at the end
    xh = x.astype(np.float16)
    pre = rng.choice(np.array([-1.0, 1.0], np.float16), 256)
    yh = oracle.had_hf(xh, pre=pre)
    want = np.concatenate([((xh * pre)[:, i:i + 128].astype(np.float64) @ H) for i in (0, 128)], axis=1)
    assert np.max(np.abs(yh.astype(np.float64) - want)) < 2e-3


def rel_rms(a, b):
    a, b = a.astype(np.float64), b.astype(np.float64)
    return np.sqrt(np.mean((a - b) ** 2) / np.mean(b ** 2))


@pytest.mark.parametrize("K,cb", [(2, 1), (4, 0), (5, 2)])
def test_reconstruct_had_is_both_side_rotation(oracle, K, cb):
    trellis, suh, svh, _ = make_linear(256, 256, K, seed=7 + K)
    what = oracle.reconstruct(trellis, cb).astype(np.float64)
    H = sylvester(128)
    want = np.zeros_like(what)
    for a in range(2):
        for b in range(2):
            blk = what[a * 128:(a + 1) * 128, b * 128:(b + 1) * 128]
            want[a * 128:(a + 1) * 128, b * 128:(b + 1) * 128] = H @ blk @ H / 128.0
    want = suh.astype(np.float64)[:, None] * want * svh.astype(np.float64)[None, :]
    got = oracle.reconstruct_had(trellis, suh, svh, cb)
    assert rel_rms(got, want) < 2e-3


@pytest.mark.parametrize("m", [1, 5])
def test_linear_equals_original_basis_product(oracle, m):
    """had(x*suh) @ W_hat -> had(.)*svh must equal x @ W with W the original-basis weight."""
    trellis, suh, svh, x = make_linear(256, 384, 4, seed=11, m=m)
    what = oracle.reconstruct(trellis, 0).astype(np.float64)
    H = sylvester(128)
    W = np.zeros_like(what)
    for a in range(2):
        for b in range(3):
            W[a * 128:(a + 1) * 128, b * 128:(b + 1) * 128] = H @ what[a * 128:(a + 1) * 128, b * 128:(b + 1) * 128] @ H / 128.0
    W = suh.astype(np.float64)[:, None] * W * svh.astype(np.float64)[None, :]
    want = x.astype(np.float64) @ W
    got16 = oracle.linear(x, trellis, suh, svh, 0)
    got32 = oracle.linear(x, trellis, suh, svh, 0, fp32_out=True)
    assert rel_rms(got16, want) < 3e-3
    assert rel_rms(got32, want) < 3e-3


def test_linear_is_linear_in_x(oracle):
    trellis, suh, svh, x = make_linear(128, 128, 3, seed=3, m=2)
    y = oracle.linear(x, trellis, suh, svh, 1, fp32_out=True)
    y2 = oracle.linear((x * np.float16(2.0)), trellis, suh, svh, 1, fp32_out=True)
    assert np.allclose(y2, 2.0 * y, rtol=1e-6, atol=1e-6)      # exact scaling by a power of two


def test_allreduce_rank_order_sum(oracle):
    rng = np.random.default_rng(9)
    parts = [rng.standard_normal(1000).astype(np.float16) for _ in range(5)]
    got = oracle.allreduce_fp16(parts)
    acc = np.zeros(1000, np.float32)
    for p in parts:
        acc = acc + p.astype(np.float32)
    assert np.array_equal(got.view(np.uint16), acc.astype(np.float16).view(np.uint16))


def test_moe_oracle_equals_composition_of_linears(oracle):
    """The MoE oracle against float64 algebra in the original basis: every expert is
    down(silu(gate x) * up x) with dense original-basis weights."""
    rng = np.random.default_rng(12)
    Hi, I, Ho, K = 128, 128, 128, 4
    H = sylvester(128)

    def dense(trellis, suh, svh):
        what = oracle.reconstruct(trellis, 0).astype(np.float64)
        return suh.astype(np.float64)[:, None] * (H @ what @ H / 128.0) * svh.astype(np.float64)[None, :]

    ex, Ws = [], []
    for e in range(3):
        trip = []
        for s, (k, n) in enumerate(((Hi, I), (Hi, I), (I, Ho))):
            t, su, sv, _ = make_linear(k, n, K, seed=40 + 3 * e + s)
            sv = (sv.astype(np.float32) / (1.2437 * np.sqrt(k))).astype(np.float16)
            trip.append((t, su, sv))
        ex.append({"gate": trip[0], "up": trip[1], "down": trip[2]})
        Ws.append([dense(*t) for t in trip])
    x = rng.standard_normal((2, Hi)).astype(np.float16)
    sel = np.array([[0, 2], [1, 0]], np.int64)
    rw = np.array([[0.7, 0.3], [0.4, 0.6]], np.float16)
    got = oracle.moe_coop(x, sel, rw, ex)
    want = np.zeros((2, Ho))
    for r in range(2):
        for k in range(2):
            Wg, Wu, Wd = Ws[sel[r, k]]
            g, u = x[r].astype(np.float64) @ Wg, x[r].astype(np.float64) @ Wu
            want[r] += float(rw[r, k]) * ((g / (1 + np.exp(-g)) * u) @ Wd)
    assert rel_rms(got, want) < 5e-3


def test_empty_shapes(oracle):
    assert oracle.reconstruct(np.zeros((0, 8, 64), np.uint16), 0).shape == (0, 128)


# ---- fixtures written by the reference's own CUDA kernels (compiled unmodified for sm_100a and
# run on a B200; generator: tests/golden/make_reference_fixtures.py) ------------------------------

def _golden_files():
    return sorted(glob.glob(os.path.join(GOLDEN, "ref_*.npz")))


@pytest.mark.parametrize("path", _golden_files() or [None])
def test_oracle_matches_reference_fixture(oracle, path):
    if path is None:
        pytest.skip("no reference fixtures committed yet")
    z = np.load(path)
    kind = str(z["kind"])
    if kind == "reconstruct":
        got = oracle.reconstruct(z["trellis"], int(z["cb"]))
        assert np.array_equal(got.view(np.uint16), z["out"].view(np.uint16))
    elif kind == "reconstruct_had":
        got = oracle.reconstruct_had(z["trellis"], z["suh"], z["svh"], int(z["cb"]))
        assert np.array_equal(got.view(np.uint16), z["out"].view(np.uint16))
    elif kind == "had_hf":
        pre = z["pre"] if z["pre"].size else None
        post = z["post"] if z["post"].size else None
        got = oracle.had_hf(z["x"], pre=pre, post=post)
        assert np.array_equal(got.view(np.uint16), z["out"].view(np.uint16))
    elif kind == "had_ff":
        post = z["post"] if z["post"].size else None
        got = oracle.had_ff(z["x"], post=post)
        assert np.array_equal(got.view(np.uint32), z["out"].view(np.uint32))
    else:
        raise AssertionError("unknown fixture kind " + kind)


def test_int8_activation_linear_against_the_fp_linear(oracle):
    """The int8-activation restatement (mul1 codebook, one scale per 128 rows of k) deviates from the
    fp32-accumulated linear by the quantisation of the activations only: a few 1e-3 relative rms
    (the reference quotes ~8e-3 for its per-slice scales), and is exact for an input whose rotated
    form is exactly representable (all zeros)."""
    import numpy as np
    from conftest import make_linear
    for K in (2, 4, 6):
        trellis, suh, svh, x = make_linear(512, 256, K, seed=40 + K, m=3)
        a = oracle.linear(x, trellis, suh, svh, 2, fp32_out=True).astype(np.float64)
        b = oracle.linear_int8(x, trellis, suh, svh, fp32_out=True).astype(np.float64)
        rms = np.sqrt(np.mean((a - b) ** 2) / np.mean(a ** 2))
        assert 1e-4 < rms < 1e-2, rms
    z = oracle.linear_int8(np.zeros((1, 512), np.float16), trellis, suh, svh, fp32_out=True)
    assert np.all(z == 0)


@pytest.mark.parametrize("KA", [1, 2, 3])
def test_half_integer_bitrates_pack_and_decode(oracle, KA):
    """Half-integer bitrates KA + 0.5: positions alternate KA and KA + 1 bits (odd positions carry the
    extra bit, Q/exl3_dq.cuh:254-284). The packer's bits come back as the low bits of the decoded
    states, and a bit-array restatement in numpy gives the same 256 states and the same weights."""
    import ctypes
    L = oracle.lib()
    rng = np.random.default_rng(40 + KA)
    bits2 = 2 * KA + 1
    p16 = lambda a: a.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16))
    codes = rng.integers(0, 65536, 256).astype(np.uint16)
    tile = np.zeros(8 * bits2, np.uint16)
    L.exl3o_pack_tile_half(p16(codes), KA, p16(tile))
    st = np.zeros(256, np.uint16)
    L.exl3o_tile_states_half(p16(tile), KA, p16(st))
    for t in range(256):
        nb = KA + (t & 1)
        assert (int(st[t]) ^ int(codes[t])) & ((1 << nb) - 1) == 0
    # numpy: the tile as a bit array (uint32 words, MSB first), windows by slicing
    tile = rng.integers(0, 65536, 8 * bits2).astype(np.uint16)
    words = tile[0::2].astype(np.uint32) | (tile[1::2].astype(np.uint32) << 16)
    bits = ((words[:, None] >> (31 - np.arange(32, dtype=np.uint32))) & 1).reshape(-1)
    ring = np.concatenate([bits, bits])
    n = bits.size
    assert n == 128 * bits2
    want = np.zeros(256, np.uint16)
    for t in range(256):
        end = (t // 2 + 1) * bits2 if t & 1 else (t // 2) * bits2 + KA
        start = (end - 16) % n
        w = ring[start:start + 16]
        want[t] = int("".join(str(int(b)) for b in w), 2)
    L.exl3o_tile_states_half(p16(tile), KA, p16(st))
    assert np.array_equal(st, want)
    # through reconstruct: a (16, 16) weight of one tile
    table = oracle.decode_table(2)
    w = oracle.reconstruct(tile.reshape(1, 1, -1), 2)
    for t in range(256):
        l, j = t // 8, t % 8
        row, col = 2 * (l % 4) + (j & 1) + 8 * ((j >> 1) & 1), (l // 4) + 8 * (j >> 2)
        assert w[row, col].view(np.uint16) == table[want[t]].view(np.uint16)
