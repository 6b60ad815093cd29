"""ctypes/numpy front end of oracle/libexl3_oracle.so (the CPU restatement of the reference's
EXL3 arithmetic). TEST INFRASTRUCTURE ONLY: used by tests/, __graft_entry__.smoke() and the
CPU-baseline legs of bench.py as the checker; the package never imports it.

fp16 data is exchanged as numpy float16 arrays; trellis tensors as uint16 (or int16) arrays of
shape (k/16, n/16, 16*K), exactly the on-disk layout the reference loads
(src/ucode/ampstein/models.uc:9-15).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

_u16p = ctypes.POINTER(ctypes.c_uint16)
_f32p = ctypes.POINTER(ctypes.c_float)


def build(force=False):
    """Compile the C restatement with the Makefile beside it."""
    so = os.path.join(_HERE, "libexl3_oracle.so")
    src = os.path.join(_HERE, "exl3_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "-B", "libexl3_oracle.so"])
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
        _LIB.exl3o_h2f.restype = ctypes.c_float
        _LIB.exl3o_h2f.argtypes = [ctypes.c_uint16]
        _LIB.exl3o_f2h.restype = ctypes.c_uint16
        _LIB.exl3o_f2h.argtypes = [ctypes.c_float]
        _LIB.exl3o_d2h.restype = ctypes.c_uint16
        _LIB.exl3o_d2h.argtypes = [ctypes.c_double]
        _LIB.exl3o_decode_state.restype = ctypes.c_uint16
        _LIB.exl3o_decode_state.argtypes = [ctypes.c_uint32, ctypes.c_int]
    return _LIB


def _p16(a):
    return a.ctypes.data_as(_u16p)


def _p32(a):
    return a.ctypes.data_as(_f32p)


def _h(a):
    """contiguous uint16 view of an fp16 / uint16 / int16 array"""
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16 or a.dtype == np.int16:
        return a.view(np.uint16)
    assert a.dtype == np.uint16, a.dtype
    return a


def trellis_dims(trellis):
    """(k, n, K) of a trellis tensor (k/16, n/16, 16 K); K is 1.5 / 2.5 / 3.5 for the half-integer
    rates, whose third dimension is 16 KA + 8."""
    tk, tn, w = trellis.shape
    assert w % 8 == 0
    return tk * 16, tn * 16, (w // 16 if w % 16 == 0 else w / 16.0)


def _is_half(K):
    return float(K) != int(K)


def decode_table(cb):
    """fp16 value of every 16-bit state (65536 entries)."""
    L = lib()
    out = np.empty(65536, np.uint16)
    for s in range(65536):
        out[s] = L.exl3o_decode_state(s, cb)
    return out.view(np.float16)


def tile_states(tile, K):
    t = _h(tile).reshape(-1)
    assert t.size == 16 * K
    out = np.empty(256, np.uint16)
    lib().exl3o_tile_states(_p16(t), K, _p16(out))
    return out


def pack_tile(codes, K):
    c = np.ascontiguousarray(codes, dtype=np.uint16)
    out = np.zeros(16 * K, np.uint16)
    lib().exl3o_pack_tile(_p16(c), K, _p16(out))
    return out


def tile_pos(t):
    r, c = ctypes.c_int(), ctypes.c_int()
    lib().exl3o_tile_pos(t, ctypes.byref(r), ctypes.byref(c))
    return r.value, c.value


def reconstruct(trellis, cb=0):
    t = _h(trellis)
    k, n, K = trellis_dims(t)
    out = np.empty((k, n), np.uint16)
    if _is_half(K):
        rc = lib().exl3o_reconstruct_half(_p16(t), k, n, int(K), cb, _p16(out))
    else:
        rc = lib().exl3o_reconstruct(_p16(t), k, n, K, cb, _p16(out))
    assert rc == 0, rc
    return out.view(np.float16)


def reconstruct_had(trellis, suh, svh, cb=0):
    t = _h(trellis)
    k, n, K = trellis_dims(t)
    out = np.empty((k, n), np.uint16)
    if _is_half(K):
        what = np.ascontiguousarray(_h(reconstruct(t, cb)))
        rc = lib().exl3o_reconstruct_had_w(_p16(what), _p16(_h(suh)), _p16(_h(svh)), k, n, _p16(out))
    else:
        rc = lib().exl3o_reconstruct_had(_p16(t), _p16(_h(suh)), _p16(_h(svh)), k, n, K, cb, _p16(out))
    assert rc == 0, rc
    return out.view(np.float16)


def had_hf(x, pre=None, post=None, scale=1.0):
    xx = _h(x)
    rows, cols = xx.shape
    out = np.empty_like(xx)
    lib().exl3o_had_hf(_p16(xx), _p16(out), rows, cols,
                       _p16(_h(pre)) if pre is not None else None,
                       _p16(_h(post)) if post is not None else None, ctypes.c_float(scale))
    return out.view(np.float16)


def had_fh(x, post=None, scale=1.0):
    xx = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = xx.shape
    out = np.empty((rows, cols), np.uint16)
    lib().exl3o_had_fh(_p32(xx), _p16(out), rows, cols,
                       _p16(_h(post)) if post is not None else None, ctypes.c_float(scale))
    return out.view(np.float16)


def had_ff(x, post=None, scale=1.0):
    xx = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = xx.shape
    out = np.empty((rows, cols), np.float32)
    lib().exl3o_had_ff(_p32(xx), _p32(out), rows, cols,
                       _p16(_h(post)) if post is not None else None, ctypes.c_float(scale))
    return out


def linear(x, trellis, suh, svh, cb=0, fp32_out=False, what=None):
    """y = had(x*suh) @ W_hat -> had(.)*svh with fp32 accumulation (the reference's
    reconstruct-then-matmul semantics). Returns fp16 (m,n), or fp32 when fp32_out."""
    xx = _h(x)
    m, k = xx.shape
    t = _h(trellis)
    kk, n, K = trellis_dims(t)
    assert kk == k
    o16 = np.empty((m, n), np.uint16)
    o32 = np.empty((m, n), np.float32)
    if what is None and _is_half(K):
        what = reconstruct(t, cb)
    if what is None:
        rc = lib().exl3o_linear(_p16(xx), _p16(t), _p16(_h(suh)), _p16(_h(svh)), m, k, n, K, cb,
                                _p16(o16), _p32(o32))
    else:
        rc = lib().exl3o_linear_w(_p16(xx), _p16(_h(what)), _p16(_h(suh)), _p16(_h(svh)), m, k, n,
                                  _p16(o16), _p32(o32))
    assert rc == 0, rc
    return o32 if fp32_out else o16.view(np.float16)


def linear_int8(x, trellis, suh, svh, fp32_out=False, residual=False):
    """The mul1 (cb 2) linear with int8-quantised rotated activations, one scale per 128 rows of k
    (the arithmetic of the int8-activation GEMV); residual: with the error-feedback codes (the
    rounding error quantised again at scale q / 254). Returns fp16 (m,n), or fp32 when fp32_out."""
    xx = _h(x)
    m, k = xx.shape
    t = _h(trellis)
    kk, n, K = trellis_dims(t)
    assert kk == k
    o16 = np.empty((m, n), np.uint16)
    o32 = np.empty((m, n), np.float32)
    fn = lib().exl3o_linear_int8_residual if residual else lib().exl3o_linear_int8
    rc = fn(_p16(xx), _p16(t), _p16(_h(suh)), _p16(_h(svh)), m, k, n, K, _p16(o16), _p32(o32))
    assert rc == 0, rc
    return o32 if fp32_out else o16.view(np.float16)


def silu_mul(g, u):
    """fp16(silu(g) * u) with fp32 math (reference: amp_silu_mul_kernel, src/torch/amp_kernels.cu:235-251)."""
    gf = np.asarray(g, np.float16).astype(np.float32)
    uf = np.asarray(u, np.float16).astype(np.float32)
    s = gf / (np.float32(1.0) + np.exp(-gf, dtype=np.float32))
    return (s * uf).astype(np.float16)


def rms_norm_res(x, res, w, eps):
    """(y, n): y = fp16(x + res); n = fp16(y * rsqrt(mean(y^2) + eps)) * w in fp16 (reference:
    amp_rms_norm_res_kernel, src/torch/amp_kernels.cu:279-360). The mean is formed in float64 here
    (the kernel's fp32 sum order is a property of its launch), which can move the scale by one fp32 ulp."""
    xf = np.asarray(x, np.float16).astype(np.float32)
    rf = np.asarray(res, np.float16).astype(np.float32)
    y = (xf + rf).astype(np.float16)
    yf = y.astype(np.float32)
    scale = (1.0 / np.sqrt(np.mean(yf.astype(np.float64) ** 2, axis=-1, keepdims=True) + eps)).astype(np.float32)
    n = (yf * scale).astype(np.float16) * np.asarray(w, np.float16)
    return y, n.astype(np.float16)


def matmul_f32(a, w):
    aa, ww = _h(a), _h(w)
    m, k = aa.shape
    k2, n = ww.shape
    assert k == k2
    y = np.empty((m, n), np.float32)
    rc = lib().exl3o_matmul_f32(_p16(aa), _p16(ww), m, k, n, _p32(y))
    assert rc == 0, rc
    return y


def allreduce_fp16(parts):
    ps = [_h(p).reshape(-1) for p in parts]
    n = ps[0].size
    arr = (_u16p * len(ps))(*[_p16(p) for p in ps])
    out = np.empty(n, np.uint16)
    lib().exl3o_allreduce_fp16(arr, len(ps), ctypes.c_long(n), _p16(out))
    return out.view(np.float16)


def num_threads():
    return lib().exl3o_num_threads()


def moe_coop(x, sel, rw, experts, act=0, act_limit=0.0, gated=True, min_expert=-1, max_expert=-1,
             cb=0, H_out=None, sh_out=None, sh_gate_w=None, gu_f16=False, biases=None):
    """Fused decode MoE on the CPU. experts: list of dicts with keys gate/up/down, each a
    (trellis, suh, svh) triple (gate may be None when not gated). Returns fp32 (bsz, H_out)."""
    xx = _h(x)
    bsz, H = xx.shape
    topk = sel.shape[1]
    up0, dn0 = experts[0]["up"], experts[0]["down"]
    Hi, I, _ = trellis_dims(_h(up0[0]))
    _, Ho, _ = trellis_dims(_h(dn0[0]))
    H_out = H if H_out is None else H_out
    keep, tabs = [], {}
    PP = ctypes.POINTER(ctypes.c_uint16)

    def table(fn):
        arr = (PP * len(experts))()
        for i, e in enumerate(experts):
            a = fn(e)
            if a is None:
                arr[i] = None
            else:
                a = np.ascontiguousarray(_h(a))
                keep.append(a)
                arr[i] = _p16(a)
        return arr

    whats = {}
    for name in ("gate", "up", "down"):
        whats[name] = table(lambda e, n=name: reconstruct(e[n][0], cb) if e.get(n) is not None else None)
        tabs[name + "_suh"] = table(lambda e, n=name: e[n][1] if e.get(n) is not None else None)
        tabs[name + "_svh"] = table(lambda e, n=name: e[n][2] if e.get(n) is not None else None)
    bias_t = []
    for name in ("gate", "up", "down"):
        if biases is not None and biases.get(name) is not None:
            bias_t.append(table(lambda e, n=name, bb=biases: bb[n][experts.index(e)]))
        else:
            bias_t.append(None)
    selc = np.ascontiguousarray(sel, dtype=np.int64)
    rwc = np.ascontiguousarray(_h(rw))
    out = np.zeros((bsz, H_out), np.float32)
    sh = np.ascontiguousarray(sh_out, dtype=np.float32) if sh_out is not None else None
    shg = np.ascontiguousarray(_h(sh_gate_w)) if sh_gate_w is not None else None
    L = lib()
    L.exl3o_moe_coop.restype = ctypes.c_int
    rc = L.exl3o_moe_coop(
        _p16(xx), ctypes.c_int(xx.strides[0] // 2), selc.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)), _p16(rwc),
        bsz, topk, H, Hi, I, Ho, H_out, min_expert, max_expert, len(experts),
        whats["gate"], whats["up"], whats["down"],
        tabs["gate_suh"], tabs["up_suh"], tabs["down_suh"],
        tabs["gate_svh"], tabs["up_svh"], tabs["down_svh"],
        bias_t[0], bias_t[1], bias_t[2],
        act, ctypes.c_float(act_limit), int(gated), int(gu_f16),
        _p32(sh) if sh is not None else None, _p16(shg) if shg is not None else None,
        _p32(out), ctypes.c_int(out.strides[0] // 4))
    assert rc == 0, rc
    return out
