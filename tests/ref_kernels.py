"""Loader of the reference's own GEMM / GEMV / fused-MoE kernels (oracle/_ref/libexl3_ref_gemm.so,
built by oracle/ref/Makefile.ref from the unmodified reference sources). Test infrastructure: a
second oracle and the bar the timing table compares this library with on the same GPU."""
import ctypes
import os

from conftest import ROOT

SO = os.path.join(ROOT, "oracle", "_ref", "libexl3_ref_gemm.so")
_lib = None


class RefMoeArgs(ctypes.Structure):
    _fields_ = [("x", ctypes.c_void_p), ("bsz", ctypes.c_int), ("H", ctypes.c_int), ("x_stride", ctypes.c_int),
                ("sel", ctypes.c_void_p), ("rw", ctypes.c_void_p), ("topk", ctypes.c_int),
                ("experts", ctypes.c_int), ("Hi", ctypes.c_int), ("I", ctypes.c_int), ("Ho", ctypes.c_int),
                ("tables", ctypes.c_void_p * 9),
                ("K", ctypes.c_int), ("cb", ctypes.c_int), ("act", ctypes.c_int), ("act_limit", ctypes.c_float),
                ("gated", ctypes.c_int),
                ("had_g", ctypes.c_void_p), ("had_u", ctypes.c_void_p), ("gu_g", ctypes.c_void_p), ("gu_u", ctypes.c_void_p),
                ("act_out", ctypes.c_void_p), ("d_out", ctypes.c_void_p),
                ("slots_max", ctypes.c_int), ("rows_max", ctypes.c_int),
                ("ctr", ctypes.c_void_p), ("ctr_len", ctypes.c_long),
                ("out", ctypes.c_void_p), ("H_out", ctypes.c_int)]


def available():
    return os.path.exists(SO)


# ---- the reference's token-sorted prefill MoE (libexl3_ref_moe.so, Makefile.ref target `moe`) ----
MOE_SO = os.path.join(ROOT, "oracle", "_ref", "libexl3_ref_moe.so")
_moe_lib = None


class RefMoeSortedArgs(ctypes.Structure):
    _fields_ = [("y", ctypes.c_void_p), ("out", ctypes.c_void_p), ("count", ctypes.c_void_p), ("tok", ctypes.c_void_p),
                ("w", ctypes.c_void_p),
                ("T", ctypes.c_int), ("H", ctypes.c_int), ("I", ctypes.c_int), ("E", ctypes.c_int), ("A", ctypes.c_long),
                ("tables", ctypes.c_void_p * 9),
                ("K", ctypes.c_int), ("cb", ctypes.c_int), ("act", ctypes.c_int), ("act_limit", ctypes.c_float),
                ("ts_g", ctypes.c_void_p), ("ts_u", ctypes.c_void_p), ("ti_g", ctypes.c_void_p), ("ti_u", ctypes.c_void_p),
                ("conc", ctypes.c_int), ("cap", ctypes.c_int),
                ("lo", ctypes.c_int), ("hi", ctypes.c_int), ("m_tile", ctypes.c_int), ("num_active", ctypes.c_int)]


def moe_available():
    return os.path.exists(MOE_SO)


def moe_lib():
    global _moe_lib
    if _moe_lib is None:
        import torch  # noqa: F401  (libtorch must be loaded first)
        _moe_lib = ctypes.CDLL(MOE_SO)
        _moe_lib.ref_exl3_moe_sorted.argtypes = [ctypes.POINTER(RefMoeSortedArgs), ctypes.c_int]
        _moe_lib.ref_exl3_moe_concurrency.argtypes = [ctypes.c_int]
    return _moe_lib


def lib():
    global _lib
    if _lib is None:
        import torch  # noqa: F401  (libtorch must be loaded first)
        # the reference's autotuner keeps a cache file: keep it out of the home directory
        os.environ.setdefault("EXLLAMAV3_TUNE_CACHE", "/tmp/exl3_ref_autotune.bin")
        _lib = ctypes.CDLL(SO)
        vp, i = ctypes.c_void_p, ctypes.c_int
        _lib.ref_exl3_gemm.argtypes = [vp] * 6 + [i] * 7
        _lib.ref_exl3_mgemm.argtypes = [vp] * 6 + [i] * 7 + [vp] * 4 + [i]
        _lib.ref_exl3_moe_coop.argtypes = [ctypes.POINTER(RefMoeArgs), i]
    return _lib


def gemm(x, trellis, out, suh, svh, a_had, cb=0):
    """out (m, n) = the reference's exl3_gemm of x (m, k) through its own dispatch; returns the
    kernel shape index it reports (90 = its GEMV kernel)."""
    m, k = x.shape
    n = trellis.shape[1] * 16
    K = trellis.shape[2] // 16
    rc = lib().ref_exl3_gemm(x.data_ptr(), trellis.data_ptr(), out.data_ptr(), suh.data_ptr(), a_had.data_ptr(),
                             svh.data_ptr(), m, k, n, K, cb, int(out.dtype.itemsize == 4), x.get_device())
    assert rc >= 0, "reference exl3_gemm raised"
    return rc


def mgemm(x, b_ptrs, c, suh_ptrs, a_had, svh_ptrs, num, num_src, m, k, width, K, cb=0, opts=None):
    o = opts or {}
    p = lambda key: o[key].data_ptr() if key in o else None
    rc = lib().ref_exl3_mgemm(x.data_ptr(), b_ptrs.data_ptr(), c.data_ptr(), suh_ptrs.data_ptr(), a_had.data_ptr(),
                              svh_ptrs.data_ptr(), num, num_src, m, k, width, K, cb,
                              p("size_n_list"), p("c_ptrs"), p("n_stride_list"), p("had_src_list"), x.get_device())
    assert rc >= 0, "reference exl3_mgemm raised"
    return rc
