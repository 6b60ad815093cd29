"""ctypes binding of libampstein_b200.so. Loading is lazy but loud: a missing or stale library
raises, nothing falls back to another implementation."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libampstein_b200.so")

_lib = None

_vp = ctypes.c_void_p
_i = ctypes.c_int
_l = ctypes.c_long
_f = ctypes.c_float

# name -> argtypes; every entry returns int except where noted. Mirrors include/ampstein_b200.h.
SIGNATURES = {
    "amp_b200_version": [],
    "amp_exl3_reconstruct": [_vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "amp_exl3_reconstruct_had": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "amp_had_r_128": [_vp, _vp, _vp, _vp, _l, _i, _i, _f, _vp],
    "amp_exl3_gemv": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "amp_exl3_gemv_allreduce": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _i, _i, ctypes.c_long, _vp],
    "amp_exl3_gemv_push": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _i, _i, ctypes.c_long, _vp],
    "amp_exl3_gemv_gathered": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, ctypes.c_long, _vp],
    "amp_exl3_mgemm_gathered": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, ctypes.c_long, _vp],
    "amp_exl3_gemv_static": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "amp_exl3_gemv_cfg": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "amp_exl3_gemv_status": [ctypes.POINTER(ctypes.c_int)],
    "amp_exl3_mgemm": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _i, _vp],
    "amp_exl3_mgemm_bf16": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _i, _vp],
    "amp_exl3_set_pdl": [_i],
    "amp_exl3_set_gemv_tc": [_i],
    "amp_diag_issue_cycles": [_i, _i, ctypes.POINTER(ctypes.c_float)],
    "amp_exl3_reconstruct_batch": [_vp, _vp, _i, _i, _i, _i, _i, _vp],
    "amp_exl3_reconstruct_had_batch": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "amp_exl3_gemv_silu_mul": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "amp_exl3_gemv_rms_norm_res": [_vp, _vp, _vp, ctypes.c_float, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "amp_exl3_mgemm_rms_norm_res": [_vp, _vp, _vp, ctypes.c_float, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp],
    "amp_exl3_gemv_allreduce_rot": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _i, _i, ctypes.c_long, _vp, _vp],
    "amp_exl3_lm_head_argmax": [_vp, _vp, _vp, ctypes.c_float, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, ctypes.c_longlong, _vp, _vp],
    "amp_b200_rms_norm_res": [_vp, _vp, _vp, _vp, _vp, ctypes.c_long, _i, ctypes.c_float, _vp],
    "amp_b200_silu_mul": [_vp, _vp, _vp, ctypes.c_long, _vp],
    "amp_b200_argmax_advance": [_vp, _i, _vp, _vp, _vp, ctypes.c_longlong, _vp, _vp],
    "amp_exl3_gemv_add_res": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "amp_exl3_gemv_normed": [_vp, _vp, _vp, ctypes.c_float, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "amp_exl3_mgemm_normed": [_vp, _vp, _vp, ctypes.c_float, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp],
    "amp_exl3_set_gemm_pair": [_i],
    "amp_exl3_set_int8_gemv": [_i, _i],
    "amp_exl3_set_gemm_relay_release": [_i],
    "amp_comm_allreduce_fp16": [_vp, _vp, _vp, _vp, _i, _i, _l, _l, _i, _i, _vp],
    "amp_comm_buffer_bytes": [_i, _l],
    "amp_comm_ctl_bytes": [],
    "amp_comm_blocks": [_i, _l],
    "amp_comm_status": [_vp, ctypes.POINTER(ctypes.c_int)],
    "amp_comm_enable_peer": [_i],
    "amp_comm_ipc_alloc": [_l, ctypes.POINTER(ctypes.c_void_p), _vp],
    "amp_comm_ipc_open": [_vp, ctypes.POINTER(ctypes.c_void_p)],
    "amp_comm_ipc_close": [_vp],
    "amp_comm_free": [_vp],
    "amp_exl3_moe_coop": [_vp, _vp],
    "amp_exl3_moe_coop_ctr_len": [_l, _l, _l, _l],
    "amp_exl3_moe_sorted": [_vp, _vp],
    "amp_exl3_moe_sorted_workspace": [_l, _l, _l, _l, _l],
    "amp_exl3_moe_sorted_status": [_vp, ctypes.POINTER(ctypes.c_int), _vp],
    "amp_exl3_set_moe_sorted_tile": [_i],
    "amp_exl3_shard_cols": [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _vp],
    "amp_exl3_shard_rows": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "amp_moe_prep": [_vp, _vp, _i, _i, _i, ctypes.c_longlong, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "amp_exl3_moe_gather": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _l, _vp],
    "amp_exl3_gemm_bf16": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "amp_exl3_gemm_status": [ctypes.POINTER(ctypes.c_int)],
    "amp_exl3_gemm": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
}


class AmpError(RuntimeError):
    """Raised for every non-zero return code of the C ABI."""

    def __init__(self, fn, rc, msg):
        super().__init__("%s failed (rc=%d): %s" % (fn, rc, msg))
        self.rc = rc


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "ampstein_b200: %s is missing; build it with `python -m ampstein_b200.build` "
                "(there is no fallback path)" % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(L, name)          # AttributeError here = stale library
            fn.argtypes = args
            fn.restype = ctypes.c_int
        L.amp_exl3_moe_coop_ctr_len.restype = ctypes.c_long
        L.amp_exl3_moe_sorted_workspace.restype = ctypes.c_long
        L.amp_comm_buffer_bytes.restype = ctypes.c_long
        L.amp_comm_ctl_bytes.restype = ctypes.c_long
        L.amp_b200_last_error.restype = ctypes.c_char_p
        L.amp_b200_last_error.argtypes = []
        _lib = L
    return _lib


def last_error():
    return lib().amp_b200_last_error().decode("utf-8", "replace")


def call(name, *args):
    """Call a C-ABI entry point; raise AmpError on a non-zero return code."""
    rc = getattr(lib(), name)(*args)
    if rc != 0:
        raise AmpError(name, rc, last_error())
    return rc
