"""B200-native EXL3 quantized-linear kernels behind Ampstein's operator boundary.

The package is a thin host layer over libampstein_b200.so (hand-written sm_100a CUDA behind a
C ABI, see include/ampstein_b200.h). There is no CPU or library fallback: every operator
raises if the shared library is missing or the tensors are not on a CUDA device.
"""
from . import _lib  # noqa: F401
from .exl3 import (  # noqa: F401
    exl3_gemm,
    exl3_gemm_add_res,
    exl3_gemm_normed,
    exl3_gemm_recon,
    exl3_gemm_rms_norm_res,
    exl3_gemm_silu_mul,
    exl3_reconstruct,
    exl3_reconstruct_batch,
    exl3_reconstruct_had,
    had_r_128,
    lm_head_argmax,
    mgemm,
    mgemm_normed,
    mgemm_rms_norm_res,
    moe_coop,
    moe_fused,
    moe_fused_status,
    exl3_shard_cols,
    exl3_shard_rows,
    moe_gather,
    moe_prep,
    moe_sort_routing,
    moe_coop_ctr_len,
    ptr_array,
    rms_norm_res,
    silu_mul,
    argmax_advance,
)

__all__ = ["exl3_gemm", "exl3_gemm_add_res", "exl3_gemm_normed", "exl3_gemm_recon", "exl3_gemm_rms_norm_res", "exl3_gemm_silu_mul", "exl3_reconstruct", "exl3_reconstruct_batch", "exl3_reconstruct_had", "had_r_128", "lm_head_argmax", "mgemm", "mgemm_normed", "mgemm_rms_norm_res", "moe_coop", "moe_coop_ctr_len", "moe_fused", "moe_fused_status", "exl3_shard_cols", "exl3_shard_rows", "moe_gather", "moe_prep", "moe_sort_routing", "ptr_array", "rms_norm_res", "silu_mul", "argmax_advance"]
