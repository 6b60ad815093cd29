"""Host-side mirror of the operators Ampstein's native module exposes for the EXL3 path
(reference: src/torch/amp_torch.cpp, handlers torch_exl3_reconstruct :11015-11060,
torch_exl3_gemm :11250-11293, torch_exl3_gemm_recon :11148-11230). Same argument order, same
meaning, same error behaviour (bad arguments raise; nothing returns None). Tensors are torch
CUDA tensors; torch only supplies device memory and the current stream, the work is done by
libampstein_b200.so.
"""
import torch

from . import _lib


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _check_cuda(name, *ts):
    for t in ts:
        if not isinstance(t, torch.Tensor):
            raise TypeError("%s: expected torch tensors" % name)
        if not t.is_cuda:
            raise RuntimeError("%s: tensors must live on a CUDA device (no CPU path exists)" % name)
        if not t.is_contiguous():
            raise ValueError("%s: tensors must be contiguous" % name)


def _cb(mul1, mcg):
    if mul1 and mcg:
        raise ValueError("Specified both mcg and mul1")
    return 2 if mul1 else (1 if mcg else 0)


def _trellis_dims(name, trellis, half_ok=False):
    """(k, n, K) of a trellis tensor (k/16, n/16, 16 K). With half_ok the half-integer rates 1.5 / 2.5 /
    3.5 (third dimension 16 KA + 8) are accepted and K comes back as a float."""
    if trellis.dim() != 3:
        raise ValueError("%s: trellis must be 3-D" % name)
    if trellis.dtype not in (torch.int16, torch.uint16):
        raise TypeError("%s: trellis must be int16" % name)
    w = trellis.shape[2]
    if half_ok and w % 16 == 8 and 1 <= w // 16 <= 3:
        return trellis.shape[0] * 16, trellis.shape[1] * 16, w / 16.0
    if w % 16 != 0 or not (1 <= w // 16 <= 8):
        raise ValueError("%s: unsupported EXL3 bitrate %s (integer 1..8%s)" % (name, w / 16, ", or 1.5 / 2.5 / 3.5" if half_ok else ""))
    return trellis.shape[0] * 16, trellis.shape[1] * 16, w // 16


def _kcode(name, K, mul1):
    """K as the C ABI takes it: the integer, or AMP_EXL3_HALF_RATE(KA) = 256 + KA for KA + 0.5."""
    if float(K) == int(K):
        return int(K)
    if not mul1:
        raise ValueError("%s: half-integer bitrates require the mul1 codebook" % name)
    return 256 + int(K)


def exl3_reconstruct(unpacked, packed, K, mul1=False, mcg=False):
    """Dequantize an EXL3 trellis tensor into `unpacked` (fp16 (k, n), in place); returns it.
    K is the bitrate (packed.shape[-1] / 16)."""
    _check_cuda("exl3_reconstruct", unpacked, packed)
    k, n, Kt = _trellis_dims("exl3_reconstruct", packed, half_ok=True)
    if float(K) != float(Kt):
        raise ValueError("exl3_reconstruct: K=%s does not match the trellis (%s)" % (K, Kt))
    if unpacked.dtype != torch.float16 or unpacked.dim() != 2:
        raise TypeError("exl3_reconstruct: unpacked must be 2-D float16")
    if unpacked.shape[0] != k or unpacked.shape[1] != n:
        raise ValueError("exl3_reconstruct: unpacked must be (%d, %d)" % (k, n))
    with torch.cuda.device(packed.device):
        _lib.call("amp_exl3_reconstruct", unpacked.data_ptr(), packed.data_ptr(), k, n, _kcode("exl3_reconstruct", Kt, mul1),
                  _cb(mul1, mcg), 0, n, _stream(packed))
    return unpacked


def exl3_reconstruct_had(unpacked, packed, suh, svh, K, mul1=False, mcg=False, n_offset=0):
    """Original-basis weight diag(suh) H W_hat H diag(svh) / 128 for columns
    [n_offset, n_offset + unpacked.shape[1]); svh is the slice's own vector (reference:
    reconstruct_had_slice, vendor/exl3/exllamav3_ext/quant/reconstruct.cu:431-503)."""
    _check_cuda("exl3_reconstruct_had", unpacked, packed, suh, svh)
    k, n, Kt = _trellis_dims("exl3_reconstruct_had", packed, half_ok=True)
    if float(K) != float(Kt):
        raise ValueError("exl3_reconstruct_had: K does not match the trellis")
    if unpacked.dtype != torch.float16 or suh.dtype != torch.float16 or svh.dtype != torch.float16:
        raise TypeError("exl3_reconstruct_had: unpacked, suh, svh must be float16")
    if unpacked.dim() != 2 or unpacked.shape[0] != k:
        raise ValueError("exl3_reconstruct_had: unpacked must have %d rows" % k)
    if suh.numel() < k or svh.numel() < unpacked.shape[1]:
        raise ValueError("reconstruct_had: suh / svh size")
    with torch.cuda.device(packed.device):
        _lib.call("amp_exl3_reconstruct_had", unpacked.data_ptr(), packed.data_ptr(), suh.data_ptr(),
                  svh.data_ptr(), k, n, _kcode("exl3_reconstruct_had", Kt, mul1), _cb(mul1, mcg), int(n_offset), unpacked.shape[1],
                  _stream(packed))
    return unpacked


def exl3_reconstruct_batch(unpacked, packed_ptrs, K, mul1=False, mcg=False, suh_ptrs=None, svh_ptrs=None):
    """Dequantize B matrices of one shape in one launch into unpacked (B, k, n) fp16; packed_ptrs is
    an int64 CUDA tensor of trellis addresses. With suh_ptrs / svh_ptrs the original-basis form
    (reference: reconstruct_batch / reconstruct_had_batch,
    vendor/exl3/exllamav3_ext/quant/reconstruct.cu:512-626)."""
    _check_cuda("exl3_reconstruct_batch", unpacked, packed_ptrs)
    if unpacked.dtype != torch.float16 or unpacked.dim() != 3:
        raise TypeError("exl3_reconstruct_batch: unpacked must be 3-D float16")
    if float(K) != int(K) or not (1 <= int(K) <= 8):
        raise ValueError("exl3_reconstruct_batch: unsupported EXL3 bitrate %s" % K)
    tables = [packed_ptrs] + [t for t in (suh_ptrs, svh_ptrs) if t is not None]
    if (suh_ptrs is None) != (svh_ptrs is None):
        raise TypeError("exl3_reconstruct_batch: suh_ptrs and svh_ptrs go together")
    B, k, n = unpacked.shape
    for t in tables:
        _check_cuda("exl3_reconstruct_batch", t)
        if t.dtype != torch.int64 or t.numel() < B:
            raise ValueError("exl3_reconstruct_batch: pointer tables must be int64 with one entry per matrix")
    with torch.cuda.device(unpacked.device):
        if suh_ptrs is None:
            _lib.call("amp_exl3_reconstruct_batch", unpacked.data_ptr(), packed_ptrs.data_ptr(), B, k, n, int(K),
                      _cb(mul1, mcg), _stream(unpacked))
        else:
            _lib.call("amp_exl3_reconstruct_had_batch", unpacked.data_ptr(), packed_ptrs.data_ptr(), suh_ptrs.data_ptr(),
                      svh_ptrs.data_ptr(), B, k, n, int(K), _cb(mul1, mcg), _stream(unpacked))
    return unpacked


def had_r_128(input, output, pre_scale=None, post_scale=None, scale=1.0):
    """output = blockwise H128(input [* pre_scale]) * scale / sqrt(128) [* post_scale]; fp16 or
    fp32, may run in place; an fp32 input with an fp16 output runs the transform in fp32 and
    rounds once (reference: had_r_128, .../quant/hadamard.cu:125-207; the mixed form is
    had_fh_r_128_inner, .../quant/hadamard_inner.cuh:216-279)."""
    ts = [input, output] + [t for t in (pre_scale, post_scale) if t is not None]
    _check_cuda("had_r_128", *ts)
    if input.shape != output.shape or input.dim() != 2:
        raise ValueError("had_r_128: input and output must be 2-D and of one shape")
    mixed = input.dtype == torch.float32 and output.dtype == torch.float16
    if (input.dtype != output.dtype and not mixed) or input.dtype not in (torch.float16, torch.float32):
        raise TypeError("had_r_128: unsupported datatype")
    if mixed and input.data_ptr() == output.data_ptr():
        raise ValueError("had_r_128: the fp32 -> fp16 form cannot run in place")
    rows, cols = input.shape
    if cols % 128:
        raise ValueError("had_r_128: columns must be divisible by 128")
    for s in (pre_scale, post_scale):
        if s is not None and (s.dtype != torch.float16 or s.numel() < cols):
            raise ValueError("had_r_128: scale vectors must be float16 with one value per column")
    with torch.cuda.device(input.device):
        _lib.call("amp_had_r_128", input.data_ptr(), output.data_ptr(),
                  pre_scale.data_ptr() if pre_scale is not None else None,
                  post_scale.data_ptr() if post_scale is not None else None,
                  rows, cols, 3 if mixed else (1 if input.dtype == torch.float32 else 0), float(scale), _stream(input))
    return output


def exl3_gemm(A, B, C, suh, svh, mul1=False, mcg=False):
    """C = had(A * suh) @ dequant(B) -> had(.) * svh, written in place; returns C.
    A (m, k) fp16, B trellis (k/16, n/16, 16K) int16, C (m, n) fp16 or fp32, suh (k), svh (n).
    Both scale vectors are required (reference: torch_exl3_gemm)."""
    if suh is None or svh is None:
        raise TypeError("expected (A, B, C, suh, svh, mul1?, mcg?)")
    _check_cuda("exl3_gemm", A, B, C, suh, svh)
    k, n, K = _trellis_dims("exl3_gemm", B, half_ok=True)
    if A.dtype not in (torch.float16, torch.bfloat16) or suh.dtype != torch.float16 or svh.dtype != torch.float16:
        raise TypeError("exl3_gemm: A must be float16 (or bfloat16), suh and svh float16")
    if C.dtype not in (torch.float16, torch.float32):
        raise TypeError("exl3_gemm: C must be float16 or float32")
    if A.shape[-1] != k or C.shape[-1] != n:
        raise ValueError("exl3_gemm: incompatible shapes (A %s, weight %d x %d, C %s)"
                         % (tuple(A.shape), k, n, tuple(C.shape)))
    m = A.numel() // k
    if C.numel() != m * n or suh.numel() != k or svh.numel() != n:
        raise ValueError("exl3_gemm: incompatible shapes")
    if m == 0:
        return C
    bf16 = A.dtype == torch.bfloat16
    half_rate = float(K) != int(K)
    if half_rate and (m > 16 or bf16):
        # half-integer bitrates, many rows: the weight is decoded once into the original basis
        # (reconstruct_had) and multiplied by a library GEMM, the reference's form of this case
        # (torch_exl3_gemm_recon, src/torch/amp_torch.cpp:11128-11230)
        w = torch.empty((k, n), dtype=torch.float16, device=A.device)
        exl3_reconstruct_had(w, B, suh, svh, K, mul1, mcg)
        y = torch.mm(A.reshape(m, k).to(torch.float16), w)
        C.copy_(y.reshape(C.shape))
        return C
    K = _kcode("exl3_gemm", K, mul1)
    # the binding allocates the input-rotation scratch per call, as the reference's does
    # (src/torch/amp_torch.cpp:11282); the decode kernel (<= 16 rows) does not need it
    # (from five rows on it lets the input be rotated once instead of by every CTA; the half-rate
    # kernel always takes its input rotated)
    A_had = torch.empty(A.shape, dtype=torch.float16, device=A.device) if (m >= 5 or bf16 or half_rate) else None
    with torch.cuda.device(A.device):
        _lib.call("amp_exl3_gemm_bf16" if bf16 else "amp_exl3_gemm", A.data_ptr(), B.data_ptr(), C.data_ptr(),
                  suh.data_ptr(), A_had.data_ptr() if A_had is not None else None, svh.data_ptr(), m, k, n, K,
                  _cb(mul1, mcg), 1 if C.dtype == torch.float32 else 0, _stream(A))
    return C


def exl3_gemm_silu_mul(gate, up, B, C, suh, svh, mul1=False, mcg=False):
    """C = linear(silu(gate) * up) in ONE launch: the gated activation of the decode step
    (reference: torch.silu_mul followed by torch.exl3_gemm, src/ucode/ampstein/graphdec.uc:205-217)
    folded into the input side of the down projection. gate / up (m, k) fp16 with m <= 16; the rest
    as exl3_gemm. Returns C."""
    _check_cuda("exl3_gemm_silu_mul", gate, up, B, C, suh, svh)
    k, n, K = _trellis_dims("exl3_gemm_silu_mul", B)
    if gate.dtype != torch.float16 or up.dtype != torch.float16 or suh.dtype != torch.float16 or svh.dtype != torch.float16:
        raise TypeError("exl3_gemm_silu_mul: gate, up, suh and svh must be float16")
    if C.dtype not in (torch.float16, torch.float32):
        raise TypeError("exl3_gemm_silu_mul: C must be float16 or float32")
    if gate.shape != up.shape or gate.shape[-1] != k or C.shape[-1] != n:
        raise ValueError("exl3_gemm_silu_mul: incompatible shapes")
    m = gate.numel() // k
    if not 1 <= m <= 16:
        raise ValueError("exl3_gemm_silu_mul: 1..16 rows (larger batches: silu_mul, then exl3_gemm)")
    if C.numel() != m * n or suh.numel() != k or svh.numel() != n:
        raise ValueError("exl3_gemm_silu_mul: incompatible shapes")
    with torch.cuda.device(gate.device):
        _lib.call("amp_exl3_gemv_silu_mul", gate.data_ptr(), up.data_ptr(), B.data_ptr(), C.data_ptr(), suh.data_ptr(),
                  svh.data_ptr(), m, k, n, K, _cb(mul1, mcg), 1 if C.dtype == torch.float32 else 0, _stream(gate))
    return C


def _norm_args(name, x, res, norm_w, y):
    _check_cuda(name, x, res, norm_w, y)
    if any(t.dtype != torch.float16 for t in (x, res, norm_w, y)):
        raise TypeError("%s: x, res, norm_w and y must be float16" % name)
    if x.shape != res.shape or x.shape != y.shape or norm_w.numel() != x.shape[-1]:
        raise ValueError("%s: x, res and y must have one shape, norm_w one value per column" % name)
    if y.data_ptr() in (x.data_ptr(), res.data_ptr()):
        raise ValueError("%s: y must not alias x or res" % name)


def exl3_gemm_rms_norm_res(x, res, norm_w, eps, y, B, C, suh, svh, mul1=False, mcg=False):
    """y = fp16(x + res) (the updated residual stream) and C = linear(RMSNorm(y) * norm_w) in ONE
    launch (reference: torch.rms_norm_res followed by torch.exl3_gemm, e.g. the final norm in front
    of the lm_head, src/ucode/ampstein/graphdec.uc:219-231). x, res, y (m, k) fp16 with m <= 16; y
    must be a buffer of its own. Returns C."""
    _norm_args("exl3_gemm_rms_norm_res", x, res, norm_w, y)
    _check_cuda("exl3_gemm_rms_norm_res", B, C, suh, svh)
    k, n, K = _trellis_dims("exl3_gemm_rms_norm_res", B)
    if C.dtype not in (torch.float16, torch.float32) or suh.dtype != torch.float16 or svh.dtype != torch.float16:
        raise TypeError("exl3_gemm_rms_norm_res: C must be float16 or float32, suh and svh float16")
    m = x.numel() // k
    if x.shape[-1] != k or not 1 <= m <= 16 or C.numel() != m * n or suh.numel() != k or svh.numel() != n:
        raise ValueError("exl3_gemm_rms_norm_res: incompatible shapes (1..16 rows)")
    with torch.cuda.device(x.device):
        _lib.call("amp_exl3_gemv_rms_norm_res", x.data_ptr(), res.data_ptr(), norm_w.data_ptr(), float(eps), y.data_ptr(),
                  B.data_ptr(), C.data_ptr(), suh.data_ptr(), svh.data_ptr(), m, k, n, K, _cb(mul1, mcg),
                  1 if C.dtype == torch.float32 else 0, _stream(x))
    return C


def exl3_gemm_add_res(x, B, suh, svh, h, y, ssq, mul1=False, mcg=False):
    """Producer side of the split residual norm: y (m, n) = fp16(h + linear(x)) and ssq (m, n / 128)
    fp32 = block sums of squares of y, in the launch of the linear itself (o_proj / down_proj). y must
    not alias h. Returns (y, ssq)."""
    _check_cuda("exl3_gemm_add_res", x, B, suh, svh, h, y, ssq)
    k, n, K = _trellis_dims("exl3_gemm_add_res", B)
    m = x.numel() // k
    if any(t.dtype != torch.float16 for t in (x, suh, svh, h, y)) or ssq.dtype != torch.float32:
        raise TypeError("exl3_gemm_add_res: fp16 tensors, fp32 ssq")
    if x.shape[-1] != k or not 1 <= m <= 16 or h.numel() != m * n or y.numel() != m * n or ssq.numel() < m * (n // 128) \
            or y.data_ptr() == h.data_ptr():
        raise ValueError("exl3_gemm_add_res: incompatible shapes (1..16 rows), or y aliases h")
    with torch.cuda.device(x.device):
        _lib.call("amp_exl3_gemv_add_res", x.data_ptr(), B.data_ptr(), suh.data_ptr(), svh.data_ptr(), h.data_ptr(), y.data_ptr(),
                  ssq.data_ptr(), m, k, n, K, _cb(mul1, mcg), _stream(x))
    return y, ssq


def exl3_gemm_normed(y, ssq, norm_w, eps, B, C, suh, svh, mul1=False, mcg=False):
    """Consumer side: C = linear(fp16(y * rsqrt(sum(ssq row) / k + eps)) * norm_w). Returns C."""
    _check_cuda("exl3_gemm_normed", y, ssq, norm_w, B, C, suh, svh)
    k, n, K = _trellis_dims("exl3_gemm_normed", B)
    m = y.numel() // k
    if y.dtype != torch.float16 or norm_w.dtype != torch.float16 or ssq.dtype != torch.float32 or C.dtype not in (torch.float16, torch.float32):
        raise TypeError("exl3_gemm_normed: y, norm_w fp16; ssq fp32; C fp16 or fp32")
    if y.shape[-1] != k or not 1 <= m <= 16 or C.numel() != m * n or ssq.numel() < m * (k // 128) or norm_w.numel() != k:
        raise ValueError("exl3_gemm_normed: incompatible shapes (1..16 rows)")
    with torch.cuda.device(y.device):
        _lib.call("amp_exl3_gemv_normed", y.data_ptr(), ssq.data_ptr(), norm_w.data_ptr(), float(eps), B.data_ptr(), C.data_ptr(),
                  suh.data_ptr(), svh.data_ptr(), m, k, n, K, _cb(mul1, mcg), 1 if C.dtype == torch.float32 else 0, _stream(y))
    return C


def mgemm_normed(y, ssq, norm_w, eps, B_ptrs, C, suh_ptrs, svh_ptrs, K, mcg, mul1, opts=None):
    """Consumer side, bundle form (tables and opts as mgemm; y (1, m, k) fp16, m <= 16). Returns C."""
    _check_cuda("mgemm_normed", y, ssq, norm_w, C)
    if y.dtype != torch.float16 or norm_w.dtype != torch.float16 or ssq.dtype != torch.float32:
        raise TypeError("mgemm_normed: y, norm_w fp16; ssq fp32")
    if y.dim() != 3 or y.shape[0] != 1 or C.dim() != 3:
        raise ValueError("mgemm_normed: y must be (1, m, k) and C (num, m, n)")
    num, m, width = C.shape
    k = y.shape[2]
    if y.shape[1] != m or not 1 <= m <= 16 or ssq.numel() < m * (k // 128) or norm_w.numel() != k:
        raise ValueError("mgemm_normed: 1..16 rows; ssq (m, k / 128); norm_w (k)")
    c_ptrs = n_stride = had_src = None
    if opts is not None:
        c_ptrs, n_stride, had_src = opts["c_ptrs"], opts["n_stride_list"], opts["had_src_list"]
    with torch.cuda.device(y.device):
        _lib.call("amp_exl3_mgemm_normed", y.data_ptr(), ssq.data_ptr(), norm_w.data_ptr(), float(eps),
                  B_ptrs.data_ptr(), C.data_ptr(), suh_ptrs.data_ptr(), svh_ptrs.data_ptr(), num, m, k, width,
                  int(K), _cb(mul1, mcg), 1 if C.dtype == torch.float32 else 0,
                  c_ptrs.data_ptr() if c_ptrs is not None else None,
                  n_stride.data_ptr() if n_stride is not None else None,
                  had_src.data_ptr() if had_src is not None else None, _stream(y))
    return C


def rms_norm_res(x, res, norm_w, eps, y=None, n=None):
    """Stand-alone residual add + RMSNorm (the arithmetic the fused entries apply): returns (y, n),
    y = fp16(x + res), n = fp16(y * rsqrt(mean(y^2) + eps)) * norm_w (reference: torch.rms_norm_res,
    src/torch/amp_kernels.cu:279-360)."""
    y = torch.empty_like(x) if y is None else y
    n = torch.empty_like(x) if n is None else n
    _check_cuda("rms_norm_res", x, res, norm_w, y, n)
    if any(t.dtype != torch.float16 for t in (x, res, norm_w, y, n)) or x.shape != res.shape or norm_w.numel() != x.shape[-1]:
        raise TypeError("rms_norm_res: float16 tensors of one shape, norm_w one value per column")
    dim = x.shape[-1]
    with torch.cuda.device(x.device):
        _lib.call("amp_b200_rms_norm_res", x.data_ptr(), res.data_ptr(), norm_w.data_ptr(), y.data_ptr(), n.data_ptr(),
                  x.numel() // dim, dim, float(eps), _stream(x))
    return y, n


def silu_mul(g, u, out=None):
    """Stand-alone fp16(silu(g) * u) with fp32 math (reference: torch.silu_mul, src/torch/amp_kernels.cu:235-271)."""
    out = torch.empty_like(g) if out is None else out
    _check_cuda("silu_mul", g, u, out)
    if g.dtype != torch.float16 or u.dtype != torch.float16 or out.dtype != torch.float16 or g.shape != u.shape:
        raise TypeError("silu_mul: float16 tensors of one shape")
    with torch.cuda.device(g.device):
        _lib.call("amp_b200_silu_mul", g.data_ptr(), u.data_ptr(), out.data_ptr(), g.numel(), _stream(g))
    return out


def argmax_advance(logits, ids, pos, log, ws):
    """Stand-alone greedy pick + state advance (reference: torch.argmax_advance,
    src/torch/amp_kernels.cu:823-960): log[pos] = ids; ids = argmax(logits); pos += 1."""
    _check_cuda("argmax_advance", logits, ids, pos, log, ws)
    if logits.dtype != torch.float16 or ids.dtype != torch.int64 or pos.dtype != torch.int64 or log.dtype != torch.int64:
        raise TypeError("argmax_advance: logits float16; ids, pos, log int64")
    with torch.cuda.device(logits.device):
        _lib.call("amp_b200_argmax_advance", logits.data_ptr(), logits.numel(), ids.data_ptr(), pos.data_ptr(), log.data_ptr(),
                  log.numel(), ws.data_ptr(), _stream(logits))


def lm_head_argmax(x, res, norm_w, eps, y, B, logits, suh, svh, ids, pos, log, ws, vocab=None, mul1=False, mcg=False):
    """The end of a greedy decode step in ONE launch: y = fp16(x + res); logits (1, n) fp16 = lm_head of
    RMSNorm(y) * norm_w; ids = argmax(logits[:vocab]) after log[pos] = ids, pos += 1 (reference:
    torch.rms_norm_res + torch.exl3_gemm + torch.argmax_advance, src/ucode/ampstein/graphdec.uc:219-240).
    ids, pos: int64 tensors of one element; log: int64; ws: at least 16 bytes of zero-filled device
    memory owned by this decoder (any dtype). Returns logits."""
    _norm_args("lm_head_argmax", x, res, norm_w, y)
    _check_cuda("lm_head_argmax", B, logits, suh, svh, ids, pos, log, ws)
    k, n, K = _trellis_dims("lm_head_argmax", B)
    if logits.dtype != torch.float16 or suh.dtype != torch.float16 or svh.dtype != torch.float16:
        raise TypeError("lm_head_argmax: logits, suh and svh must be float16")
    if x.numel() != k or logits.numel() != n or suh.numel() != k or svh.numel() != n:
        raise ValueError("lm_head_argmax: one row; shapes must match the weight")
    if ids.dtype != torch.int64 or pos.dtype != torch.int64 or log.dtype != torch.int64 or ids.numel() < 1 or pos.numel() < 1:
        raise TypeError("lm_head_argmax: ids, pos and log must be int64 tensors")
    if ws.numel() * ws.element_size() < 16 or ws.data_ptr() % 8:
        raise ValueError("lm_head_argmax: ws must hold at least 16 bytes, 8-byte aligned")
    vocab = n if vocab is None else int(vocab)
    if not 1 <= vocab <= n:
        raise ValueError("lm_head_argmax: vocab out of range")
    with torch.cuda.device(x.device):
        _lib.call("amp_exl3_lm_head_argmax", x.data_ptr(), res.data_ptr(), norm_w.data_ptr(), float(eps), y.data_ptr(),
                  B.data_ptr(), logits.data_ptr(), suh.data_ptr(), svh.data_ptr(), k, n, K, _cb(mul1, mcg), vocab,
                  ids.data_ptr(), pos.data_ptr(), log.data_ptr(), log.numel(), ws.data_ptr(), _stream(x))
    return logits


def mgemm_rms_norm_res(x, res, norm_w, eps, y, B_ptrs, C, suh_ptrs, svh_ptrs, K, mcg, mul1, opts=None):
    """The bundle form: y = fp16(x + res), then every matrix / slice of the bundle applied to
    RMSNorm(y) * norm_w in ONE launch (reference: torch.rms_norm_res followed by the q|k|v or gate|up
    mgemm, src/ucode/ampstein/graphdec.uc:163-172,196-203). x, res, y (1, m, k) fp16, m <= 16; tables
    and opts as mgemm. Returns C."""
    _norm_args("mgemm_rms_norm_res", x, res, norm_w, y)
    for name, t in (("B_ptrs", B_ptrs), ("suh_ptrs", suh_ptrs), ("svh_ptrs", svh_ptrs)):
        if not isinstance(t, torch.Tensor) or t.dtype != torch.int64 or not t.is_cuda:
            raise TypeError("mgemm_rms_norm_res: %s must be an int64 CUDA tensor" % name)
    _check_cuda("mgemm_rms_norm_res", C)
    if x.dim() != 3 or x.shape[0] != 1 or C.dim() != 3 or C.dtype not in (torch.float16, torch.float32):
        raise ValueError("mgemm_rms_norm_res: x must be (1, m, k) and C (num, m, n) float16 or float32")
    num, m, width = C.shape
    k = x.shape[2]
    if x.shape[1] != m or not 1 <= m <= 16:
        raise ValueError("mgemm_rms_norm_res: 1..16 rows, the same in x and C")
    c_ptrs = n_stride = had_src = None
    if opts is not None:
        c_ptrs, n_stride, had_src = opts["c_ptrs"], opts["n_stride_list"], opts["had_src_list"]
        if opts["size_n_list"].numel() != num or c_ptrs.numel() != num:
            raise ValueError("mgemm_rms_norm_res: slice tables do not match C")
    if B_ptrs.numel() < num or svh_ptrs.numel() < num:
        raise ValueError("mgemm_rms_norm_res: pointer tables shorter than the matrix count")
    with torch.cuda.device(x.device):
        _lib.call("amp_exl3_mgemm_rms_norm_res", x.data_ptr(), res.data_ptr(), norm_w.data_ptr(), float(eps), y.data_ptr(),
                  B_ptrs.data_ptr(), C.data_ptr(), suh_ptrs.data_ptr(), svh_ptrs.data_ptr(), num, m, k, width,
                  int(K), _cb(mul1, mcg), 1 if C.dtype == torch.float32 else 0,
                  c_ptrs.data_ptr() if c_ptrs is not None else None,
                  n_stride.data_ptr() if n_stride is not None else None,
                  had_src.data_ptr() if had_src is not None else None, _stream(x))
    return C


# Widest weight that takes the reconstruct-then-matmul form in exl3_gemm_recon. Measured on B200 at
# 256..4096 rows (k = 4096 / 5120, 5 bits): up to 2048 columns the decode-once form is 1.25-2.2x
# faster than the tensor-core trellis GEMM (whose k loop is as long for a narrow weight as for a
# wide one, with most SMs idle), at 4096 columns the two are level, above it the trellis GEMM wins.
RECON_MM_MAX_N = 2048


def exl3_gemm_recon(x, trellis, suh, svh, K, mul1=False, mcg=False, out=None, scratch=None):
    """EXL3 matmul for many rows (prefill); returns a (rows, n) fp16 tensor (reference:
    torch_exl3_gemm_recon, src/torch/amp_torch.cpp:11128-11230). Narrow weights (n <= RECON_MM_MAX_N)
    take the reference's own form of this operator -- the weight decoded ONCE into fp16 with both
    Hadamards and scales folded in (this library's reconstruct_had kernel), then one plain library
    GEMM; wider ones the tensor-core trellis GEMM, which never writes the decoded weight to memory.
    out / scratch: optional preallocated result and (k, n) fp16 buffer for the decoded weight (the
    reference allocates both per call from the caching allocator; so does this function without them)."""
    _check_cuda("exl3_gemm_recon", x, trellis, suh, svh)
    k, n, Kt = _trellis_dims("exl3_gemm_recon", trellis, half_ok=True)
    if x.dim() != 2 or x.shape[1] != k or suh.numel() != k or svh.numel() != n or n > 32768:
        raise ValueError("exl3_gemm_recon: incompatible shapes (x %s, weight %d x %d)"
                         % (tuple(x.shape), k, n))
    if float(K) != float(Kt):
        raise ValueError("exl3_gemm_recon: K does not match the trellis")
    y = out if out is not None else torch.empty((x.shape[0], n), dtype=torch.float16, device=x.device)
    if (n <= RECON_MM_MAX_N or float(Kt) != int(Kt)) and x.dtype == torch.float16 and x.shape[0] > 16:
        w = scratch if scratch is not None else torch.empty((k, n), dtype=torch.float16, device=x.device)
        exl3_reconstruct_had(w, trellis, suh, svh, K, mul1, mcg)
        return torch.mm(x, w, out=y)
    return exl3_gemm(x, trellis, y, suh, svh, mul1, mcg)


def ptr_array(values, device=None):
    """1-D int64 CUDA tensor of raw device addresses: the pointer tables mgemm consumes
    (reference: torch.ptr_array, src/torch/amp_torch.cpp:10332-...)."""
    if not all(isinstance(v, int) for v in values):
        raise TypeError("ptr_array: values must be integers")
    return torch.tensor(list(values), dtype=torch.int64, device=device if device is not None else "cuda")


def mgemm(x, B_ptrs, C, suh_ptrs, A_had, svh_ptrs, K, mcg, mul1, opts=None):
    """Several EXL3 weights against one shared input in ONE launch (reference: torch.mgemm,
    src/torch/amp_torch.cpp:10193-10322). x (1, m, k) fp16; B_ptrs / suh_ptrs / svh_ptrs int64
    CUDA pointer tables; C (num, m, n) stacked output. opts selects sliced mode:
    {size_n_list, c_ptrs, n_stride_list, had_src_list, num_had_src}; C is then only a
    (num_slices, m, width) descriptor. A_had is a (sources, m, k) fp16 scratch, sources =
    num_had_src or num: unused up to 4 rows, optional up to 16 (when given, the input is rotated once
    by a launch of its own), required above (one tensor-core grid over all slices). x may
    be bfloat16 (tensor-core path at any row count; not in the reference). Returns C."""
    for name, t in (("B_ptrs", B_ptrs), ("suh_ptrs", suh_ptrs), ("svh_ptrs", svh_ptrs)):
        if not isinstance(t, torch.Tensor) or t.dtype != torch.int64 or not t.is_cuda:
            raise TypeError("mgemm: %s must be an int64 CUDA tensor" % name)
    _check_cuda("mgemm", x, C)
    if x.dtype not in (torch.float16, torch.bfloat16) or C.dtype not in (torch.float16, torch.float32):
        raise TypeError("mgemm: x must be float16 (or bfloat16), C float16 or float32")
    if x.dim() != 3 or x.shape[0] != 1 or C.dim() != 3:
        raise ValueError("mgemm: x must be (1, m, k) and C (num, m, n)")
    if float(K) != int(K) or not (1 <= int(K) <= 8):
        raise ValueError("mgemm: unsupported EXL3 bitrate %s" % K)
    num, m, width = C.shape
    k = x.shape[2]
    if x.shape[1] != m:
        raise ValueError("mgemm: row count of x and C differ")
    c_ptrs = n_stride = had_src = None
    num_had_src = 0
    if opts is not None:
        if not isinstance(opts, dict):
            raise TypeError("mgemm: opts must be an object")
        want = {"size_n_list": torch.int32, "c_ptrs": torch.int64, "n_stride_list": torch.int32,
                "had_src_list": torch.int32}
        for key, dt in want.items():
            t = opts.get(key)
            if not isinstance(t, torch.Tensor) or t.dtype != dt or not t.is_cuda or not t.is_contiguous():
                raise TypeError("mgemm: opts.%s must be a contiguous %s CUDA tensor" % (key, dt))
        if not isinstance(opts.get("num_had_src"), int):
            raise TypeError("mgemm: num_had_src missing")
        c_ptrs, n_stride, had_src = opts["c_ptrs"], opts["n_stride_list"], opts["had_src_list"]
        num_had_src = opts["num_had_src"]
        if opts["size_n_list"].numel() != num or c_ptrs.numel() != num:
            raise ValueError("mgemm: slice tables do not match C")
    if B_ptrs.numel() < num or svh_ptrs.numel() < num:
        raise ValueError("mgemm: pointer tables shorter than the matrix count")
    bf16 = x.dtype == torch.bfloat16
    if m > 16 or bf16 or (m >= 5 and A_had is not None):
        sources = num_had_src if had_src is not None else num
        if A_had is None:
            raise ValueError("mgemm: A_had scratch is required above 16 rows")
        _check_cuda("mgemm", A_had)
        if A_had.dtype != torch.float16 or not A_had.is_contiguous() or A_had.numel() < sources * m * k:
            raise ValueError("mgemm: A_had must be a contiguous float16 tensor of (sources, m, k)")
        if not x.is_contiguous():
            raise ValueError("mgemm: x must be contiguous")
    with torch.cuda.device(x.device):
        _lib.call("amp_exl3_mgemm_bf16" if bf16 else "amp_exl3_mgemm", x.data_ptr(), B_ptrs.data_ptr(), C.data_ptr(), suh_ptrs.data_ptr(),
                  A_had.data_ptr() if A_had is not None else None, svh_ptrs.data_ptr(), num, m, k, width,
                  int(K), _cb(mul1, mcg), 1 if C.dtype == torch.float32 else 0,
                  c_ptrs.data_ptr() if c_ptrs is not None else None,
                  n_stride.data_ptr() if n_stride is not None else None,
                  had_src.data_ptr() if had_src is not None else None, num_had_src, _stream(x))
    return C


class _MoeArgs(__import__("ctypes").Structure):
    """ctypes image of amp_moe_coop_args (include/ampstein_b200.h)."""
    import ctypes as _c
    _fields_ = [
        ("x", _c.c_void_p), ("x_stride", _c.c_int), ("sel", _c.c_void_p), ("rw", _c.c_void_p),
        ("bsz", _c.c_int), ("topk", _c.c_int), ("H", _c.c_int), ("Hi", _c.c_int), ("I", _c.c_int),
        ("Ho", _c.c_int), ("H_out", _c.c_int), ("min_expert", _c.c_int), ("max_expert", _c.c_int),
        ("n_local", _c.c_int),
        ("g_trellis", _c.c_void_p), ("g_suh", _c.c_void_p), ("g_svh", _c.c_void_p),
        ("u_trellis", _c.c_void_p), ("u_suh", _c.c_void_p), ("u_svh", _c.c_void_p),
        ("d_trellis", _c.c_void_p), ("d_suh", _c.c_void_p), ("d_svh", _c.c_void_p),
        ("g_bias", _c.c_void_p), ("u_bias", _c.c_void_p), ("d_bias", _c.c_void_p),
        ("Kgu", _c.c_int), ("Kd", _c.c_int), ("cb", _c.c_int), ("act", _c.c_int),
        ("act_limit", _c.c_float), ("gated", _c.c_int),
        ("gu_g", _c.c_void_p), ("gu_u", _c.c_void_p), ("gu_f32", _c.c_int), ("d_out", _c.c_void_p),
        ("ctr", _c.c_void_p), ("ctr_len", _c.c_long), ("slots_max", _c.c_int),
        ("out", _c.c_void_p), ("out_stride", _c.c_int),
        ("sh_out", _c.c_void_p), ("sh_gate_w", _c.c_void_p),
        ("g_bits", _c.c_void_p), ("u_bits", _c.c_void_p), ("d_bits", _c.c_void_p),
        ("kmask_gu", _c.c_int), ("kmask_d", _c.c_int),
    ]


def _moe_bit_masks(who, cfg, n_local, gated):
    """Mixed bit widths: checks the uint8 tables g_bits / u_bits / d_bits of a cfg object and returns
    (kmask_gu, kmask_d), bit K-1 set for every width K that occurs. The tables are static: they are
    read back once and the masks kept in cfg["_kmask"]."""
    for n in (("g_bits", "u_bits", "d_bits") if gated else ("u_bits", "d_bits")):
        t = cfg.get(n)
        if not isinstance(t, torch.Tensor) or t.dtype != torch.uint8 or not t.is_cuda or not t.is_contiguous() \
                or t.numel() < n_local:
            raise TypeError("%s: give all three bit width tables (contiguous uint8 CUDA, one entry per expert) or none" % who)
    if "_kmask" not in cfg:
        if gated and not torch.equal(cfg["g_bits"][:n_local], cfg["u_bits"][:n_local]):
            raise ValueError("%s: gate and up of an expert must share a bit width" % who)
        masks = []
        for n in ("u_bits", "d_bits"):
            ks = torch.unique(cfg[n][:n_local]).tolist()
            if not ks or min(ks) < 1 or max(ks) > 8:
                raise ValueError("%s: bit widths must be 1..8" % who)
            masks.append(sum(1 << (int(k) - 1) for k in ks))
        cfg["_kmask"] = tuple(masks)
    return cfg["_kmask"]


def moe_coop_ctr_len(slots_max, rows_max=None, I=0, Ho=None):
    """int32 entries of the `ctr` scratch (reference: exl3_moe_coop_ctr_len,
    .../quant/exl3_moe_coop.cuh:164-167). Without rows_max / Ho an upper bound is returned (one
    token per slot, outputs up to 16384 wide)."""
    rows_max = slots_max if rows_max is None else rows_max
    Ho = 16384 if Ho is None else Ho
    return int(_lib.lib().amp_exl3_moe_coop_ctr_len(int(slots_max), int(rows_max), int(I), int(Ho)))


def moe_coop(x, sel, rw, cfg, sh_out=None):
    """Fused decode-shaped MoE (reference: torch.moe_coop, src/torch/amp_torch.cpp:7852-7934):
    every (token, expert) slot of x through gate/up, the activation and down, weighted by rw and
    summed per token into cfg["out"] (fp32). Routing stays on the device. cfg holds the static
    parts under the reference's keys: int64 pointer tables g_trellis g_suh g_svh u_* d_*, scratch
    gu_g gu_u d_out ctr out, numbers Hi Kg Ku Kd act act_limit min_expert max_expert, booleans
    mcg mul1 (had_g, had_u, act_out are accepted and unused; optional g_bias u_bias d_bias tables,
    sh_gate_w, gated; optional uint8 tables g_bits u_bits d_bits for experts of different bit
    widths, in which case Kg Ku Kd are not used)."""
    import ctypes
    if not isinstance(cfg, dict):
        raise TypeError("moe_coop: cfg must be an object")
    need = ["g_trellis", "g_suh", "g_svh", "u_trellis", "u_suh", "u_svh", "d_trellis", "d_suh", "d_svh",
            "gu_g", "gu_u", "d_out", "ctr", "out"]
    for n in need:
        if not isinstance(cfg.get(n), torch.Tensor):
            raise TypeError("moe_coop: cfg.%s must be a tensor" % n)
    _check_cuda("moe_coop", x, sel, rw)
    if x.dtype != torch.float16 or sel.dtype != torch.int64 or rw.dtype != torch.float16:
        raise TypeError("moe_coop: x fp16, sel int64, rw fp16 expected")
    if sel.shape != rw.shape or sel.dim() != 2 or sel.shape[0] != x.shape[0] or x.dim() != 2:
        raise ValueError("exl3_moe_coop: sel/rw must be (bsz, topk)")
    for n in ("g_trellis", "g_suh", "g_svh", "u_trellis", "u_suh", "u_svh", "d_trellis", "d_suh", "d_svh"):
        if cfg[n].dtype != torch.int64 or not cfg[n].is_contiguous():
            raise TypeError("exl3_moe_coop: pointer tables must be contiguous int64")
    if cfg["ctr"].dtype != torch.int32:
        raise TypeError("exl3_moe_coop: ctr must be int32")
    if cfg["d_out"].dtype != torch.float32 or cfg["out"].dtype != torch.float32:
        raise TypeError("exl3_moe_coop: d_out and out must be float32")
    gu_dt = cfg["gu_u"].dtype
    if gu_dt not in (torch.float16, torch.float32) or cfg["gu_g"].dtype != gu_dt:
        raise TypeError("exl3_moe_coop: gate/up scratch dtype mismatch")
    mcg, mul1 = bool(cfg.get("mcg", False)), bool(cfg.get("mul1", False))
    Kg, Ku, Kd = cfg.get("Kg", 0), cfg.get("Ku", 0), cfg.get("Kd", 0)
    gated = bool(cfg.get("gated", True))
    if gated and Kg != Ku:
        raise ValueError("exl3_moe_coop: gate and up must share a bit width")
    I, Ho = cfg["gu_u"].shape[-1], cfg["d_out"].shape[-1]
    out = cfg["out"]
    slots_max = min(cfg["gu_g"].numel() // I, cfg["gu_u"].numel() // I, cfg["d_out"].numel() // Ho)
    bsz, topk = sel.shape
    if bsz > out.shape[-2]:
        raise ValueError("exl3_moe_coop: batch exceeds the scratch")
    if cfg["ctr"].numel() < moe_coop_ctr_len(slots_max, bsz, I, Ho):
        raise ValueError("exl3_moe_coop: counter scratch too small")
    if sh_out is not None:
        _check_cuda("moe_coop", sh_out)
        if sh_out.dtype != torch.float32 or sh_out.shape[-1] != x.shape[1] or sh_out.numel() < x.numel():
            raise ValueError("exl3_moe_coop: shared expert output shape")
    a = _MoeArgs()
    p = lambda t: t.data_ptr() if t is not None else None
    a.x, a.x_stride, a.sel, a.rw = p(x), x.stride(0), p(sel), p(rw)
    a.bsz, a.topk, a.H = bsz, topk, x.shape[1]
    a.Hi, a.I, a.Ho, a.H_out = int(cfg.get("Hi", 0)), I, Ho, out.shape[-1]
    a.min_expert, a.max_expert = int(cfg.get("min_expert", -1)), int(cfg.get("max_expert", -1))
    a.n_local = cfg["u_trellis"].shape[0]
    for n in ("g_trellis", "g_suh", "g_svh", "u_trellis", "u_suh", "u_svh", "d_trellis", "d_suh", "d_svh"):
        setattr(a, n, p(cfg[n]))
    for n in ("g_bias", "u_bias", "d_bias"):
        setattr(a, n, p(cfg.get(n)))
    a.Kgu, a.Kd, a.cb = int(Ku), int(Kd), _cb(mul1, mcg)
    a.act, a.act_limit, a.gated = int(cfg.get("act", 0)), float(cfg.get("act_limit", 0.0)), int(gated)
    a.gu_g, a.gu_u, a.gu_f32, a.d_out = p(cfg["gu_g"]), p(cfg["gu_u"]), int(gu_dt == torch.float32), p(cfg["d_out"])
    a.ctr, a.ctr_len, a.slots_max = p(cfg["ctr"]), cfg["ctr"].numel(), slots_max
    a.out, a.out_stride = p(out), out.stride(-2)
    a.sh_out = p(sh_out)
    a.sh_gate_w = p(cfg.get("sh_gate_w"))
    if any(cfg.get(n) is not None for n in ("g_bits", "u_bits", "d_bits")):
        # mixed bit widths: uint8 tables, one entry per expert
        if any(cfg.get(n) is None for n in ("g_bits", "u_bits", "d_bits")):
            raise TypeError("exl3_moe_coop: give all three bit width tables (contiguous uint8 CUDA, one entry per expert) or none")
        _moe_bit_masks("exl3_moe_coop", cfg, a.n_local, gated)
        a.g_bits, a.u_bits, a.d_bits = p(cfg["g_bits"]), p(cfg["u_bits"]), p(cfg["d_bits"])
        a.kmask_gu, a.kmask_d = cfg["_kmask"]
    with torch.cuda.device(x.device):
        _lib.call("amp_exl3_moe_coop", ctypes.byref(a), _stream(x))
    return None


class _MoeSortedArgs(__import__("ctypes").Structure):
    """ctypes image of amp_moe_sorted_args (include/ampstein_b200.h)."""
    import ctypes as _c
    _fields_ = [
        ("y", _c.c_void_p), ("out", _c.c_void_p), ("count", _c.c_void_p), ("tok_sorted", _c.c_void_p),
        ("w_sorted", _c.c_void_p),
        ("T", _c.c_int), ("H", _c.c_int), ("I", _c.c_int), ("E", _c.c_int), ("A", _c.c_long),
        ("g_trellis", _c.c_void_p), ("g_suh", _c.c_void_p), ("g_svh", _c.c_void_p),
        ("u_trellis", _c.c_void_p), ("u_suh", _c.c_void_p), ("u_svh", _c.c_void_p),
        ("d_trellis", _c.c_void_p), ("d_suh", _c.c_void_p), ("d_svh", _c.c_void_p),
        ("Kg", _c.c_int), ("Ku", _c.c_int), ("Kd", _c.c_int), ("cb", _c.c_int), ("act", _c.c_int),
        ("act_limit", _c.c_float), ("gated", _c.c_int), ("count_lo", _c.c_int), ("count_hi", _c.c_int),
        ("workspace", _c.c_void_p), ("workspace_bytes", _c.c_long),
        ("scratch", _c.c_void_p), ("slot_base", _c.c_void_p), ("scratch_rows", _c.c_long),
        ("g_bits", _c.c_void_p), ("u_bits", _c.c_void_p), ("d_bits", _c.c_void_p),
        ("kmask_gu", _c.c_int), ("kmask_d", _c.c_int),
    ]


def moe_sort_routing(sel, rw, n_experts, e0=0, with_inverse=False):
    """Routing of a prefill chunk sorted by expert, as the reference prepares it for torch.moe_fused
    (moe_sorted_begin, src/ucode/ampstein/glm5.uc:1096-1170): sel / rw (T, picks) -> count
    (n_experts + 1) int64, tok_sorted (T * picks) int64, w_sorted (T * picks) fp16. Picks outside
    [e0, e0 + n_experts) fall into the sentinel bin n_experts, which no kernel touches. The sort is
    stable: inside an expert the rows keep their token order. with_inverse: also the tables
    torch.moe_gather takes -- flat_expert (local expert of every pick), inv_order (each pick's
    position in the sorted list) and start (first sorted position of every bin)."""
    T, K = sel.shape
    fe = sel.reshape(-1).to(torch.int64) - int(e0)
    fe = torch.where((fe < 0) | (fe >= n_experts), torch.full_like(fe, n_experts), fe)
    order = torch.sort(fe, stable=True).indices
    tok = (torch.arange(T * K, device=sel.device, dtype=torch.int64) // K)[order].contiguous()
    wts = rw.reshape(-1).to(torch.float16)[order].contiguous()
    count = torch.bincount(fe, minlength=n_experts + 1).to(torch.int64)
    if with_inverse:
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel(), device=order.device, dtype=torch.int64)
        start = (torch.cumsum(count, 0) - count).contiguous()
        return count, tok, wts, fe.contiguous(), inv, start
    return count, tok, wts


def exl3_shard_cols(trellis, svh, ranges):
    """Column shard of an EXL3 linear cut on the device in one launch (reference: sub_columns / cols,
    src/ucode/ampstein/models.uc:440-545): the output columns of `ranges` ([start, length] pairs,
    multiples of 128) concatenated. Returns (trellis (k/16, total/16, 16K), svh (total))."""
    import ctypes
    _check_cuda("exl3_shard_cols", trellis, svh)
    k, n, K = _trellis_dims("exl3_shard_cols", trellis, half_ok=True)
    K = _kcode("exl3_shard_cols", K, True)
    if svh.dtype != torch.float16 or svh.numel() != n:
        raise ValueError("exl3_shard_cols: svh must be fp16 with one value per output column")
    ranges = [(int(a), int(b)) for a, b in ranges]
    for a, ln in ranges:
        if a % 128 or ln % 128 or a < 0 or ln <= 0 or a + ln > n:
            raise ValueError("models.sub_columns: range [%d, %d] not 128-aligned/in bounds" % (a, ln))
    if not 1 <= len(ranges) <= 16:
        raise ValueError("exl3_shard_cols: 1..16 ranges")
    total = sum(ln for _, ln in ranges)
    out = torch.empty((k // 16, total // 16, trellis.shape[2]), dtype=trellis.dtype, device=trellis.device)
    out_svh = torch.empty(total, dtype=torch.float16, device=trellis.device)
    flat = (ctypes.c_int * (2 * len(ranges)))(*[v for r in ranges for v in r])
    with torch.cuda.device(trellis.device):
        _lib.call("amp_exl3_shard_cols", trellis.data_ptr(), svh.data_ptr(), out.data_ptr(), out_svh.data_ptr(), k, n, K,
                  ctypes.cast(flat, ctypes.c_void_p), len(ranges), _stream(trellis))
    return out, out_svh


def exl3_shard_rows(trellis, suh, k0, klen):
    """Row shard (reference: rows, src/ucode/ampstein/models.uc:547-562): input rows [k0, k0 + klen),
    multiples of 128, of the trellis and of suh, as copies of their own."""
    _check_cuda("exl3_shard_rows", trellis, suh)
    k, n, K = _trellis_dims("exl3_shard_rows", trellis, half_ok=True)
    K = _kcode("exl3_shard_rows", K, True)
    if suh.dtype != torch.float16 or suh.numel() != k:
        raise ValueError("exl3_shard_rows: suh must be fp16 with one value per input row")
    k0, klen = int(k0), int(klen)
    if k0 % 128 or klen % 128 or k0 < 0 or klen <= 0 or k0 + klen > k:
        raise ValueError("models.rows: range [%d, %d] not 128-aligned/in bounds" % (k0, klen))
    out = torch.empty((klen // 16, n // 16, trellis.shape[2]), dtype=trellis.dtype, device=trellis.device)
    out_suh = torch.empty(klen, dtype=torch.float16, device=trellis.device)
    with torch.cuda.device(trellis.device):
        _lib.call("amp_exl3_shard_rows", trellis.data_ptr(), suh.data_ptr(), out.data_ptr(), out_suh.data_ptr(), k, n, K,
                  k0, klen, _stream(trellis))
    return out, out_suh


def moe_prep(idx, w, n_experts, e0=0):
    """Token-sorted MoE dispatch in one kernel (reference: torch.moe_prep, src/torch/amp_torch.cpp:8168-8215):
    idx (T, K) int64 global expert ids, w (T, K) fp32 -> [fe (A) int64, order (A) int64, tok (A) int64,
    wts (A) fp16, count (E + 1) int64, start (E + 1) int64, inv (A) int64, kind (E) int64] for the
    experts [e0, e0 + E): a stable sort of the assignments by local expert, foreign picks last."""
    _check_cuda("moe_prep", idx, w)
    E = int(n_experts)
    if idx.dim() != 2 or idx.dtype != torch.int64 or w.dtype != torch.float32 or w.shape != idx.shape \
            or w.device != idx.device or E < 1 or E > 4096:
        raise ValueError("moe_prep: idx (T, K) int64 and w (T, K) fp32, contiguous on one CUDA device, 1 <= E <= 4096")
    A, K = idx.numel(), idx.shape[1]
    lo = dict(dtype=torch.int64, device=idx.device)
    fe, order, tok, inv = (torch.empty(A, **lo) for _ in range(4))
    wts = torch.empty(A, dtype=torch.float16, device=idx.device)
    count, start, kind = torch.empty(E + 1, **lo), torch.empty(E + 1, **lo), torch.empty(E, **lo)
    if A == 0:
        return [fe, order, tok, wts, count.zero_(), start.zero_(), inv, kind.zero_()]
    with torch.cuda.device(idx.device):
        _lib.call("amp_moe_prep", idx.data_ptr(), w.data_ptr(), A, K, E, int(e0), fe.data_ptr(), order.data_ptr(),
                  tok.data_ptr(), wts.data_ptr(), count.data_ptr(), start.data_ptr(), inv.data_ptr(), kind.data_ptr(), _stream(idx))
    return [fe, order, tok, wts, count, start, inv, kind]


def moe_fused(y, out, count, tok_sorted, w_sorted, cfg, num_active=-1, lo=1, hi=0, m_tile=16,
              scratch=None, slot_base=None):
    """Token-sorted MoE for prefill chunks (reference: torch.moe_fused, src/torch/amp_torch.cpp:9257-9345,
    kernel exl3_moe, .../quant/exl3_moe.cu:139-531): experts with lo <= rows <= hi (hi <= 0: no upper
    bound) run gate / up / activation / down on their rows of y, and weight * result is summed per
    token in a fixed order and added to out (fp32, zero-initialised by the caller, same shape as y).
    cfg: the pointer tables g_/u_/d_ {trellis,suh,svh} and Kg Ku Kd act act_limit mcg mul1 [gated]
    [g_bits u_bits d_bits] of moe_coop; the reference's temps ts_g ts_u ti_g ti_u are not needed (one
    workspace, kept in cfg).
    num_active and m_tile are accepted and unused (one call covers every row count; the reference's
    three tiered calls still work). With scratch (fp32 [slots, hidden]) and slot_base (int64 per
    expert) the sum is deferred as in the reference: out is left alone, weight * result of every
    assignment goes to its slot, and moe_gather adds the slots up in pick order. The workspace lives in
    cfg: calls that share a cfg object must be ordered on one stream (use one cfg per stream otherwise)."""
    import ctypes
    if not isinstance(cfg, dict):
        raise TypeError("moe_fused: cfg must be an object")
    names = ["u_trellis", "u_suh", "u_svh", "d_trellis", "d_suh", "d_svh"]
    gated = bool(cfg.get("gated", True))
    if gated:
        names += ["g_trellis", "g_suh", "g_svh"]
    for n in names:
        t = cfg.get(n)
        if not isinstance(t, torch.Tensor):
            raise TypeError("moe_fused: cfg.%s must be a tensor" % n)
        if t.dtype != torch.int64 or not t.is_contiguous():
            raise TypeError("moe_fused: pointer tables must be contiguous int64")
    _check_cuda("moe_fused", y, out, count, tok_sorted, w_sorted)
    if y.dtype != torch.float16 or out.dtype != torch.float32 or count.dtype != torch.int64 \
            or tok_sorted.dtype != torch.int64 or w_sorted.dtype != torch.float16:
        raise TypeError("moe_fused: y fp16, out fp32, count int64, tok_sorted int64, w_sorted fp16 expected")
    if y.dim() != 2 or out.shape != y.shape or not y.is_contiguous() or not out.is_contiguous():
        raise ValueError("moe_fused: y and out must be contiguous (T, hidden) of one shape")
    E = cfg["u_trellis"].shape[0]
    if count.numel() < E + 1 or tok_sorted.numel() != w_sorted.numel():
        raise ValueError("moe_fused: count must hold experts + 1 entries, tok_sorted and w_sorted one per pick")
    I = int(cfg.get("I", 0)) or (cfg["gu_u"].shape[-1] if isinstance(cfg.get("gu_u"), torch.Tensor) else 0)
    if I <= 0:
        raise ValueError("moe_fused: cfg.I (intermediate width) is required")
    T, H, A = y.shape[0], y.shape[1], tok_sorted.numel()
    if T == 0 or A == 0:
        return None
    need = int(_lib.lib().amp_exl3_moe_sorted_workspace(T, A, E, H, I))
    if need <= 0:
        raise ValueError("moe_fused: unsupported sizes")
    ws = cfg.get("_sorted_ws")
    if ws is None or ws.numel() < need or ws.device != y.device:
        ws = torch.empty(need, dtype=torch.uint8, device=y.device)
        cfg["_sorted_ws"] = ws
    a = _MoeSortedArgs()
    p = lambda t: t.data_ptr() if t is not None else None
    a.y, a.out, a.count, a.tok_sorted, a.w_sorted = p(y), p(out), p(count), p(tok_sorted), p(w_sorted)
    a.T, a.H, a.I, a.E, a.A = T, H, I, E, A
    for n in ("g_trellis", "g_suh", "g_svh", "u_trellis", "u_suh", "u_svh", "d_trellis", "d_suh", "d_svh"):
        setattr(a, n, p(cfg.get(n)))
    a.Kg, a.Ku, a.Kd = int(cfg.get("Kg", 0)), int(cfg.get("Ku", 0)), int(cfg.get("Kd", 0))
    a.cb = _cb(bool(cfg.get("mul1", False)), bool(cfg.get("mcg", False)))
    a.act, a.act_limit, a.gated = int(cfg.get("act", 0)), float(cfg.get("act_limit", 0.0)), int(gated)
    a.count_lo, a.count_hi = int(lo), int(hi)
    a.workspace, a.workspace_bytes = p(ws), ws.numel()
    if any(cfg.get(n) is not None for n in ("g_bits", "u_bits", "d_bits")):
        a.kmask_gu, a.kmask_d = _moe_bit_masks("moe_fused", cfg, E, gated)
        a.g_bits, a.u_bits, a.d_bits = p(cfg.get("g_bits") if gated else None), p(cfg["u_bits"]), p(cfg["d_bits"])
    if (scratch is None) != (slot_base is None):
        raise ValueError("moe_fused: scratch needs slot_base")
    if scratch is not None:
        _check_cuda("moe_fused", scratch, slot_base)
        if scratch.dtype != torch.float32 or scratch.dim() != 2 or scratch.shape[1] != H or slot_base.dtype != torch.int64 \
                or slot_base.numel() < E:
            raise TypeError("moe_fused: scratch must be fp32 [slots, hidden], slot_base int64 with one entry per expert")
        a.scratch, a.slot_base, a.scratch_rows = p(scratch), p(slot_base), scratch.shape[0]
    with torch.cuda.device(y.device):
        _lib.call("amp_exl3_moe_sorted", ctypes.byref(a), _stream(y))
    return None


def moe_fused_status(cfg, device=None):
    """Status word of the last moe_fused call that used cfg's workspace (0 = clean; see
    amp_exl3_moe_sorted_status). Synchronises."""
    import ctypes
    ws = cfg.get("_sorted_ws")
    if ws is None:
        return 0
    out = ctypes.c_int(0)
    with torch.cuda.device(ws.device):
        _lib.call("amp_exl3_moe_sorted_status", ws.data_ptr(), ctypes.byref(out), _stream(ws))
    return out.value


def moe_gather(out, scratch, flat_expert, inv_order, expert_start, slot_base, slot_kind, w_sorted):
    """Reference: torch.moe_gather (src/torch/amp_torch.cpp:9347-9372, exl3_moe_gather): the fixed-order
    reduction of moe_fused's per-assignment slots. Every token's picks are summed in pick order and
    added to its row of out (fp32). flat_expert: (T * picks) local expert id per assignment;
    inv_order: position of each assignment in the expert-sorted list; expert_start / slot_base /
    slot_kind: per-expert tables (kind 0 = no slots, 1 = slots hold weighted outputs, 2 = unweighted:
    multiplied by w_sorted here)."""
    _check_cuda("moe_gather", out, scratch, flat_expert, inv_order, expert_start, slot_base, slot_kind, w_sorted)
    if out.dtype != torch.float32 or scratch.dtype != torch.float32 or w_sorted.dtype != torch.float16:
        raise TypeError("moe_gather: out and scratch fp32, w_sorted fp16 expected")
    for t in (flat_expert, inv_order, expert_start, slot_base, slot_kind):
        if t.dtype != torch.int64:
            raise TypeError("moe_gather: index tensors must be int64")
    if out.dim() != 2 or scratch.dim() != 2 or scratch.shape[1] != out.shape[1]:
        raise ValueError("moe_gather: scratch must be [slots, hidden]")
    T, H = out.shape
    if T == 0:
        return None
    if flat_expert.numel() % T or inv_order.numel() != flat_expert.numel():
        raise ValueError("moe_gather: assignments / tokens")
    E = slot_kind.numel()
    if slot_base.numel() < E or expert_start.numel() < E:
        raise ValueError("moe_gather: table sizes")
    with torch.cuda.device(out.device):
        _lib.call("amp_exl3_moe_gather", out.data_ptr(), scratch.data_ptr(), flat_expert.data_ptr(), inv_order.data_ptr(),
                  expert_start.data_ptr(), slot_base.data_ptr(), slot_kind.data_ptr(), w_sorted.data_ptr(),
                  T, H, flat_expert.numel() // T, E, scratch.shape[0], _stream(out))
    return None
