"""Host-side mirror of the reference's linear classes and CUDA-graph decode step, restricted to
the EXL3 linears (reference: src/ucode/ampstein/models.uc:49-107 LinearEXL3,
src/ucode/ampstein/graphdec.uc:151-282 step capture and replay).

LinearEXL3 derives everything from the trellis tensor:
    K = trellis.shape[-1] / 16, in_features = trellis.shape[0] * 16, out_features = shape[1] * 16
forward(x) picks the many-rows operator above RECON_ROWS rows, the decode operator otherwise,
exactly as the reference does.
"""
import torch

from . import exl3

RECON_ROWS = 144          # models.uc:36
RECON_MAX_N = 32768       # models.uc:37


class LinearEXL3:
    def __init__(self, trellis, suh, svh, bias=None, mul1=False, mcg=False):
        if mul1 and mcg:
            raise ValueError("LinearEXL3: both mul1 and mcg set")
        if trellis.dim() != 3 or trellis.shape[2] % 8:
            raise ValueError("LinearEXL3: trellis must be (k/16, n/16, 16 K)")
        if trellis.shape[2] % 16 and not (mul1 and 1 <= trellis.shape[2] // 16 <= 3):
            # (reference: models.uc:9-15, 68-71: K = shape[2] / 16 as a float; bits_k.cuh:14-20)
            raise ValueError("LinearEXL3: half-integer bitrates are 1.5 / 2.5 / 3.5 with the mul1 codebook")
        self.trellis, self.suh, self.svh, self.bias = trellis, suh, svh, bias
        self.K = trellis.shape[2] // 16 if trellis.shape[2] % 16 == 0 else trellis.shape[2] / 16.0     # 1.5 / 2.5 / 3.5: 16 K + 8 words
        self.mul1, self.mcg = mul1, mcg
        self.in_features = trellis.shape[0] * 16
        self.out_features = trellis.shape[1] * 16

    def forward(self, x, out=None):
        m = x.shape[0]
        if out is None and m > RECON_ROWS and self.out_features <= RECON_MAX_N:
            out = exl3.exl3_gemm_recon(x.contiguous(), self.trellis, self.suh, self.svh, self.K,
                                       self.mul1, self.mcg)
        else:
            if out is None:
                out = torch.empty((m, self.out_features), dtype=torch.float16, device=x.device)
            exl3.exl3_gemm(x, self.trellis, out, self.suh, self.svh, self.mul1, self.mcg)
        if self.bias is not None:
            out = out.add(self.bias)
        return out

    def forward_silu_mul(self, gate, up, out=None):
        """out = this linear of silu(gate) * up in one launch (the down projection behind a gate|up
        bundle, up to 16 rows); larger batches take the two-step path of the caller."""
        m = gate.shape[0]
        if out is None:
            out = torch.empty((m, self.out_features), dtype=torch.float16, device=gate.device)
        exl3.exl3_gemm_silu_mul(gate, up, self.trellis, out, self.suh, self.svh, self.mul1, self.mcg)
        if self.bias is not None:
            out = out.add(self.bias)
        return out

    def forward_add_res(self, x, h, y, ssq):
        """y = fp16(h + this linear of x), ssq = block sums of squares of y: the linear and the residual
        add of the norm that follows, in one launch (up to 16 rows)."""
        return exl3.exl3_gemm_add_res(x, self.trellis, self.suh, self.svh, h, y, ssq, self.mul1, self.mcg)

    def weight_bytes(self):
        return self.trellis.numel() * 2


def linear(ws, key, dev=0):
    """EXL3 linear `key` of a weight set on device `dev` (reference: models.uc LinearEXL3(ws, key, dev),
    :49-110): <key>.trellis / .suh / .svh (+ optional .bias), the codebook from the marker tensors
    <key>.mul1 / <key>.mcg (mutually exclusive), the bitrate from the trellis shape."""
    mul1, mcg = ws.has(key + ".mul1"), ws.has(key + ".mcg")
    if mul1 and mcg:
        raise ValueError("LinearEXL3: %s: both .mul1 and .mcg marker tensors present" % key)
    bias = ws.gpu16(key + ".bias", dev) if ws.has(key + ".bias") else None
    return LinearEXL3(ws.gpu(key + ".trellis", dev), ws.gpu(key + ".suh", dev), ws.gpu(key + ".svh", dev), bias=bias,
                      mul1=mul1, mcg=mcg)


def split_n(total, unit, weights):
    """Cut `total` (a multiple of `unit`) into per-rank [start, length] ranges proportional to
    `weights` by largest remainder (reference: src/ucode/ampstein/qwen35_tp.uc:40-72)."""
    n, tot = total // unit, float(sum(weights))
    cnt, rem, used = [], [], 0
    for g, w in enumerate(weights):
        exact = n * w / tot
        c = int(exact)
        cnt.append(c)
        rem.append((exact - c, g))
        used += c
    rem.sort(key=lambda a: (-a[0], a[1]))
    k = 0
    while used < n:
        cnt[rem[k % len(weights)][1]] += 1
        k += 1
        used += 1
    out, at = [], 0
    for c in cnt:
        out.append((at * unit, c * unit))
        at += c
    return out


def cols(lin, ranges):
    """Column-parallel shard: output columns ([start, length] pairs, 256-aligned) concatenated;
    suh whole, svh sliced (reference: models.uc cols(), :537-545)."""
    for n0, w in ranges:
        if n0 % 128 or w % 128 or n0 < 0 or w <= 0 or n0 + w > lin.out_features:
            raise ValueError("models.sub_columns: range [%d, %d] not 128-aligned/in bounds" % (n0, w))
    if lin.trellis.is_cuda:
        tr, svh = exl3.exl3_shard_cols(lin.trellis, lin.svh, ranges)        # one launch on the device
    else:
        # weights still in host memory (before the upload): plain slices of the host tensors
        tr = torch.cat([lin.trellis[:, n0 // 16:(n0 + w) // 16] for n0, w in ranges], dim=1).contiguous()
        svh = torch.cat([lin.svh[n0:n0 + w] for n0, w in ranges]).contiguous()
    return LinearEXL3(tr, lin.suh, svh, mul1=lin.mul1, mcg=lin.mcg)


def rows(lin, k0, klen):
    """Row-parallel shard: input rows [k0, k0 + klen), 128-aligned, with the matching suh slice
    and the whole svh; the shards' outputs SUM to the full product (reference: models.uc rows(),
    :547-562)."""
    if k0 % 128 or klen % 128 or k0 < 0 or klen <= 0 or k0 + klen > lin.in_features:
        raise ValueError("models.rows: range [%d, %d] not 128-aligned/in bounds" % (k0, klen))
    if lin.trellis.is_cuda:
        tr, suh = exl3.exl3_shard_rows(lin.trellis, lin.suh, k0, klen)
    else:
        tr, suh = lin.trellis[k0 // 16:(k0 + klen) // 16].clone(), lin.suh[k0:k0 + klen].clone()
    return LinearEXL3(tr, suh, lin.svh, mul1=lin.mul1, mcg=lin.mcg)


def _bundle_check(linears):
    a = linears[0]
    for i, w in enumerate(linears[1:], 1):
        if (w.K, w.mul1, w.mcg, w.in_features) != (a.K, a.mul1, a.mcg, a.in_features):
            raise ValueError("models.bundle: fused linears must share K, in_features and codebook "
                             "(matrix %d differs)" % i)


class Multi:
    """Equal-shape bundle (reference: models.uc multi(), :338-361): run(x) writes all outputs
    stacked into `out` (num, m, n) with ONE launch. x is (1, m, k)."""

    def __init__(self, linears, out):
        _bundle_check(linears)
        dev = out.device
        self.linears, self.out = linears, out
        self.B = exl3.ptr_array([w.trellis.data_ptr() for w in linears], dev)
        self.suh = exl3.ptr_array([w.suh.data_ptr() for w in linears], dev)
        self.svh = exl3.ptr_array([w.svh.data_ptr() for w in linears], dev)

    def run(self, x, a_had=None):
        """a_had: (num, m, k) fp16 scratch, used from five rows up (allocated here if missing)"""
        a = self.linears[0]
        m = x.shape[1]
        if a_had is None and (m >= 5 or x.dtype == torch.bfloat16):
            a_had = torch.empty((len(self.linears), m, a.in_features), dtype=torch.float16, device=x.device)
        return exl3.mgemm(x, self.B, self.out, self.suh, a_had, self.svh, a.K, a.mcg, a.mul1)

    def run_norm(self, x, res, norm_w, eps, y):
        """The bundle applied to RMSNorm(x + res) * norm_w, y = fp16(x + res): one launch (up to 16 rows)."""
        return _run_norm(self, self.out, x, res, norm_w, eps, y, None)

    def run_normed(self, y, ssq, norm_w, eps):
        """The bundle applied to the norm of a residual stream whose block sums of squares the producing
        linear left in ssq (LinearEXL3.forward_add_res)."""
        a = self.linears[0]
        return exl3.mgemm_normed(y, ssq, norm_w, eps, self.B, self.out, self.suh, self.svh, a.K, a.mcg, a.mul1)


def _run_norm(bundle, carrier, x, res, norm_w, eps, y, opts):
    a = bundle.linears[0]
    return exl3.mgemm_rms_norm_res(x, res, norm_w, eps, y, bundle.B, carrier, bundle.suh, bundle.svh, a.K, a.mcg, a.mul1, opts)


class Sliced:
    """Bundle for unequal widths such as Q/K/V (reference: models.uc sliced(), :367-432): every
    matrix is cut into column slices of the widths' gcd (a multiple of 128); outputs are written
    in place into `outs`, one (1, m, out_features) buffer per linear."""

    def __init__(self, linears, outs):
        import math
        _bundle_check(linears)
        dev = outs[0].device
        width = 0
        for w in linears:
            width = math.gcd(width, w.out_features)
        if width % 128 or width < 128:
            raise ValueError("models.sliced: unsuitable slice width %d" % width)
        t, svh, cp, stride, src = [], [], [], [], []
        for i, w in enumerate(linears):
            tw = w.trellis.shape[2]
            for n0 in range(0, w.out_features, width):
                t.append(w.trellis.data_ptr() + (n0 // 16) * tw * 2)
                svh.append(w.svh.data_ptr() + n0 * 2)
                cp.append(outs[i].data_ptr() + n0 * 2)
                stride.append(w.out_features)
                src.append(i)
        self.linears, self.outs, self.width, self.slices = linears, outs, width, len(t)
        m = outs[0].shape[1]
        self.B = exl3.ptr_array(t, dev)
        self.svh = exl3.ptr_array(svh, dev)
        self.suh = exl3.ptr_array([w.suh.data_ptr() for w in linears], dev)
        i32 = dict(dtype=torch.int32, device=dev)
        self.opts = {
            "size_n_list": torch.tensor([width] * len(t), **i32),
            "c_ptrs": exl3.ptr_array(cp, dev),
            "n_stride_list": torch.tensor(stride, **i32),
            "had_src_list": torch.tensor(src, **i32),
            "num_had_src": len(linears),
        }
        # descriptor only: (num_slices, m, width); the data goes through c_ptrs
        self.carrier = torch.empty((len(t), m, width), dtype=torch.float16, device=dev)

    def run(self, x, a_had=None):
        """a_had: (linears, m, k) fp16 scratch, used from five rows up (allocated here if missing)"""
        a = self.linears[0]
        m = x.shape[1]
        if a_had is None and (m >= 5 or x.dtype == torch.bfloat16):
            a_had = torch.empty((len(self.linears), m, a.in_features), dtype=torch.float16, device=x.device)
        exl3.mgemm(x, self.B, self.carrier, self.suh, a_had, self.svh, a.K, a.mcg, a.mul1, self.opts)
        return self.outs

    def run_norm(self, x, res, norm_w, eps, y):
        """The bundle applied to RMSNorm(x + res) * norm_w, y = fp16(x + res): one launch (up to 16 rows)."""
        _run_norm(self, self.carrier, x, res, norm_w, eps, y, self.opts)
        return self.outs

    def run_normed(self, y, ssq, norm_w, eps):
        """The bundle applied to the norm of a residual stream whose block sums of squares the producing
        linear left in ssq (LinearEXL3.forward_add_res)."""
        a = self.linears[0]
        exl3.mgemm_normed(y, ssq, norm_w, eps, self.B, self.carrier, self.suh, self.svh, a.K, a.mcg, a.mul1, self.opts)
        return self.outs


class DecodeGraph:
    """Captures `step_fn()` (a sequence of operator calls on fixed buffers) in one CUDA graph
    after warm-up runs, then replays it: one host->device crossing per step, as the reference's
    graphdec does. Everything the step touches must exist before capture."""

    def __init__(self, step_fn, warmup=3, stream=None):
        self.stream = stream if stream is not None else torch.cuda.Stream()
        with torch.cuda.stream(self.stream):
            for _ in range(warmup):
                step_fn()
            self.stream.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self.stream):
                step_fn()
        torch.cuda.synchronize()

    def replay(self):
        self.graph.replay()
