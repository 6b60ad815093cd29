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
        if trellis.dim() != 3 or trellis.shape[2] % 16:
            raise ValueError("LinearEXL3: half-integer bitrates are not supported")
        self.trellis, self.suh, self.svh, self.bias = trellis, suh, svh, bias
        self.K = trellis.shape[2] // 16
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

    def weight_bytes(self):
        return self.trellis.numel() * 2


class DecodeGraph:
    """Captures `step_fn()` (a sequence of operator calls on fixed buffers) in one CUDA graph
    after warm-up runs, then replays it: one host->device crossing per step, as the reference's
    graphdec does. Everything the step touches must exist before capture."""

    def __init__(self, step_fn, warmup=3):
        self.stream = torch.cuda.Stream()
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
