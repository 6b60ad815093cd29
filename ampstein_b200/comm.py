"""Host side of the tensor-parallel all-reduce communicator (reference: torch.p2p_comm /
comm.allreduce / comm.info, src/torch/amp_torch.cpp:7606-7781).

Two ways to build one:

  p2p_comm(devices, cap, mode)          one process drives every GPU, rank = position in
                                        `devices` (the reference's model); allreduce(x, rank)
  P2PComm.from_process_group(cap, ...)  one process per GPU over torch.distributed: buffers are
                                        exchanged as CUDA IPC handles through the group (NCCL or
                                        gloo carries only the 64-byte handles, never the data);
                                        allreduce(x)

comm.allreduce returns a new tensor holding the sum, bit-identical on all ranks; every rank must
issue the same sequence of calls. The transport is this repository's NVLink kernel
(amp_comm_allreduce_fp16), not NCCL.
"""
import ctypes

import torch

from . import _lib

MAXN = 8
MODES = {"oneshot": 0, "twophase": 1}


class CudaBackend:
    """Device memory + launch through the C ABI. Tests substitute a fake with the same methods."""

    def buffer_bytes(self, N, cap):
        return int(_lib.lib().amp_comm_buffer_bytes(N, cap))

    def ctl_bytes(self):
        return int(_lib.lib().amp_comm_ctl_bytes())

    def blocks(self, N, n):
        return int(_lib.lib().amp_comm_blocks(N, n))

    def alloc(self, nbytes):
        """-> (pointer, 64-byte IPC handle)"""
        p = ctypes.c_void_p()
        h = ctypes.create_string_buffer(64)
        _lib.call("amp_comm_ipc_alloc", nbytes, ctypes.byref(p), h)
        return p.value, h.raw

    def open(self, handle):
        p = ctypes.c_void_p()
        _lib.call("amp_comm_ipc_open", handle, ctypes.byref(p))
        return p.value

    def close(self, ptr):
        _lib.call("amp_comm_ipc_close", ptr)

    def free(self, ptr):
        _lib.call("amp_comm_free", ptr)

    def enable_peer(self, peer):
        _lib.call("amp_comm_enable_peer", peer)

    def launch(self, x_ptr, out_ptr, bufs, ctls, rank, N, n, cap, mode, blocks, stream):
        rc = _lib.lib().amp_comm_allreduce_fp16(x_ptr, out_ptr, bufs, ctls, rank, N, n, cap, mode, blocks, stream)
        if rc != 0:
            raise _lib.AmpError("amp_comm_allreduce_fp16", rc, _lib.last_error())

    def status(self, ctl_ptr):
        v = ctypes.c_int(0)
        _lib.call("amp_comm_status", ctl_ptr, ctypes.byref(v))
        return v.value


def _resolve_mode(mode, N):
    if mode is None or mode == "auto":
        # NVSwitch: every peer is one hop at full bandwidth, so the one-shot form wins for decode
        # payloads at every N (the reference switches to two-phase above 3 ranks on PCIe)
        return 0
    if mode not in MODES:
        raise ValueError("mode must be auto, oneshot or twophase")
    return MODES[mode]


class P2PComm:
    def __init__(self, N, cap, mode, backend):
        if not (2 <= N <= MAXN):
            raise ValueError("2..8 devices supported")
        if not isinstance(cap, int) or cap <= 0 or cap % 8:
            raise TypeError("expected (devices array, cap (multiple of 8), mode?)")
        self.N, self.cap, self.mode = N, cap, _resolve_mode(mode, N)
        self.backend = backend or CudaBackend()
        self.devices = None            # single-process form: device index per rank
        self.rank = None               # process-group form: this process's rank
        self._bufs = {}                # rank (or 0 in process-group form) -> ctypes arrays
        self._local = {}               # rank -> (buf ptr, ctl ptr) owned here
        self._opened = []

    # ---- construction ------------------------------------------------------------------

    @classmethod
    def single_process(cls, devices, cap, mode=None, backend=None):
        devices = list(devices)
        for d in devices:
            if not isinstance(d, int) or d < 0 or (backend is None and d >= torch.cuda.device_count()):
                raise ValueError("bad device index")
        self = cls(len(devices), cap, mode, backend)
        self.devices = devices
        be = self.backend
        ptrs = []
        for a in devices:
            with _device(a, backend):
                for b in devices:
                    if a != b:
                        be.enable_peer(b)
                buf, _ = be.alloc(be.buffer_bytes(self.N, cap))
                ctl, _ = be.alloc(be.ctl_bytes())
                ptrs.append((buf, ctl))
        for r in range(self.N):
            self._local[r] = ptrs[r]
            self._bufs[r] = self._arrays(ptrs)
        return self

    @classmethod
    def from_process_group(cls, cap, mode=None, group=None, backend=None):
        import torch.distributed as dist
        N, rank = dist.get_world_size(group), dist.get_rank(group)
        self = cls(N, cap, mode, backend)
        self.rank = rank
        be = self.backend
        buf, hbuf = be.alloc(be.buffer_bytes(N, cap))
        ctl, hctl = be.alloc(be.ctl_bytes())
        self._local[rank] = (buf, ctl)
        gathered = [None] * N
        dist.all_gather_object(gathered, (rank, hbuf, hctl), group=group)
        ptrs = [None] * N
        for r, hb, hc in gathered:
            if r == rank:
                ptrs[r] = (buf, ctl)
            else:
                pb, pc = be.open(hb), be.open(hc)
                self._opened += [pb, pc]
                ptrs[r] = (pb, pc)
        self._bufs[rank] = self._arrays(ptrs)
        # nobody may push into a peer's buffer before every rank has mapped everything
        dist.barrier(group=group)
        return self

    @staticmethod
    def _arrays(ptrs):
        n = len(ptrs)
        bufs = (ctypes.c_void_p * n)(*[p[0] for p in ptrs])
        ctls = (ctypes.c_void_p * n)(*[p[1] for p in ptrs])
        return bufs, ctls

    # ---- operations ------------------------------------------------------------------------

    def allreduce(self, x, rank=None, out=None):
        """Sum of every rank's x, returned as a new tensor (or written into `out`, a contiguous
        fp16 tensor of x's size on the same device, for callers that keep fixed buffers)."""
        if rank is None:
            rank = self.rank
        if rank is None or not (0 <= rank < self.N):
            raise ValueError("expected (x, rank)")
        if self.rank is not None and rank != self.rank:
            raise ValueError("comm.allreduce: this process is rank %d" % self.rank)
        ok = (isinstance(x, torch.Tensor) and x.is_cuda and x.dtype == torch.float16 and x.is_contiguous()
              and x.numel() % 8 == 0 and 0 < x.numel() <= self.cap)
        if ok and self.devices is not None:
            ok = x.get_device() == self.devices[rank]
        if not ok:
            raise ValueError("comm.allreduce: x must be contiguous fp16 on the rank's device, "
                             "n % 8 == 0, n <= cap")
        n = x.numel()
        if out is None:
            out = torch.empty_like(x)
        elif not (isinstance(out, torch.Tensor) and out.is_cuda and out.dtype == torch.float16 and out.is_contiguous()
                  and out.numel() == n and out.device == x.device):
            raise ValueError("comm.allreduce: out must be a contiguous fp16 tensor of x's size on x's device")
        bufs, ctls = self._bufs[rank]
        with torch.cuda.device(x.device):
            self.backend.launch(x.data_ptr(), out.data_ptr(), bufs, ctls, rank, self.N, n, self.cap,
                                self.mode, self.backend.blocks(self.N, n),
                                torch.cuda.current_stream(x.device).cuda_stream)
        return out

    def linear_allreduce(self, lin, x, out, rank=None):
        """Row-parallel EXL3 linear with the all-reduce fused into its kernel: out (m, n) fp16 =
        sum over ranks of lin(x). `lin` is a models.LinearEXL3 holding this rank's row shard; x
        (m, k_local) fp16, m <= 16, m * n <= cap. Equivalent to lin.forward followed by
        allreduce (same bits), without the extra launch."""
        from . import _lib
        rank = self.rank if rank is None else rank
        if rank is None or not (0 <= rank < self.N):
            raise ValueError("expected (lin, x, out, rank)")
        m = x.shape[0]
        n = lin.out_features
        ok = (x.is_cuda and x.dtype == torch.float16 and x.is_contiguous() and x.dim() == 2
              and x.shape[1] == lin.in_features and 1 <= m <= 16 and m * n <= self.cap
              and out.is_cuda and out.dtype == torch.float16 and out.is_contiguous() and out.numel() == m * n
              and out.device == x.device and lin.bias is None)
        if not ok:
            raise ValueError("comm.linear_allreduce: x (m <= 16, k) and out (m, n) must be contiguous fp16 on the "
                             "rank's device, m * n <= cap, no bias")
        bufs, ctls = self._bufs[rank]
        cb = 2 if lin.mul1 else (1 if lin.mcg else 0)
        with torch.cuda.device(x.device):
            # from five rows on, a scratch lets the input be rotated once instead of by every CTA
            rot = torch.empty_like(x) if m >= 5 else None
            _lib.call("amp_exl3_gemv_allreduce_rot", x.data_ptr(), lin.trellis.data_ptr(), out.data_ptr(),
                      lin.suh.data_ptr(), lin.svh.data_ptr(), m, lin.in_features, n, lin.K, cb,
                      bufs, ctls, rank, self.N, self.cap, rot.data_ptr() if rot is not None else None,
                      torch.cuda.current_stream(x.device).cuda_stream)
        return out

    # ---- split exchange: push in the producer, gather in the consumer's prologue ----

    def linear_push(self, lin, x, rank=None):
        """Row-parallel EXL3 linear whose result is not written anywhere: every finished column
        block is pushed, as this rank's fp16 partial, into every rank's buffer. The next launch on
        this communicator must be a gathered one (gathered_linear / gathered_bundle) on every
        rank; it consumes the sum."""
        from . import _lib
        rank = self.rank if rank is None else rank
        if rank is None or not (0 <= rank < self.N):
            raise ValueError("expected (lin, x, rank)")
        m, n = x.shape[0], lin.out_features
        ok = (x.is_cuda and x.dtype == torch.float16 and x.is_contiguous() and x.dim() == 2
              and x.shape[1] == lin.in_features and 1 <= m <= 16 and m * n <= self.cap and lin.bias is None)
        if not ok:
            raise ValueError("comm.linear_push: x (m <= 16, k) must be contiguous fp16 on the rank's device, "
                             "m * n <= cap, no bias")
        bufs, ctls = self._bufs[rank]
        cb = 2 if lin.mul1 else (1 if lin.mcg else 0)
        with torch.cuda.device(x.device):
            _lib.call("amp_exl3_gemv_push", x.data_ptr(), lin.trellis.data_ptr(), lin.suh.data_ptr(), lin.svh.data_ptr(),
                      m, lin.in_features, n, lin.K, cb, bufs, ctls, rank, self.N, self.cap,
                      torch.cuda.current_stream(x.device).cuda_stream)

    def gathered_linear(self, lin, out, rank=None):
        """out (m, n) = lin(all-reduced input): the input (m, k) is the sum of the partials the
        ranks pushed with their last linear_push, added up inside the kernel's input rotation."""
        from . import _lib
        rank = self.rank if rank is None else rank
        m, n = out.shape[0], lin.out_features
        if not (out.is_cuda and out.is_contiguous() and out.dim() == 2 and out.shape[1] == n and 1 <= m <= 16
                and out.dtype in (torch.float16, torch.float32) and m * lin.in_features <= self.cap and lin.bias is None):
            raise ValueError("comm.gathered_linear: out must be a contiguous (m <= 16, n) fp16/fp32 CUDA tensor, m * k <= cap")
        buf, ctl = self._local[rank]
        cb = 2 if lin.mul1 else (1 if lin.mcg else 0)
        with torch.cuda.device(out.device):
            _lib.call("amp_exl3_gemv_gathered", lin.trellis.data_ptr(), out.data_ptr(), lin.suh.data_ptr(), lin.svh.data_ptr(),
                      m, lin.in_features, n, lin.K, cb, int(out.dtype == torch.float32), buf, ctl, self.N, self.cap,
                      torch.cuda.current_stream(out.device).cuda_stream)
        return out

    def gathered_bundle(self, bundle, m, rank=None):
        """A models.Multi or models.Sliced bundle run on the all-reduced input (see
        gathered_linear); writes the bundle's own output buffers."""
        from . import _lib
        rank = self.rank if rank is None else rank
        a = bundle.linears[0]
        if not (1 <= m <= 16 and m * a.in_features <= self.cap):
            raise ValueError("comm.gathered_bundle: m <= 16 and m * k <= cap")
        buf, ctl = self._local[rank]
        cb = 2 if a.mul1 else (1 if a.mcg else 0)
        opts = getattr(bundle, "opts", None)
        if opts is None:
            C, num, width = bundle.out, len(bundle.linears), a.out_features
            cp = ns = hs = None
        else:
            C, num, width = bundle.carrier, bundle.slices, bundle.width
            cp, ns, hs = opts["c_ptrs"].data_ptr(), opts["n_stride_list"].data_ptr(), opts["had_src_list"].data_ptr()
        with torch.cuda.device(C.device):
            _lib.call("amp_exl3_mgemm_gathered", bundle.B.data_ptr(), C.data_ptr(), bundle.suh.data_ptr(), bundle.svh.data_ptr(),
                      num, m, a.in_features, width, a.K, cb, 0, cp, ns, hs, buf, ctl, self.N, self.cap,
                      torch.cuda.current_stream(C.device).cuda_stream)

    def status(self, rank=None):
        """Non-zero when a bounded wait for a peer ran out since the last query."""
        rank = self.rank if rank is None else rank
        return self.backend.status(self._local[rank][1])

    def info(self):
        return {"ranks": self.N, "cap": self.cap, "mode": "twophase" if self.mode else "oneshot"}

    def close(self):
        for p in self._opened:
            self.backend.close(p)
        self._opened = []
        for buf, ctl in self._local.values():
            self.backend.free(buf)
            self.backend.free(ctl)
        self._local = {}


class _device:
    def __init__(self, idx, backend):
        self.ctx = torch.cuda.device(idx) if backend is None else None

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *a):
        if self.ctx is not None:
            self.ctx.__exit__(*a)


def p2p_comm(devices, cap, mode=None):
    """torch.p2p_comm(devices, cap, mode?): one process, rank = position in `devices`."""
    if not isinstance(devices, (list, tuple)):
        raise TypeError("expected (devices array, cap (multiple of 8), mode?)")
    return P2PComm.single_process(devices, cap, mode)
