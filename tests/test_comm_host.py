"""CPU tests of the all-reduce communicator's host logic: argument checks, mode resolution, and
the one-process-per-GPU construction over a world_size-2 gloo group with a fake device backend
(handles travel through the group, every rank ends up with the same rank-ordered pointer table)."""
import multiprocessing as mp
import os
import socket

import pytest

torch = pytest.importorskip("torch")


class FakeBackend:
    """Stands in for the CUDA backend: 'pointers' are integers derived from the owning rank,
    'handles' are their 64-byte encodings."""

    def __init__(self, rank):
        self.rank, self.n_alloc, self.launches = rank, 0, []

    def buffer_bytes(self, N, cap):
        return (2 * N + 2) * (cap // 2) * 8

    def ctl_bytes(self):
        return 128

    def blocks(self, N, n):
        return max(1, min(16, n // 4 // 2048))

    def alloc(self, nbytes):
        self.n_alloc += 1
        ptr = 0x10000 * (self.rank + 1) + 0x100 * self.n_alloc
        return ptr, ptr.to_bytes(8, "little") + bytes(56)

    def open(self, handle):
        return int.from_bytes(handle[:8], "little") + 0x1000000      # a different address space

    def close(self, ptr):
        pass

    def free(self, ptr):
        pass

    def enable_peer(self, peer):
        pass

    def launch(self, *args):
        self.launches.append(args)

    def status(self, ctl):
        return 0


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    import torch.distributed as dist
    from ampstein_b200.comm import P2PComm
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        be = FakeBackend(rank)
        comm = P2PComm.from_process_group(4096, backend=be)
        bufs, ctls = comm._bufs[rank]
        q.put((rank, comm.info(), [int(v) for v in bufs], [int(v) for v in ctls], comm.rank))
    finally:
        dist.destroy_process_group()


def test_process_group_construction_gloo_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, info, bufs, ctls, crank in res:
        assert info == {"ranks": 2, "cap": 4096, "mode": "oneshot"} and crank == rank
        for r in range(2):
            own_buf, own_ctl = 0x10000 * (r + 1) + 0x100, 0x10000 * (r + 1) + 0x200
            if r == rank:
                assert (bufs[r], ctls[r]) == (own_buf, own_ctl)          # local pointers stay local
            else:
                assert (bufs[r], ctls[r]) == (own_buf + 0x1000000, own_ctl + 0x1000000)   # peers are mapped


def test_argument_checks_and_modes():
    from ampstein_b200.comm import P2PComm, p2p_comm
    be = FakeBackend(0)
    with pytest.raises(ValueError):
        P2PComm.single_process([0], 1024, backend=be)                    # 2..8 devices
    with pytest.raises(ValueError):
        P2PComm.single_process(list(range(9)), 1024, backend=be)
    with pytest.raises(TypeError):
        P2PComm.single_process([0, 1], 1001, backend=be)                 # cap multiple of 8
    with pytest.raises(ValueError):
        P2PComm.single_process([0, 1], 1024, mode="ring", backend=be)
    with pytest.raises(TypeError):
        p2p_comm(3, 1024)
    c = P2PComm.single_process([0, 1, 2, 3], 1024, backend=be)
    assert c.info() == {"ranks": 4, "cap": 1024, "mode": "oneshot"}     # auto = one-shot at every N
    assert P2PComm.single_process([0, 1], 1024, mode="twophase", backend=be).info()["mode"] == "twophase"
    x = torch.zeros(64, dtype=torch.float16)                             # CPU tensor
    with pytest.raises(ValueError):
        c.allreduce(x, 0)
    with pytest.raises(ValueError):
        c.allreduce(x, 7)


def test_c_abi_rejects_bad_arguments_without_a_gpu():
    import ctypes
    from ampstein_b200 import _lib
    L = _lib.lib()
    assert L.amp_comm_buffer_bytes(1, 1024) == -1 and L.amp_comm_buffer_bytes(9, 1024) == -1
    assert L.amp_comm_buffer_bytes(2, 1001) == -1
    assert L.amp_comm_buffer_bytes(8, 40960) == 18 * 20480 * 8
    assert L.amp_comm_blocks(8, 5120) == 3 and L.amp_comm_blocks(8, 40960) == 16 and L.amp_comm_blocks(2, 8) == 1
    arr = (ctypes.c_void_p * 2)(1, 2)
    bad = [dict(N=1), dict(n=12), dict(n=2048, cap=1024), dict(blocks=17), dict(rank=2), dict(mode=2)]
    for kw in bad:
        a = dict(rank=0, N=2, n=1024, cap=1024, mode=0, blocks=1)
        a.update(kw)
        rc = L.amp_comm_allreduce_fp16(1, 1, arr, arr, a["rank"], a["N"], a["n"], a["cap"], a["mode"], a["blocks"], None)
        assert rc == 1, kw          # cudaErrorInvalidValue, as the reference returns
