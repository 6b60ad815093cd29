"""GPU tests of the NVLink all-reduce. Ranks run on DIFFERENT GPUs (kernels that wait on one
another are never co-scheduled on one device); with fewer GPUs than ranks the tests skip. The
bounded-wait test uses one kernel on one GPU whose peer never arrives."""
import os
import subprocess
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from conftest import ROOT


def ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def partial(rank, n, call):
    i = np.arange(n, dtype=np.float64)
    return (np.sin(0.37 * i + 1.7 * rank + 0.11 * call) * (1.0 + 0.25 * rank)).astype(np.float16)


@pytest.mark.parametrize("mode", ["oneshot", "twophase"])
def test_allreduce_exact_single_process(oracle, mode):
    """Every N = 2..min(GPUs, 8): result == fp32 rank-order sum rounded once (exact), identical on
    all ranks, 21 back-to-back calls over 7 sizes including ones no rank count divides."""
    if ngpu() < 2:
        pytest.skip("needs at least two GPUs")
    from ampstein_b200.comm import p2p_comm
    sizes = [8, 5120, 40, 40960, 1000 * 8, 8 * 1237, 65536]
    for N in range(2, min(ngpu(), 8) + 1):
        comm = p2p_comm(list(range(N)), 65536, mode)
        for call in range(21):
            n = sizes[call % len(sizes)]
            parts = [partial(r, n, call) for r in range(N)]
            outs = []
            for r in range(N):
                x = torch.from_numpy(parts[r]).to("cuda:%d" % r)
                outs.append(comm.allreduce(x, r))
            want = oracle.allreduce_fp16(parts).view(np.uint16)
            for r in range(N):
                got = outs[r].cpu().numpy().view(np.uint16)
                assert np.array_equal(got, want), (N, call, n, r)
        for r in range(N):
            assert comm.status(r) == 0
        comm.close()


def test_allreduce_inside_cuda_graphs(oracle):
    """64 all-reduces captured in one CUDA graph per rank and replayed: the call sequence number
    lives on the device."""
    if ngpu() < 2:
        pytest.skip("needs at least two GPUs")
    from ampstein_b200.comm import p2p_comm
    N, n = 2, 5120
    comm = p2p_comm([0, 1], 5120)
    xs = [torch.from_numpy(partial(r, n, 0)).to("cuda:%d" % r) for r in range(N)]
    for r in range(N):                         # warm-up outside capture
        comm.allreduce(xs[r], r)
    for r in range(N):
        torch.cuda.synchronize(r)
    graphs, outs = [], []
    for r in range(N):
        with torch.cuda.device(r):
            g = torch.cuda.CUDAGraph()
            s = torch.cuda.Stream()
            with torch.cuda.stream(s), torch.cuda.graph(g, stream=s):
                y = xs[r]
                for _ in range(64):
                    y = comm.allreduce(xs[r], r)
            graphs.append(g)
            outs.append(y)
    for rep in range(3):
        for r in range(N):
            with torch.cuda.device(r):
                graphs[r].replay()
        for r in range(N):
            torch.cuda.synchronize(r)
    want = oracle.allreduce_fp16([partial(r, n, 0) for r in range(N)]).view(np.uint16)
    for r in range(N):
        assert np.array_equal(outs[r].cpu().numpy().view(np.uint16), want)
        assert comm.status(r) == 0
    comm.close()


def test_one_process_per_gpu_over_torch_distributed(oracle):
    """torchrun-style: two processes, one GPU each, buffers exchanged as CUDA IPC handles."""
    if ngpu() < 2:
        pytest.skip("needs at least two GPUs")
    script = os.path.join(ROOT, "tests", "comm_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29731", script],
                       capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "comm_worker ok rank 0" in r.stdout and "comm_worker ok rank 1" in r.stdout


def test_wait_for_a_missing_peer_runs_out_and_reports():
    """A rank whose peer never launches: the kernel's bounded wait expires (about a second), the
    call returns, the status word says so and the context stays usable. One kernel, one GPU,
    nothing it waits for ever runs."""
    from ampstein_b200.comm import P2PComm
    comm = P2PComm.single_process([0, 0], 1024)          # both ranks' buffers on device 0
    x = torch.ones(1024, dtype=torch.float16, device="cuda:0")
    out = comm.allreduce(x, 0)                           # rank 1 never calls
    torch.cuda.synchronize()
    assert comm.status(0) == 1
    assert comm.status(0) == 0                           # reading clears it
    y = (out.float() + 1).sum().item()                   # the context still works
    assert np.isfinite(y)
    comm.close()


def test_fused_linear_allreduce_matches_gemv_then_allreduce(oracle):
    """Row-parallel linear with the exchange fused into the GEMV epilogue: bit-identical to the
    plain GEMV followed by the stand-alone all-reduce on every rank, equal to the oracle's
    rank-order sum of the fp16 partials, and mixable with plain all-reduce calls on the same
    communicator (shared sequence numbers). Covers the cluster and the global form of the
    partial-sum exchange, batches 1 to 3, and 8 / 13 rows (rotated-input instance)."""
    if ngpu() < 2:
        pytest.skip("needs at least two GPUs")
    from conftest import make_linear
    from ampstein_b200.comm import p2p_comm
    from ampstein_b200.models import LinearEXL3
    for N in sorted({2, min(ngpu(), 8)}):
        comm = p2p_comm(list(range(N)), 4 * 1024)
        for call, (k_local, n, m) in enumerate([(1024, 512, 1), (256, 1024, 3), (1024, 512, 1), (2048, 256, 2),
                                                (1024, 512, 8), (512, 256, 13)]):     # 5+ rows: input rotated by its own launch
            shards = [make_linear(k_local, n, 4, seed=8800 + 10 * call + r, m=m) for r in range(N)]
            lins, xs = [], []
            for r, (trellis, suh, svh, x) in enumerate(shards):
                d = "cuda:%d" % r
                svh = (svh.astype(np.float32) / 40.0).astype(np.float16)
                shards[r] = (trellis, suh, svh, x)
                lins.append(LinearEXL3(torch.from_numpy(trellis.view(np.int16)).to(d), torch.from_numpy(suh).to(d),
                                       torch.from_numpy(svh).to(d)))
                xs.append(torch.from_numpy(x).to(d))
            # reference on the GPU: plain GEMV per rank, then the stand-alone all-reduce
            parts = [lins[r].forward(xs[r]) for r in range(N)]
            plain = [comm.allreduce(parts[r].view(-1), r) for r in range(N)]
            fused = [torch.empty((m, n), dtype=torch.float16, device="cuda:%d" % r) for r in range(N)]
            for r in range(N):
                comm.linear_allreduce(lins[r], xs[r], fused[r], r)
            for r in range(N):
                torch.cuda.synchronize(r)
            for r in range(N):
                assert torch.equal(fused[r].view(-1).cpu(), plain[r].cpu()), (N, call, r)
            # oracle: fp16 partials of every shard, summed in fp32 in rank order, rounded once
            oparts = [oracle.linear(x, t, s, v, 0, fp32_out=False).reshape(-1) for (t, s, v, x) in shards]
            want = oracle.allreduce_fp16(oparts).astype(np.float32)
            got = fused[0].view(-1).float().cpu().numpy()
            assert np.max(np.abs(got - want)) / np.max(np.abs(want)) < 1e-2      # max relative error
        for r in range(N):
            assert comm.status(r) == 0
        comm.close()


def test_split_exchange_push_then_gather_in_the_consumer(oracle):
    """The exchange split between producer and consumer: every rank's row-parallel linear only
    pushes its partial (linear_push); the next linear / bundle adds the ranks' partials up inside
    its input rotation (gathered_linear / gathered_bundle). The consumer's output must equal, bit
    for bit, the same linear applied to the stand-alone all-reduce of the partials; plain and fused
    all-reduce calls on the same communicator stay in step. Batches 1 and 3, a stacked and a
    sliced bundle as consumers."""
    if ngpu() < 2:
        pytest.skip("needs at least two GPUs")
    from conftest import make_linear
    from ampstein_b200.comm import p2p_comm
    from ampstein_b200.models import LinearEXL3, Multi, Sliced

    def lin_on(k, n, seed, d, scale=40.0):
        t, su, sv, _ = make_linear(k, n, 4, seed=seed)
        sv = (sv.astype(np.float32) / scale).astype(np.float16)
        return LinearEXL3(torch.from_numpy(t.view(np.int16)).to(d), torch.from_numpy(su).to(d), torch.from_numpy(sv).to(d))

    for N in sorted({2, min(ngpu(), 8)}):
        hidden = 512
        comm = p2p_comm(list(range(N)), 3 * hidden)
        for call, (k_local, m) in enumerate([(1024, 1), (256, 3), (2048, 2)]):
            prod, xs, cons, bund, sl = [], [], [], [], []
            for r in range(N):
                d = "cuda:%d" % r
                prod.append(lin_on(k_local, hidden, 9000 + 10 * call + r, d))
                xs.append(torch.randn((m, k_local), generator=torch.Generator().manual_seed(call * 10 + r)).to(torch.float16).to(d))
                cons.append(lin_on(hidden, 384, 9100 + call, d, 30.0))                       # the same consumer on every rank
                g, u = lin_on(hidden, 256, 9200 + call, d, 30.0), lin_on(hidden, 256, 9300 + call, d, 30.0)
                bund.append(Multi([g, u], torch.empty((2, m, 256), dtype=torch.float16, device=d)))
                q, kk = lin_on(hidden, 512, 9400 + call, d, 30.0), lin_on(hidden, 128, 9500 + call, d, 30.0)
                sl.append(Sliced([q, kk], [torch.empty((1, m, 512), dtype=torch.float16, device=d),
                                           torch.empty((1, m, 128), dtype=torch.float16, device=d)]))
            # the all-reduced hidden state by the stand-alone path
            parts = [prod[r].forward(xs[r]) for r in range(N)]
            summed = [comm.allreduce(parts[r].view(-1), r).view(m, hidden) for r in range(N)]
            for consumer in ("linear", "multi", "sliced"):
                for r in range(N):
                    comm.linear_push(prod[r], xs[r], r)
                outs, want = [], []
                for r in range(N):
                    d = "cuda:%d" % r
                    if consumer == "linear":
                        y = torch.full((m, 384), float("nan"), dtype=torch.float16, device=d)
                        comm.gathered_linear(cons[r], y, r)
                        outs.append([y])
                        want.append([cons[r].forward(summed[r])])
                    elif consumer == "multi":
                        bund[r].out.fill_(float("nan"))
                        comm.gathered_bundle(bund[r], m, r)
                        outs.append([bund[r].out.clone()])
                        bund[r].run(summed[r].view(1, m, hidden))
                        want.append([bund[r].out.clone()])
                    else:
                        comm.gathered_bundle(sl[r], m, r)
                        outs.append([o.clone() for o in sl[r].outs])
                        sl[r].run(summed[r].view(1, m, hidden))
                        want.append([o.clone() for o in sl[r].outs])
                for r in range(N):
                    torch.cuda.synchronize(r)
                for r in range(N):
                    for a, b in zip(outs[r], want[r]):
                        assert torch.equal(a.cpu(), b.cpu()), (N, call, consumer, r)
                # a fused call in between keeps the sequence numbers of all call kinds in step
                fused = [torch.empty((m, hidden), dtype=torch.float16, device="cuda:%d" % r) for r in range(N)]
                for r in range(N):
                    comm.linear_allreduce(prod[r], xs[r], fused[r], r)
                for r in range(N):
                    torch.cuda.synchronize(r)
                    assert torch.equal(fused[r].cpu(), summed[r].cpu())
        for r in range(N):
            assert comm.status(r) == 0
        comm.close()
