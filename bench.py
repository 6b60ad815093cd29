#!/usr/bin/env python
"""Benchmark of the EXL3 quantized-linear hot path on B200.

Workload (N = 1): the Llama-3-8B-shaped decode step at batch 1 -- 32 layers of q/k/v/o/gate/up/
down EXL3 linears at 4 bits per weight plus a 6-bit lm_head, chained through their activations
and replayed as ONE CUDA graph per token. Weights are seeded synthetic trellis words (every bit
pattern is a valid stream); svh carries random signs scaled so that chained activations stay
O(1) in fp16 without extra kernels. A step streams 3.89 GB of packed weights, far more than the
126 MB L2, so no cache flush is needed between steps.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--mode tp|replicas]
    python bench.py --workload tp5 [--batch 1|8]       (the 64-layer 5-bit tensor-parallel stack)
    python bench.py --workload prefill | moe [--tokens 1|4|16] | issue        (secondary, one GPU)

With N > 1 GPUs (one process per GPU under torchrun) the stack is decoded tensor-parallel, as the
reference shards it: q|k|v and gate|up column-parallel, o and down row-parallel, each followed
by the fp16 all-reduce of the hidden state over NVLink (this library's kernel, inside the graph);
lm_head is split by vocabulary. All ranks decode the same token, so the work is fixed as N grows
(strong scaling). Before timing, every rank checks the exchange after o_proj / down_proj of layer 0
against the fp32 rank-order sum (rounded once) of the gathered partial products. `--exchange` picks
its form: fused into the producer (default), split between producer and consumer, or a launch of
its own. `--mode replicas` runs N independent copies of the 1-GPU step instead.

One JSON line on stdout (rank 0). The `--steps` block is repeated until at least a second has
been timed and the median block is reported. `--impl reference` times the CPU restatement of the
reference's reconstruct-then-matmul path (the reference has no CPU code of its own for this
codebook) on the host cores, on a bounded sample of the same workload.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode tok/s (8B-shape EXL3 4bpw stack)"
UNIT = "tok/s"

# hidden, q width, kv width, ffn, vocabulary (0: no lm_head), layers, bits per weight (layers, head)
STACKS = {
    "decode": dict(name="llama3-8b-shaped", hidden=4096, q=4096, kv=1024, ffn=14336, vocab=128256, layers=32, K=4, K_head=6),
    "tp5": dict(name="64-layer dense 5 bpw (hidden 5120)", hidden=5120, q=6144, kv=1024, ffn=25600, vocab=0, layers=64, K=5, K_head=0),
}
MIN_TIMED_S = 1.0


def layer_linears(S, rank=0, world=1):
    """(name, in, out, in of the unsharded matrix) of one layer for a rank of a tensor-parallel
    group: column-parallel q/k/v/gate/up, row-parallel o/down (reference:
    src/ucode/ampstein/models.uc:527-562); attention by kv head (128 wide), the MLP in 256-column
    units by largest remainder (src/ucode/ampstein/qwen35_tp.uc:40-79)."""
    from ampstein_b200.models import split_n
    h, q, kv, ffn = S["hidden"], S["q"], S["kv"], S["ffn"]
    if world == 1:
        fl = ffn
    else:
        if (kv // 128) % world or (q // 128) % world:
            raise SystemExit("bench.py: %d kv heads do not split %d ways" % (kv // 128, world))
        fl = split_n(ffn, 256, [1] * world)[rank][1]
    ql, kl = q // world, kv // world
    return [("q", h, ql, h), ("k", h, kl, h), ("v", h, kl, h), ("o", ql, h, q),
            ("gate", h, fl, h), ("up", h, fl, h), ("down", fl, h, ffn)]


def head_shape(S, rank=0, world=1):
    if not S["vocab"]:
        return None
    blocks = S["vocab"] // 128
    b0, b1 = blocks * rank // world, blocks * (rank + 1) // world
    return (S["hidden"], (b1 - b0) * 128)


def algorithmic_bytes(S, m=1, rank=0, world=1):
    """Bytes a step must move on one GPU: packed weights + suh/svh + activations in and out."""
    total = 0
    for _, k, n, _ in layer_linears(S, rank, world):
        total += k * n * S["K"] // 8 + 2 * (k + n) + 2 * m * (k + n)
    total *= S["layers"]
    hs = head_shape(S, rank, world)
    if hs:
        total += hs[0] * hs[1] * S["K_head"] // 8 + 2 * (hs[0] + hs[1]) + 2 * m * (hs[0] + hs[1])
    return total


# ------------------------------------------------------------------------------------------
# clocks sampled during the timed region
# ------------------------------------------------------------------------------------------

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for (t, r) in self.rows if t0 - 0.05 <= t <= t1 + 0.15 and len(r) >= 6] or \
               [r for (_, r) in self.rows if len(r) >= 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        mhz = sorted(int(r[0]) for r in rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None,
                "sm_max_mhz": int(rows[0][1]) if rows[0][1].isdigit() else None,
                "reasons": reasons, "samples": len(rows)}


def _peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        return {}


def timed_blocks(torch, fn, steps, stream=None, barrier=None, reduce_max=None, min_s=MIN_TIMED_S, max_blocks=400):
    """Runs blocks of `steps` calls of fn, each bracketed by CUDA events on `stream`, until at
    least min_s seconds have been timed; returns (median block ms, blocks, total ms)."""
    stream = stream or torch.cuda.current_stream()
    times = []
    total = 0.0
    while total < min_s * 1e3 and len(times) < max_blocks:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if barrier:
            barrier()
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
        if barrier:
            barrier()
        else:
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if reduce_max:
            ms = reduce_max(ms)              # the same value on every rank: all ranks stop together
        times.append(ms)
        total += ms
    times.sort()
    return times[len(times) // 2], len(times), total


# ------------------------------------------------------------------------------------------
# the decode arm (1 GPU, replicas, or tensor parallel)
# ------------------------------------------------------------------------------------------

def build_stack(torch, device, seed, S, rank=0, world=1):
    """Distinct synthetic tensors for every linear of the stack."""
    from ampstein_b200.models import LinearEXL3
    g = torch.Generator(device=device)
    g.manual_seed(seed)

    def make(k, n, K, k_full=None):
        trellis = torch.randint(-32768, 32768, (k // 16, n // 16, 16 * K), dtype=torch.int16,
                                device=device, generator=g)
        sgn = lambda c: (torch.randint(0, 2, (c,), device=device, generator=g).to(torch.float16) * 2 - 1)
        suh = sgn(k)
        # decoded weights have std 1.2437: keep chained activations at unit scale
        svh = sgn(n) * (1.0 / (1.2437 * math.sqrt(k_full or k)))
        return LinearEXL3(trellis, suh, svh.to(torch.float16))

    shapes = layer_linears(S, rank, world)
    layers = [{name: make(k, n, S["K"], kf) for name, k, n, kf in shapes} for _ in range(S["layers"])]
    hs = head_shape(S, rank, world)
    head = make(hs[0], hs[1], S["K_head"]) if hs else None
    return layers, head


def run_decode(args, S):
    import torch
    import ampstein_b200  # noqa: F401  (raises if the CUDA library is missing)
    from ampstein_b200.models import DecodeGraph, Multi, Sliced

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the path has no CPU fallback)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    m = args.batch
    H = S["hidden"]
    tp = world if (world > 1 and args.mode == "tp") else 1
    shapes = {name: (k, n) for name, k, n, _ in layer_linears(S, rank if tp > 1 else 0, tp)}
    layers, head = build_stack(torch, device, 1234 + rank, S, rank if tp > 1 else 0, tp)
    f16 = dict(dtype=torch.float16, device=device)
    h_in = torch.empty((1, m, H), **f16)
    bufs = {"q": torch.empty((1, m, shapes["q"][1]), **f16), "k": torch.empty((1, m, shapes["k"][1]), **f16),
            "v": torch.empty((1, m, shapes["v"][1]), **f16), "a": torch.empty((1, m, H), **f16),
            "gu": torch.empty((2, m, shapes["gate"][1]), **f16), "h": torch.empty((1, m, H), **f16)}
    out_buf = torch.empty((m, head.out_features), **f16) if head else bufs["h"][0]
    comm = None
    if tp > 1:
        # partial sums of the row-parallel o / down, all-reduced over NVLink inside the graph
        from ampstein_b200.comm import P2PComm
        bufs["a_part"] = torch.empty((1, m, H), **f16)
        bufs["h_part"] = torch.empty((1, m, H), **f16)
        comm = P2PComm.from_process_group(cap=m * H)
    # the reference's decode step runs q|k|v as one sliced bundle and gate|up as one stacked bundle
    # (src/ucode/ampstein/graphdec.uc:163-210): four launches per layer
    qkv = [Sliced([L["q"], L["k"], L["v"]], [bufs["q"], bufs["k"], bufs["v"]]) for L in layers]
    gu = [Multi([L["gate"], L["up"]], bufs["gu"]) for L in layers]
    launches = [0]

    exchange = args.exchange if comm is not None else None

    def step(stub=False):
        # stub: the row-parallel linears without their all-reduce (to price the exchange)
        x = h_in
        n = 0
        mode = None if stub else exchange
        pushed = False                                   # split: the hidden state is still in the exchange buffers
        last = len(layers) - 1
        for i, L in enumerate(layers):
            if pushed:
                comm.gathered_bundle(qkv[i], m)
            else:
                qkv[i].run(x)
            if mode is None:
                L["o"].forward(bufs["q"][0], bufs["a"][0])        # attention itself is outside the path
                gu[i].run(bufs["a"])
            elif mode == "separate":
                L["o"].forward(bufs["q"][0], bufs["a_part"][0])
                comm.allreduce(bufs["a_part"], out=bufs["a"])
                gu[i].run(bufs["a"])
            elif mode == "fused":
                comm.linear_allreduce(L["o"], bufs["q"][0], bufs["a"][0])
                gu[i].run(bufs["a"])
            else:
                comm.linear_push(L["o"], bufs["q"][0])
                comm.gathered_bundle(gu[i], m)
            pushed = False
            if mode is None:
                L["down"].forward(bufs["gu"][0], bufs["h"][0])
            elif mode == "separate":
                L["down"].forward(bufs["gu"][0], bufs["h_part"][0])
                comm.allreduce(bufs["h_part"], out=bufs["h"])
            elif mode == "fused" or (i == last and head is None):
                comm.linear_allreduce(L["down"], bufs["gu"][0], bufs["h"][0])     # (split: the step's output must exist)
            else:
                comm.linear_push(L["down"], bufs["gu"][0])
                pushed = True
            n += 6 if mode == "separate" else 4
            x = bufs["h"]
        if head:
            if pushed:
                comm.gathered_linear(head, out_buf)
            else:
                head.forward(x[0], out_buf)
            n += 1
        if not stub:
            launches[0] = n

    host_x = torch.randn((m, H), dtype=torch.float16).pin_memory()
    host_out = torch.empty(tuple(out_buf.shape), dtype=torch.float16).pin_memory()
    h_in.copy_(host_x.view(1, m, H))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    allreduce_check = None
    if comm is not None:
        # Parity of the exchange, once before timing: the fused row-parallel linears of layer 0 must
        # equal, bit for bit and on every rank, the fp32 rank-order sum (rounded once) of the ranks'
        # fp16 partial products; so must the stand-alone all-reduce.
        gen = torch.Generator(device=device)
        gen.manual_seed(99 + rank)
        ok = True
        for name in ("o", "down"):
            xin = torch.randn((m, shapes[name][0]), device=device, generator=gen).to(torch.float16)
            part = torch.empty((m, H), **f16)
            layers[0][name].forward(xin, part)
            gathered = [torch.empty_like(part) for _ in range(world)]
            dist.all_gather(gathered, part)
            acc = gathered[0].float()
            for p in gathered[1:]:
                acc = acc + p.float()
            want = acc.to(torch.float16)
            fused = torch.empty((m, H), **f16)
            comm.linear_allreduce(layers[0][name], xin, fused)
            sep = torch.empty((1, m, H), **f16)
            comm.allreduce(part.view(1, m, H), out=sep)
            # split form: push, then a consumer that gathers; the consumer applied to `want` must agree
            comm.linear_push(layers[0][name], xin)
            got = torch.empty((m, shapes["q"][1]), **f16)
            comm.gathered_linear(layers[0]["q"], got)
            ref = torch.empty_like(got)
            layers[0]["q"].forward(want, ref)
            torch.cuda.synchronize()
            ok = ok and torch.equal(fused, want) and torch.equal(sep[0], want) and torch.equal(got, ref)
        flag = torch.tensor([1 if ok else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) != 1:
            raise SystemExit("bench.py: the all-reduce of layer 0 differs from the fp32 rank-order sum of the partial products")
        allreduce_check = "exact"

    graph = DecodeGraph(step, warmup=2)
    stream = graph.stream

    def resident_step():
        graph.replay()

    def e2e_step():
        h_in.copy_(host_x.view(1, m, H), non_blocking=True)
        graph.replay()
        host_out.copy_(out_buf, non_blocking=True)

    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            e2e_step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    t0 = time.time()
    ms, nblk, tot = timed_blocks(torch, resident_step, args.steps, stream, barrier, reduce_max)
    ms_e2e, _, _ = timed_blocks(torch, e2e_step, args.steps, stream, barrier, reduce_max)
    t1 = time.time()
    ms_stub = None
    if comm is not None:
        # the same graph without the exchange: the difference is what the all-reduces cost
        # (values diverge between ranks here; only the time is used)
        stub_graph = DecodeGraph(lambda: step(stub=True), warmup=1, stream=stream)
        ms_stub, _, _ = timed_blocks(torch, stub_graph.replay, args.steps, stream, barrier, reduce_max)
    clocks = sampler.stop(t0, t1) if sampler else None

    res = host_out.float()
    if not torch.isfinite(res).all() or float(res.abs().max()) == 0.0:
        raise SystemExit("bench.py: step produced non-finite or all-zero outputs")

    if comm is not None:
        t = torch.tensor([comm.status()], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if int(t.item()):
            raise SystemExit("bench.py: an all-reduce gave up waiting for a peer (status %d)" % int(t.item()))

    per_shape = None
    if world == 1 and args.workload == "decode" and not args.no_secondary:
        per_shape = per_shape_us(torch, layers, head, bufs, h_in, out_buf, qkv, gu, stream)
    if rank != 0:
        return
    ms_step = ms / args.steps
    # tensor parallel: every rank decodes the same tokens; replicas: one batch per rank
    streams = 1 if tp > 1 else world
    tok_s = streams * m * 1000.0 / ms_step
    tok_s_e2e = streams * m * 1000.0 / (ms_e2e / args.steps)
    gemv_launches = 4 * S["layers"] + (1 if head else 0)
    bytes_step = algorithmic_bytes(S, m, 0, tp)
    peaks = _peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = bytes_step / (ms_step * 1e-3) / 1e9
    metric = METRIC if args.workload == "decode" else "decode tok/s (64-layer 5 bpw tensor-parallel stack, hidden 5120)"
    wl = "%s decode step, batch %d, EXL3 %d bpw x%d layers%s, one CUDA graph" % (
        S["name"], m, S["K"], S["layers"], (" + %d bpw lm_head" % S["K_head"]) if head else "")
    line = {
        "metric": metric, "value": round(tok_s, 2), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "strong" if tp > 1 else "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": wl,
                   "l2": "inputs larger than L2 (%.2f GB of weights streamed per step and GPU)" % (bytes_step / 1e9),
                   "parallelism": ("tp%d: column-parallel q|k|v, gate|up; row-parallel o, down with the fp16 all-reduce (%d per step) over NVLink %s%s"
                                   % (tp, 2 * S["layers"], {"separate": "as separate launches", "fused": "fused into the GEMV epilogue",
                                                              "split": "pushed from the GEMV epilogue and gathered in the consuming GEMV's prologue"}[args.exchange],
                                      "; lm_head by vocabulary" if head else "")) if tp > 1 else ("replicas x%d" % world),
                   "timing": "median of %d blocks of %d steps (%.2f s timed)" % (nblk, args.steps, tot / 1e3)},
        "e2e": {"value": round(tok_s_e2e, 2), "unit": UNIT,
                "h2d_bytes_per_step": host_x.numel() * 2, "d2h_bytes_per_step": host_out.numel() * 2},
        "gpu_launches": launches[0] * args.steps,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4),
                     "peak_source": "measured (MEASURED_PEAKS.json)" if "hbm_gbs" in peaks else "fallback",
                     "kernel": "exl3_gemv_kernel", "bytes_per_launch": bytes_step // gemv_launches,
                     "launches_per_step": gemv_launches, "per": "gpu",
                     # DRAM bytes per launch: dram__bytes_read + write of an ncu capture of the four
                     # layer shapes came to 1.004 x the algorithmic bytes (traffic scales with the weights)
                     "traffic": int(1.004 * bytes_step) // gemv_launches,
                     "traffic_source": "ncu capture on a 2-layer stack, scaled by weight bytes"},
    }
    if ms_stub is not None:
        line["allreduce"] = {"per_step": 2 * S["layers"], "bytes": m * H * 2,
                             "ms_per_step_without": round(ms_stub / args.steps, 4),
                             "share_of_step": round(max(0.0, 1.0 - ms_stub / ms), 4),
                             "us_each": round(max(0.0, ms - ms_stub) / args.steps / (2 * S["layers"]) * 1e3, 2)}
        line["allreduce_check"] = allreduce_check
    if per_shape:
        line["per_shape_us"] = per_shape
    if world == 1 and args.workload == "decode":
        line["cpu_baseline"] = cpu_baseline()
        if not args.no_secondary:
            line["secondary"] = secondary()
    print(json.dumps(line), flush=True)


def per_shape_us(torch, layers, head, bufs, h_in, out_buf, qkv, gu, stream):
    """Time of each of the layer's four launches (and the lm_head) on their own: one CUDA graph per
    shape that runs the launch of every layer in turn (distinct weights, larger than L2), so that
    the step reads as the sum of its launches."""
    from ampstein_b200.models import DecodeGraph
    n = len(layers)
    progs = {
        "q|k|v": lambda: [qkv[i].run(h_in) for i in range(n)],
        "o": lambda: [L["o"].forward(bufs["q"][0], bufs["a"][0]) for L in layers],
        "gate|up": lambda: [gu[i].run(bufs["a"]) for i in range(n)],
        "down": lambda: [L["down"].forward(bufs["gu"][0], bufs["h"][0]) for L in layers],
    }
    out = {}
    for name, fn in progs.items():
        g = DecodeGraph(fn, warmup=1, stream=stream)
        ms, _, _ = timed_blocks(torch, g.replay, 8, stream, min_s=0.1)
        out[name] = round(ms / 8 / n * 1e3, 2)
    total = sum(out.values()) * n
    if head:
        g = DecodeGraph(lambda: head.forward(bufs["h"][0], out_buf), warmup=1, stream=stream)
        ms, _, _ = timed_blocks(torch, g.replay, 8, stream, min_s=0.1)
        out["lm_head"] = round(ms / 8 * 1e3, 2)
        total += out["lm_head"]
    out["sum_per_step_ms"] = round(total / 1e3, 4)
    return out


# ------------------------------------------------------------------------------------------
# secondary workloads (one GPU): the prefill GEMM, the fused decode MoE, the issue microbenchmark
# ------------------------------------------------------------------------------------------

LAYER_8B = [("q", 4096, 4096), ("k", 4096, 1024), ("v", 4096, 1024), ("o", 4096, 4096),
            ("gate", 4096, 14336), ("up", 4096, 14336), ("down", 14336, 4096)]


def measure_prefill(steps, warmup, bundles=True):
    """One decoder layer's seven linears at M = 2048 tokens, bf16 activations, mixed bit widths
    (attention K=5, gate/up K=3, down K=4): the tensor-core (tcgen05) trellis-decode GEMM,
    including the input rotation kernels. q|k|v and gate|up run as bundles (one grid each, the
    reference's mgemm with its sliced / stacked tables) unless bundles is False; one step = the
    layer's seven GEMMs."""
    import torch
    import ampstein_b200 as amp
    from ampstein_b200.models import LinearEXL3, Multi, Sliced
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    M = 2048
    bits = {"q": 5, "k": 5, "v": 5, "o": 5, "gate": 3, "up": 3, "down": 4}
    lin, xs, ys = {}, {}, {}
    for name, k, n in LAYER_8B:
        K = bits[name]
        t = torch.randint(-32768, 32768, (k // 16, n // 16, 16 * K), dtype=torch.int16, device=dev, generator=g)
        sgn = lambda c: (torch.randint(0, 2, (c,), device=dev, generator=g).to(torch.float16) * 2 - 1)
        svh = (sgn(n) * (1.0 / (1.2437 * math.sqrt(k)))).to(torch.float16)
        lin[name] = LinearEXL3(t, sgn(k), svh)
        xs[name] = torch.randn((1, M, k), device=dev, generator=g).to(torch.bfloat16)
        ys[name] = torch.empty((1, M, n), dtype=torch.float16, device=dev)
    flops = sum(2.0 * M * k * n for _, k, n in LAYER_8B)
    gu_out = torch.empty((2, M, 14336), dtype=torch.float16, device=dev)
    qkv = Sliced([lin["q"], lin["k"], lin["v"]], [ys["q"], ys["k"], ys["v"]])
    gu = Multi([lin["gate"], lin["up"]], gu_out)
    had3 = torch.empty((3, M, 4096), dtype=torch.float16, device=dev)

    def single(name):
        w = lin[name]
        amp.exl3_gemm(xs[name][0], w.trellis, ys[name][0], w.suh, w.svh)

    def step():
        if bundles:
            qkv.run(xs["q"], had3)
            single("o")
            gu.run(xs["gate"], had3)
        else:
            for name in ("q", "k", "v", "o", "gate", "up"):
                single(name)
        single("down")

    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    t0 = time.time()
    ms_blk, nblk, _ = timed_blocks(torch, step, steps, min_s=0.5)
    clocks = sampler.stop(t0, time.time())
    ms = ms_blk / steps
    outs = [ys[n] for n in ("q", "k", "v", "o", "down")] + ([gu_out] if bundles else [ys["gate"], ys["up"]])
    if not all(torch.isfinite(o.float()).all() for o in outs):
        raise SystemExit("bench.py: prefill produced non-finite outputs")
    peaks = _peaks()
    peak = float(peaks.get("bf16_tflops", 1590.0))
    tf = flops / ms / 1e9
    launches = 8 if bundles else 14
    return {
        "metric": "prefill TFLOP/s (one 8B-shaped layer, M=2048, EXL3 K=5/3/4)", "value": round(tf, 1), "unit": "TFLOP/s",
        "n_gpus": 1, "steps": steps, "warmup": max(warmup, 3), "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "prefill: 7 linears of one llama3-8b-shaped layer, M=2048 bf16 tokens, K=5 attention / 3 gate,up / 4 down",
                   "launches": "q|k|v and gate|up as bundles (one grid each), o and down single" if bundles else "seven separate GEMMs",
                   "l2": "operands of a step: 0.23 GB (weights read once per GEMM)",
                   "timing": "median of %d blocks of %d steps" % (nblk, steps)},
        "gpu_launches": launches * steps, "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": round(tf, 1), "peak": peak, "unit": "TFLOP/s", "frac": round(tf / peak, 4),
                     "peak_source": "measured burst (MEASURED_PEAKS.json)" if "bf16_tflops" in peaks else "fallback",
                     "kernel": "exl3_gemm_tc2_kernel", "traffic": None}}


def moe_launches(T):
    """kernels per fused MoE layer: (run table for more than one token,) gate|up, down"""
    return 2 if T == 1 else 3


def measure_moe(steps, warmup, T):
    """Fused decode MoE: 128 experts 2048 -> 768 -> 2048 at K=3, top-8 routing from fp32 router
    logits ~ N(0,1), T tokens per step. Eight different routings are captured in one CUDA graph so
    that successive layers hit different experts; one step = one MoE layer."""
    import numpy as np
    import torch
    import ampstein_b200 as amp
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(11)
    E, Hi, I, Ho, K, topk = 128, 2048, 768, 2048, 3, 8
    tr = lambda k, n: torch.randint(-32768, 32768, (k // 16, n // 16, 16 * K), dtype=torch.int16, device=dev, generator=g)
    sg = lambda c, s=1.0: ((torch.randint(0, 2, (c,), device=dev, generator=g).to(torch.float16) * 2 - 1) * s).to(torch.float16)
    ex = [dict(g=(tr(Hi, I), sg(Hi), sg(I, 1 / (1.2437 * math.sqrt(Hi)))), u=(tr(Hi, I), sg(Hi), sg(I, 1 / (1.2437 * math.sqrt(Hi)))),
               d=(tr(I, Ho), sg(I), sg(Ho, 1 / (1.2437 * math.sqrt(I))))) for _ in range(E)]
    tab = lambda key, i: amp.ptr_array([e[key][i].data_ptr() for e in ex])
    slots = T * topk
    cfg = dict(g_trellis=tab("g", 0), g_suh=tab("g", 1), g_svh=tab("g", 2), u_trellis=tab("u", 0), u_suh=tab("u", 1), u_svh=tab("u", 2),
               d_trellis=tab("d", 0), d_suh=tab("d", 1), d_svh=tab("d", 2),
               gu_g=torch.zeros(slots, I, dtype=torch.float16, device=dev), gu_u=torch.zeros(slots, I, dtype=torch.float16, device=dev),
               d_out=torch.zeros(slots, Ho, dtype=torch.float32, device=dev),
               ctr=torch.zeros(amp.moe_coop_ctr_len(slots, T, I, Ho), dtype=torch.int32, device=dev),
               out=torch.zeros(T, Hi, dtype=torch.float32, device=dev), Hi=Hi, Kg=K, Ku=K, Kd=K, act=0, act_limit=0.0)
    sets = []
    for _ in range(8):
        w, sel = torch.topk(torch.randn(T, E, device=dev, generator=g), topk, dim=1)
        sets.append((torch.randn(T, Hi, device=dev, generator=g).to(torch.float16), sel.contiguous(),
                     torch.softmax(w, 1).to(torch.float16).contiguous()))
    distinct = float(np.mean([len(torch.unique(s[1])) for s in sets]))
    gr, st = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(st):                       # (the stream's workspace is created here, before capture)
        for x, sel, rw in sets:
            amp.moe_coop(x, sel, rw, cfg)
    torch.cuda.synchronize()
    with torch.cuda.stream(st), torch.cuda.graph(gr, stream=st):
        for x, sel, rw in sets:
            amp.moe_coop(x, sel, rw, cfg)
    for _ in range(max(warmup, 3)):
        gr.replay()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    t0 = time.time()
    ms_blk, _, _ = timed_blocks(torch, gr.replay, steps, min_s=0.3)
    clocks = sampler.stop(t0, time.time())
    us = ms_blk * 1e3 / (steps * len(sets))
    if not torch.isfinite(cfg["out"]).all():
        raise SystemExit("bench.py: MoE produced non-finite outputs")
    byt = distinct * 3 * Hi * I * K // 8
    peaks = _peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    gbs = byt / us / 1e3
    return {
        "metric": "fused decode MoE layer time (128 experts, top-8, K=3)", "value": round(us, 2), "unit": "us/layer",
        "n_gpus": 1, "steps": steps, "warmup": max(warmup, 3), "ms_per_step": round(us * len(sets) / 1e3, 4),
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "moe decode: 128 experts 2048->768->2048 K=3, top-8, %d token(s), 8 routings per graph" % T,
                   "distinct_experts_per_layer": round(distinct, 1),
                   "l2": "expert weights in total 226 MB (larger than L2); each layer touches %.1f MB" % (byt / 1e6)},
        "gpu_launches": moe_launches(T) * len(sets) * steps, "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(gbs / peak, 4),
                     "peak_source": "measured (MEASURED_PEAKS.json)" if "hbm_gbs" in peaks else "fallback",
                     "kernel": "exl3_gemv_kernel (grouped modes)", "bytes_per_launch": int(byt) // 2, "traffic": None}}


def measure_moe_prefill(steps, warmup, T=2048):
    """Token-sorted MoE of a prefill chunk: 128 experts 2048 -> 768 -> 2048 at K=3, top-8 routing
    from fp32 router logits ~ N(0,1), T tokens per step (about T / 16 rows per expert). The routing
    is sorted by expert beforehand (as for the reference's torch.moe_fused, which takes the sorted
    lists); one step = one call of moe_fused = one MoE layer; four routings take turns."""
    import torch
    import ampstein_b200 as amp
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(13)
    E, H, I, K, topk = 128, 2048, 768, 3, 8
    tr = lambda k, n: torch.randint(-32768, 32768, (k // 16, n // 16, 16 * K), dtype=torch.int16, device=dev, generator=g)
    sg = lambda c, s=1.0: ((torch.randint(0, 2, (c,), device=dev, generator=g).to(torch.float16) * 2 - 1) * s).to(torch.float16)
    ex = [dict(g=(tr(H, I), sg(H), sg(I, 1 / (1.2437 * math.sqrt(H)))), u=(tr(H, I), sg(H), sg(I, 1 / (1.2437 * math.sqrt(H)))),
               d=(tr(I, H), sg(I), sg(H, 1 / (1.2437 * math.sqrt(I))))) for _ in range(E)]
    tab = lambda key, i: amp.ptr_array([e[key][i].data_ptr() for e in ex])
    cfg = dict(g_trellis=tab("g", 0), g_suh=tab("g", 1), g_svh=tab("g", 2), u_trellis=tab("u", 0), u_suh=tab("u", 1), u_svh=tab("u", 2),
               d_trellis=tab("d", 0), d_suh=tab("d", 1), d_svh=tab("d", 2), I=I, Kg=K, Ku=K, Kd=K, act=0, act_limit=0.0)
    sets = []
    for _ in range(4):
        w, sel = torch.topk(torch.randn(T, E, device=dev, generator=g), topk, dim=1)
        pr = amp.moe_prep(sel.contiguous(), torch.softmax(w, 1).contiguous(), E, 0)      # [fe, order, tok, wts, count, ...]
        sets.append((torch.randn(T, H, device=dev, generator=g).to(torch.float16), pr[4], pr[2], pr[3]))
    out = torch.zeros(T, H, dtype=torch.float32, device=dev)
    rows_max = int(max(s[1][:E].max().item() for s in sets))

    def layer():
        for y, count, tok, wts in sets:
            amp.moe_fused(y, out, count, tok, wts, cfg)

    for _ in range(max(warmup, 3)):
        layer()
    torch.cuda.synchronize()
    if amp.moe_fused_status(cfg) != 0 or not torch.isfinite(out).all():
        raise SystemExit("bench.py: the sorted MoE reported an error or produced non-finite outputs")
    out.zero_()
    sampler = ClockSampler(0)
    t0 = time.time()
    ms_blk, _, _ = timed_blocks(torch, layer, steps, min_s=0.3)
    clocks = sampler.stop(t0, time.time())
    ms = ms_blk / (steps * len(sets))
    flops = 6.0 * T * topk * H * I
    peaks = _peaks()
    peak = float(peaks.get("bf16_tflops", 1590.0))
    tf = flops / ms / 1e9
    return {
        "metric": "token-sorted prefill MoE layer time (128 experts, top-8, K=3)", "value": round(ms * 1e3, 1), "unit": "us/layer",
        "n_gpus": 1, "steps": steps, "warmup": max(warmup, 3), "ms_per_step": round(ms, 4),
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "moe prefill: 128 experts 2048->768->2048 K=3, top-8, %d tokens per chunk, 4 routings in turn" % T,
                   "rows_per_expert_max": rows_max, "tokens_per_s": round(T / ms * 1e3),
                   "l2": "expert weights 226 MB + %d MB of rotated rows and intermediates per layer (larger than L2)"
                         % ((T * topk * (2 * H * 2 + 3 * I * 2 + H * 4)) >> 20)},
        "gpu_launches": 6 * len(sets) * steps, "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": round(tf, 1), "peak": peak, "unit": "TFLOP/s", "frac": round(tf / peak, 4),
                     "peak_source": "measured (MEASURED_PEAKS.json), burst" if "bf16_tflops" in peaks else "fallback",
                     "kernel": "exl3_gemm_tc_kernel<K, CB, grouped>", "flops_per_layer": int(flops), "traffic": None}}


def measure_gemm(steps, warmup, shape, rows):
    """One prefill shape (rows x k through a k x n weight at K bits) through both many-row forms:
    the tensor-core trellis GEMM (exl3_gemm) and reconstruct_had + a library GEMM (what
    exl3_gemm_recon takes for narrow weights). Distinct weight copies exceed L2; eager launches."""
    import torch
    import ampstein_b200 as amp
    k, n, K = shape
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(6)
    wbytes = k * n * K // 8
    copies = max(2, min(32, -(-2 * 126 * 2 ** 20 // (wbytes + 2 * k * n))))
    mats = [torch.randint(-32768, 32768, (k // 16, n // 16, 16 * K), dtype=torch.int16, device=dev, generator=g) for _ in range(copies)]
    sgn = lambda c: (torch.randint(0, 2, (c,), device=dev, generator=g).to(torch.float16) * 2 - 1)
    suh, svh = sgn(k), (sgn(n) / (1.2437 * math.sqrt(k))).to(torch.float16)
    x = torch.randn((rows, k), device=dev, generator=g).to(torch.float16)
    y = torch.empty((rows, n), dtype=torch.float16, device=dev)
    w = torch.empty((k, n), dtype=torch.float16, device=dev)

    def trellis():
        for t in mats:
            amp.exl3_gemm(x, t, y, suh, svh)

    def recon():
        for t in mats:
            amp.exl3_reconstruct_had(w, t, suh, svh, K)
            torch.mm(x, w, out=y)

    out = {}
    sampler = ClockSampler(0)
    t0 = time.time()
    for name, fn in (("trellis_gemm", trellis), ("reconstruct_plus_library_gemm", recon)):
        for _ in range(max(warmup, 3)):
            fn()
        ms_blk, _, _ = timed_blocks(torch, fn, steps, min_s=0.2)
        us = ms_blk * 1e3 / (steps * copies)
        out[name] = {"us": round(us, 1), "tflops": round(2.0 * rows * k * n / us / 1e6, 1)}
    clocks = sampler.stop(t0, time.time())
    pick = "reconstruct_plus_library_gemm" if n <= amp.exl3.RECON_MM_MAX_N else "trellis_gemm"
    return {"metric": "prefill GEMM time (%d rows x %dx%d, K=%d)" % (rows, k, n, K), "value": out[pick]["us"], "unit": "us/launch",
            "n_gpus": 1, "steps": steps, "warmup": max(warmup, 3), "higher_is_better": False, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "one prefill shape, %d distinct weight copies in turn (larger than L2), eager launches" % copies,
                       "exl3_gemm_recon_takes": pick},
            "forms": out, "gpu_launches": copies * steps, "clocks": clocks}


def measure_gemv(steps, warmup, shape, m, tmem=False, mul1=False, silu_mul=False, norm=False):
    """One decode GEMV shape on its own (k x n at K bits, m rows): as many distinct copies of the
    matrix as it takes to exceed L2 twice over, one launch per copy, all in one CUDA graph."""
    import torch
    import ampstein_b200 as amp
    from ampstein_b200.models import DecodeGraph
    k, n, K = shape
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    wbytes = int(k * n * K) // 8
    copies = max(1, min(64, -(-2 * 126 * 2 ** 20 // wbytes)))
    mats = [torch.randint(-32768, 32768, (k // 16, n // 16, int(16 * K)), dtype=torch.int16, device=dev, generator=g) for _ in range(copies)]
    sgn = lambda c: (torch.randint(0, 2, (c,), device=dev, generator=g).to(torch.float16) * 2 - 1)
    suh, svh = sgn(k), (sgn(n) / (1.2437 * math.sqrt(k))).to(torch.float16)
    x = torch.randn((m, k), device=dev, generator=g).to(torch.float16)
    y = torch.empty((m, n), dtype=torch.float16, device=dev)
    if norm:
        x2 = (0.5 * torch.randn((m, k), device=dev, generator=g)).to(torch.float16)
        nw = (1.0 + 0.05 * torch.randn((k,), device=dev, generator=g)).to(torch.float16)
        yy = torch.empty((m, k), dtype=torch.float16, device=dev)
        graph = DecodeGraph(lambda: [amp.exl3_gemm_rms_norm_res(x, x2, nw, 1e-5, yy, t, y, suh, svh, mul1=mul1) for t in mats],
                            warmup=max(warmup, 3))
    elif silu_mul:
        x2 = torch.randn((m, k), device=dev, generator=g).to(torch.float16)
        graph = DecodeGraph(lambda: [amp.exl3_gemm_silu_mul(x, x2, t, y, suh, svh, mul1=mul1) for t in mats], warmup=max(warmup, 3))
    else:
        graph = DecodeGraph(lambda: [amp.exl3_gemm(x, t, y, suh, svh, mul1=mul1) for t in mats], warmup=max(warmup, 3))
    sampler = ClockSampler(0)
    t0 = time.time()
    ms_blk, nblk, _ = timed_blocks(torch, graph.replay, steps, graph.stream, min_s=0.3)
    clocks = sampler.stop(t0, time.time())
    us = ms_blk * 1e3 / (steps * copies)
    if not torch.isfinite(y.float()).all():
        raise SystemExit("bench.py: GEMV produced non-finite outputs")
    byt = wbytes + 2 * (k + n) + 2 * m * (k + n)
    peaks = _peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    gbs = byt / us / 1e3
    return {
        "metric": "decode GEMV time (%dx%d, K=%s, m=%d)" % (k, n, K, m), "value": round(us, 2), "unit": "us/launch",
        "n_gpus": 1, "steps": steps, "warmup": max(warmup, 3), "ms_per_step": round(us * copies / 1e3, 4),
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "one GEMV shape, %d distinct weight copies per graph (%.0f MB, larger than L2)" % (copies, copies * wbytes / 1e6),
                   "kernel_form": "tensor memory (tcgen05)" if tmem else "mma.sync",
                   "codebook": "mul1" if mul1 else "default",
                   "input": "RMSNorm(x + res) * w formed in the prologue" if norm else ("silu(gate) * up formed in the prologue" if silu_mul else "plain"),
                   "timing": "median of %d blocks of %d graph replays" % (nblk, steps)},
        "gpu_launches": copies * steps, "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(gbs / peak, 4),
                     "peak_source": "measured (MEASURED_PEAKS.json)" if "hbm_gbs" in peaks else "fallback",
                     "kernel": "exl3_gemv_tc_kernel" if tmem else "exl3_gemv_kernel", "bytes_per_launch": byt, "traffic": None}}


def measure_step_with_neighbours(steps, warmup, n_layers=0):
    """The decode step of the 8B-shaped stack WITH the element-wise kernels that sit between its
    linears (src/ucode/ampstein/graphdec.uc:151-240; attention itself stays outside): residual add +
    RMSNorm in front of q|k|v and gate|up, silu(gate) * up in front of down, final norm, lm_head and
    greedy pick. Three CUDA graphs over the same weights: the linears alone (the headline step), the
    step with its neighbours as separate launches, and with them folded into the linears."""
    import torch
    import ampstein_b200 as amp
    from ampstein_b200.models import DecodeGraph, Multi, Sliced
    S = dict(STACKS["decode"])
    if n_layers:
        S["layers"] = n_layers
    dev = torch.device("cuda", 0)
    layers, head = build_stack(torch, dev, 1234, S)
    H, I, nl = S["hidden"], S["ffn"], len(layers)
    f16 = dict(dtype=torch.float16, device=dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(3)
    norm_w = [(1.0 + 0.05 * torch.randn((2, H), device=dev, generator=gen)).to(torch.float16) for _ in range(nl + 1)]
    q, k_, v = (torch.empty((1, 1, n), **f16) for n in (H, S["kv"], S["kv"]))
    gu_out = torch.empty((2, 1, I), **f16)
    hbuf = [torch.empty((1, 1, H), **f16) for _ in range(2)]            # residual stream, ping-pong
    r = torch.empty((1, 1, H), **f16)
    a = torch.empty((1, I), **f16)
    o_out, d_out = torch.empty((1, H), **f16), torch.zeros((1, H), **f16)
    logits = torch.empty((1, head.out_features), **f16)
    ids, pos = torch.zeros(1, dtype=torch.int64, device=dev), torch.zeros(1, dtype=torch.int64, device=dev)
    log = torch.zeros(1 << 20, dtype=torch.int64, device=dev)
    ws = torch.zeros(4, dtype=torch.int32, device=dev)
    qkv = [Sliced([L["q"], L["k"], L["v"]], [q, k_, v]) for L in layers]
    gu = [Multi([L["gate"], L["up"]], gu_out) for L in layers]
    eps = 1e-5
    h0 = torch.randn((1, 1, H), device=dev, generator=gen).to(torch.float16)

    def linears_only():
        x = hbuf[0]
        for i, L in enumerate(layers):
            qkv[i].run(x)
            L["o"].forward(q[0], o_out)
            gu[i].run(o_out.view(1, 1, H))
            L["down"].forward(gu_out[0], d_out)
            x = d_out.view(1, 1, H)
        head.forward(x[0], logits)

    def unfused():
        cur = 0
        for i, L in enumerate(layers):
            amp.rms_norm_res(hbuf[cur], d_out.view(1, 1, H), norm_w[i][0], eps, hbuf[cur], r)
            qkv[i].run(r)
            L["o"].forward(q[0], o_out)
            amp.rms_norm_res(hbuf[cur], o_out.view(1, 1, H), norm_w[i][1], eps, hbuf[cur], r)
            gu[i].run(r)
            amp.silu_mul(gu_out[0], gu_out[1], a)
            L["down"].forward(a, d_out)
        amp.rms_norm_res(hbuf[cur], d_out.view(1, 1, H), norm_w[nl][0], eps, hbuf[cur], r)
        head.forward(r[0], logits)
        amp.argmax_advance(logits, ids, pos, log, ws)

    def mixed(f_norm, f_act, f_tail):
        def fn():
            cur = 0
            for i, L in enumerate(layers):
                if f_norm:
                    qkv[i].run_norm(hbuf[cur], d_out.view(1, 1, H), norm_w[i][0], eps, hbuf[1 - cur])
                    cur = 1 - cur
                else:
                    amp.rms_norm_res(hbuf[cur], d_out.view(1, 1, H), norm_w[i][0], eps, hbuf[cur], r)
                    qkv[i].run(r)
                L["o"].forward(q[0], o_out)
                if f_norm:
                    gu[i].run_norm(hbuf[cur], o_out.view(1, 1, H), norm_w[i][1], eps, hbuf[1 - cur])
                    cur = 1 - cur
                else:
                    amp.rms_norm_res(hbuf[cur], o_out.view(1, 1, H), norm_w[i][1], eps, hbuf[cur], r)
                    gu[i].run(r)
                if f_act:
                    L["down"].forward_silu_mul(gu_out[0], gu_out[1], d_out)
                else:
                    amp.silu_mul(gu_out[0], gu_out[1], a)
                    L["down"].forward(a, d_out)
            if f_tail:
                amp.lm_head_argmax(hbuf[cur][0], d_out, norm_w[nl][0], eps, hbuf[1 - cur][0], head.trellis, logits, head.suh,
                                   head.svh, ids, pos, log, ws)
            else:
                amp.rms_norm_res(hbuf[cur], d_out.view(1, 1, H), norm_w[nl][0], eps, hbuf[cur], r)
                head.forward(r[0], logits)
                amp.argmax_advance(logits, ids, pos, log, ws)
        return fn

    fused = mixed(True, True, True)
    ssq = torch.zeros((1, H // 128), dtype=torch.float32, device=dev)

    def split_norm():
        # the norm split between producer and consumer: o and down add their output to the residual
        # stream and leave block sums of squares; q|k|v, gate|up and the lm_head scale in their prologue.
        # (The very first norm of the step has no producing linear in front of it.)
        cur = 0
        amp.rms_norm_res(hbuf[cur], d_out.view(1, 1, H), norm_w[0][0], eps, hbuf[cur], r)
        for i, L in enumerate(layers):
            if i == 0:
                qkv[i].run(r)
            else:
                qkv[i].run_normed(hbuf[cur], ssq, norm_w[i][0], eps)
            L["o"].forward_add_res(q[0], hbuf[cur][0], hbuf[1 - cur][0], ssq)
            cur = 1 - cur
            gu[i].run_normed(hbuf[cur], ssq, norm_w[i][1], eps)
            amp.silu_mul(gu_out[0], gu_out[1], a)
            L["down"].forward_add_res(a, hbuf[cur][0], hbuf[1 - cur][0], ssq)
            cur = 1 - cur
        amp.exl3_gemm_normed(hbuf[cur][0], ssq, norm_w[nl][0], eps, head.trellis, logits, head.suh, head.svh)
        amp.argmax_advance(logits, ids, pos, log, ws)

    out = {}
    picks = {}
    forms = [("linears_only", linears_only, 4 * nl + 1), ("neighbours_separate", unfused, 7 * nl + 3),
             ("neighbours_fused", fused, 4 * nl + 1), ("norm_split_producer_consumer", split_norm, 5 * nl + 3)]
    if os.environ.get("AMP_BENCH_STEP_PARTS"):          # which fusion buys what
        forms += [("fused_norms_only", mixed(True, False, False), 5 * nl + 3), ("fused_activation_only", mixed(False, True, False), 6 * nl + 3),
                  ("fused_tail_only", mixed(False, False, True), 7 * nl + 1)]
    for name, fn, launches in forms:
        hbuf[0].copy_(h0)
        d_out.zero_()
        graph = DecodeGraph(fn, warmup=max(warmup, 3))
        hbuf[0].copy_(h0)
        d_out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        picks[name] = int(ids.item())
        if not torch.isfinite(logits.float()).all():
            raise SystemExit("bench.py: non-finite logits in %s" % name)
        ms_blk, nblk, _ = timed_blocks(torch, graph.replay, steps, graph.stream, min_s=0.5)
        out[name] = {"ms_per_step": round(ms_blk / steps, 4), "tok_s": round(steps * 1e3 / ms_blk, 1), "launches_per_step": launches}
        del graph
    return {"metric": "decode step with its element-wise neighbours (8B-shaped stack, batch 1)", "unit": "ms/step",
            "n_gpus": 1, "steps": steps, "warmup": max(warmup, 3), "data": "synthetic", "dtype": "f16",
            "config": {"workload": "%d layers x (norm, q|k|v, o, norm, gate|up, silu*mul, down) + final norm, lm_head, greedy pick; "
                                   "attention not included" % nl,
                       "same_pick": len(set(picks[n] for n in picks if n != "linears_only")) == 1},
            "forms": out}


def measure_issue():
    """Cycles one SM scheduler needs per 8 decoded weights and lane (K = 4 decode mix) with the dot
    product fed by two mma.sync, by one tcgen05.st, not at all, and for the two mma.sync alone."""
    import ctypes
    from ampstein_b200 import _lib
    names = ["decode + 2 mma.sync m16n8k16", "decode + tcgen05.st (8 registers)", "decode + checksum (4 lop3)", "2 mma.sync only"]
    table = {}
    for v, name in enumerate(names):
        row = {}
        for w in (1, 2, 3, 4, 6, 8):
            c = ctypes.c_float(0)
            _lib.call("amp_diag_issue_cycles", v, w, ctypes.byref(c))
            row[str(w)] = round(c.value, 2)
        table[name] = row
    return table


def secondary():
    """The other configurations, measured in the same run so that the record holds them."""
    out = {}
    p = measure_prefill(10, 3)
    out["prefill"] = {k: p[k] for k in ("metric", "value", "unit", "ms_per_step", "roofline", "clocks")}
    st = measure_step_with_neighbours(10, 3)
    out["decode_step_with_neighbours"] = {"metric": st["metric"], "unit": st["unit"], "config": st["config"], "forms": st["forms"]}
    for T in (1, 4, 16):
        r = measure_moe(20, 3, T)
        out["moe_T%d" % T] = {"metric": r["metric"], "value": r["value"], "unit": r["unit"],
                              "distinct_experts": r["config"]["distinct_experts_per_layer"],
                              "roofline": r["roofline"], "clocks": r["clocks"]}
    r = measure_moe_prefill(5, 3)
    out["moe_prefill_T2048"] = {k: r[k] for k in ("metric", "value", "unit", "config", "roofline", "clocks")}
    return out


# ------------------------------------------------------------------------------------------
# CPU legs (the oracle as the timed thing: allowed only here)
# ------------------------------------------------------------------------------------------

HEAD_SLICE = 8192          # lm_head columns in the CPU sample (of 128256)


def cpu_sample_seconds(repeats=1):
    """One layer of the 8B stack (7 linears at 4 bits, 218 M weights) and a 8192-column slice of
    the 6-bit lm_head (33.6 M weights) through the CPU restatement of reconstruct-then-matmul;
    returns (seconds per layer, seconds per head slice, threads)."""
    import numpy as np
    from oracle import exl3_oracle as o
    S = STACKS["decode"]
    rng = np.random.default_rng(0)

    def mat(k, n, K):
        trellis = rng.integers(0, 65536, size=(k // 16, n // 16, 16 * K), dtype=np.uint16)
        suh = rng.choice(np.array([-1.0, 1.0], np.float16), k)
        svh = rng.choice(np.array([-1.0, 1.0], np.float16), n)
        return (rng.standard_normal((1, k)).astype(np.float16), trellis, suh, svh)

    mats = [mat(k, n, S["K"]) for _, k, n in LAYER_8B]
    headm = mat(S["hidden"], HEAD_SLICE, S["K_head"])
    best_l = best_h = None
    for _ in range(repeats):
        t = time.time()
        for x, trellis, suh, svh in mats:
            o.linear(x, trellis, suh, svh, 0)
        dl = time.time() - t
        t = time.time()
        o.linear(*headm, 0)
        dh = time.time() - t
        best_l = dl if best_l is None else min(best_l, dl)
        best_h = dh if best_h is None else min(best_h, dh)
    return best_l, best_h, o.num_threads()


def cpu_step_seconds(sec_layer, sec_head):
    S = STACKS["decode"]
    return sec_layer * S["layers"] + sec_head * (S["vocab"] / HEAD_SLICE)


CPU_SAMPLE = ("one of 32 layers (7 linears at 4 bits, 218M weights) and 8192 of the 128256 lm_head columns at 6 bits, "
              "reconstructed and multiplied; step = 32 x layer + 15.66 x head slice")


def cpu_baseline(repeats=2):
    sl, sh, threads = cpu_sample_seconds(repeats)
    return {"value": round(1.0 / cpu_step_seconds(sl, sh), 5), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": CPU_SAMPLE + ", best of %d" % repeats}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t_all = []
    for _ in range(max(args.warmup, 0)):
        cpu_sample_seconds(1)
    t0 = time.time()
    for _ in range(args.steps):
        t_all.append(cpu_sample_seconds(1))
    sec_step = cpu_step_seconds(sum(t[0] for t in t_all) / len(t_all), sum(t[1] for t in t_all) / len(t_all))
    threads = t_all[0][2]
    val = round(1.0 / sec_step, 5)
    S = STACKS["decode"]
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT,
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(sec_step * 1e3, 1), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "%s decode step, batch 1, EXL3 %d bpw x%d layers + %d bpw lm_head" % (S["name"], S["K"], S["layers"], S["K_head"]),
                   "note": "CPU reconstruct-then-matmul; the reference ships no CPU code for this codebook, "
                           "so the timed code is the CPU restatement (oracle port)"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": "each step = " + CPU_SAMPLE},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": round(time.time() - t0, 1),
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--mode", default="tp", choices=["tp", "replicas"],
                    help="with --gpus N > 1: tensor-parallel decode of one stack (default) or N independent replicas")
    ap.add_argument("--exchange", default="fused", choices=["split", "fused", "separate"],
                    help="tensor-parallel mode: how the all-reduce after o / down runs. fused (default): push and gather in the "
                         "producing GEMV's epilogue; split: the producer only pushes its partial, the consuming GEMV adds the ranks' "
                         "partials up in its prologue (measured slower); separate: a stand-alone all-reduce launch")
    ap.add_argument("--workload", default="decode", choices=["decode", "tp5", "prefill", "moe", "moe-prefill", "gemv", "gemm", "step", "issue"],
                    help="decode (default, the headline step), tp5 (the 64-layer 5-bit tensor-parallel stack), or a secondary "
                         "one-GPU workload: the prefill GEMM / the fused decode MoE / one GEMV shape (--shape) / the decode "
                         "step with its element-wise neighbours, separate and fused (step) / the issue-rate microbenchmark")
    ap.add_argument("--shape", default="4096x229376x4", help="--workload gemv: k x n x K (rows, columns, bits per weight)")
    ap.add_argument("--batch", type=int, default=1, help="tokens per decode step (decode / tp5 workloads), 1..16")
    ap.add_argument("--tokens", type=int, default=0,
                    help="tokens per step of --workload moe (1, 4 or 16; default 1) / per chunk of --workload moe-prefill / rows of --workload gemm (default 2048)")
    ap.add_argument("--tmem-gemv", action="store_true",
                    help="A/B: run the decode GEMVs on the tensor-memory (tcgen05) kernel instead of the mma.sync kernel")
    ap.add_argument("--mul1", action="store_true", help="--workload gemv: the mul1 codebook (one row then takes the int8-activation form)")
    ap.add_argument("--silu-mul", action="store_true", help="--workload gemv: the down projection with silu(gate) * up folded into its prologue")
    ap.add_argument("--norm", action="store_true", help="--workload gemv: the linear with the residual add + RMSNorm folded into its prologue")
    ap.add_argument("--no-int8", action="store_true", help="--workload gemv --mul1: keep the fp16 kernel (A/B)")
    ap.add_argument("--int8-residual", action="store_true",
                    help="--workload gemv --mul1: the int8 form with the error-feedback pass (the reference's EXL3_INT8_GEMV=1)")
    ap.add_argument("--separate", action="store_true",
                    help="--workload prefill: seven separate GEMM calls instead of the q|k|v and gate|up bundles")
    ap.add_argument("--tile-sub", type=int, default=0, choices=[0, 1, 2, 4],
                    help="--workload moe-prefill: rows per GEMM tile / 128 (A/B; default 0 = chosen per call)")
    ap.add_argument("--no-secondary", action="store_true",
                    help="decode workload on one GPU: skip the per-shape and secondary measurements (profiler captures)")
    ap.add_argument("--layers", type=int, default=0,
                    help="layers of the stack (default: the full stack; fewer only for a small profiler capture)")
    args = ap.parse_args()
    if not 1 <= args.batch <= 16:
        raise SystemExit("bench.py: --batch must be 1..16")
    if args.tmem_gemv and args.impl != "reference":
        from ampstein_b200 import _lib
        _lib.lib().amp_exl3_set_gemv_tc(1)
    if args.impl == "reference":
        if args.steps > 5:
            args.steps = 5                 # each step is seconds of CPU work
        args.warmup = min(args.warmup, 1)
        run_reference(args)
        return
    if args.workload == "moe" and (args.tokens or 1) not in (1, 4, 16):
        raise SystemExit("bench.py: --workload moe takes --tokens 1, 4 or 16")
    if args.workload in ("prefill", "moe", "moe-prefill", "gemv", "gemm", "step", "issue"):
        import torch
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device (the path has no CPU fallback)")
        if args.workload == "prefill":
            print(json.dumps(measure_prefill(args.steps, args.warmup, not args.separate)), flush=True)
        elif args.workload == "moe":
            print(json.dumps(measure_moe(args.steps, args.warmup, args.tokens or 1)), flush=True)
        elif args.workload == "moe-prefill":
            if args.tile_sub:
                from ampstein_b200 import _lib
                _lib.lib().amp_exl3_set_moe_sorted_tile(args.tile_sub)
            print(json.dumps(measure_moe_prefill(args.steps, args.warmup, args.tokens or 2048)), flush=True)
        elif args.workload == "step":
            print(json.dumps(measure_step_with_neighbours(args.steps, args.warmup, args.layers)), flush=True)
        elif args.workload == "gemm":
            try:
                shape = tuple(int(v) for v in args.shape.lower().split("x"))
                assert len(shape) == 3 and shape[0] % 128 == 0 and shape[1] % 128 == 0 and 1 <= shape[2] <= 8
            except (ValueError, AssertionError):
                raise SystemExit("bench.py: --shape must be KxNxBITS with k, n multiples of 128 and 1..8 bits")
            print(json.dumps(measure_gemm(args.steps, args.warmup, shape, args.tokens or 2048)), flush=True)
        elif args.workload == "gemv":
            try:
                parts = args.shape.lower().split("x")
                bits = float(parts[2])
                shape = (int(parts[0]), int(parts[1]), int(bits) if bits == int(bits) else bits)
                assert len(parts) == 3 and shape[0] % 128 == 0 and shape[1] % 128 == 0 and (bits in (1.5, 2.5, 3.5) or (bits == int(bits) and 1 <= bits <= 8))
                assert bits == int(bits) or args.mul1
            except (ValueError, AssertionError, IndexError):
                raise SystemExit("bench.py: --shape must be KxNxBITS with k, n multiples of 128 and 1..8 bits (1.5 / 2.5 / 3.5 with --mul1)")
            if args.no_int8 or args.int8_residual:
                from ampstein_b200 import _lib
                _lib.lib().amp_exl3_set_int8_gemv(1 if args.int8_residual else 0, 0)
            print(json.dumps(measure_gemv(args.steps, args.warmup, shape, args.batch, args.tmem_gemv, args.mul1, args.silu_mul, args.norm)), flush=True)
        else:
            print(json.dumps({"metric": "scheduler cycles per 8 decoded weights and lane (K=4 mix)", "unit": "cycles",
                              "by_warps_per_scheduler": measure_issue()}), flush=True)
        return
    S = dict(STACKS[args.workload])
    if args.layers:
        S["layers"] = args.layers
    run_decode(args, S)


if __name__ == "__main__":
    main()
