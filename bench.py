#!/usr/bin/env python
"""Benchmark of the EXL3 quantized-linear hot path on B200.

Workload (N = 1): the Llama-3-8B-shaped decode step at batch 1 -- 32 layers of q/k/v/o/gate/up/
down EXL3 linears at 4 bits per weight plus a 6-bit lm_head, chained through their activations
and replayed as ONE CUDA graph per token. Weights are seeded synthetic trellis words (every bit
pattern is a valid stream); svh carries random signs scaled so that chained activations stay
O(1) in fp16 without extra kernels. A step streams 3.89 GB of packed weights, far more than the
126 MB L2, so no cache flush is needed between steps.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--mode tp|replicas]
    python bench.py --workload prefill | --workload moe [--tokens 1|4|16]      (secondary, one GPU)

With N > 1 GPUs (one process per GPU under torchrun) the same stack is decoded tensor-parallel, as
the reference shards it: q|k|v and gate|up column-parallel, o and down row-parallel, each followed
by the fp16 all-reduce of the hidden state over NVLink (this library's kernel, inside the graph);
lm_head is split by vocabulary. All ranks decode the same token, so the work is fixed as N grows
(strong scaling). `--mode replicas` runs N independent copies of the 1-GPU step instead.

One JSON line on stdout (rank 0). `--impl reference` times the CPU restatement of the
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

HIDDEN, KV, FFN, VOCAB, LAYERS = 4096, 1024, 14336, 128256, 32
K_LAYER, K_HEAD = 4, 6
# (name, in, out) of one layer, in launch order
LAYER_LINEARS = [("q", HIDDEN, HIDDEN), ("k", HIDDEN, KV), ("v", HIDDEN, KV), ("o", HIDDEN, HIDDEN),
                 ("gate", HIDDEN, FFN), ("up", HIDDEN, FFN), ("down", FFN, HIDDEN)]


def algorithmic_bytes(m=1):
    """Bytes a step must move: packed weights + suh/svh + activations in and out (no scratch)."""
    total = 0
    for _, k, n in LAYER_LINEARS:
        total += k * n * K_LAYER // 8 + 2 * (k + n) + 2 * m * (k + n)
    total *= LAYERS
    total += HIDDEN * VOCAB * K_HEAD // 8 + 2 * (HIDDEN + VOCAB) + 2 * m * (HIDDEN + VOCAB)
    return total


def total_weights():
    return LAYERS * sum(k * n for _, k, n in LAYER_LINEARS) + HIDDEN * VOCAB


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


# ------------------------------------------------------------------------------------------
# the GPU arm
# ------------------------------------------------------------------------------------------

def tp_shapes(rank, world):
    """(name, in, out, in of the unsharded matrix) of one layer and the lm_head for a rank of a
    tensor-parallel group: column-parallel q/k/v/gate/up, row-parallel o/down (reference:
    src/ucode/ampstein/models.uc:527-562), lm_head by blocks of 128 vocabulary entries."""
    layer = []
    for name, k, n in LAYER_LINEARS:
        if name in ("o", "down"):
            layer.append((name, k // world, n, k))
        else:
            layer.append((name, k, n // world, k))
    blocks = VOCAB // 128
    b0, b1 = blocks * rank // world, blocks * (rank + 1) // world
    return layer, (HIDDEN, (b1 - b0) * 128)


def build_stack(torch, device, seed, shapes=None):
    """Distinct synthetic tensors for every linear of the stack (3.9 GB in all)."""
    from ampstein_b200.models import LinearEXL3
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    layer_shapes = [(name, k, n, k) for name, k, n in LAYER_LINEARS] if shapes is None else shapes[0]
    head_shape = (HIDDEN, VOCAB) if shapes is None else shapes[1]

    def make(k, n, K, k_full=None):
        trellis = torch.randint(-32768, 32768, (k // 16, n // 16, 16 * K), dtype=torch.int16,
                                device=device, generator=g)
        sgn = lambda c: (torch.randint(0, 2, (c,), device=device, generator=g).to(torch.float16) * 2 - 1)
        suh = sgn(k)
        # decoded weights have std 1.2437: keep chained activations at unit scale
        svh = sgn(n) * (1.0 / (1.2437 * math.sqrt(k_full or k)))
        return LinearEXL3(trellis, suh, svh.to(torch.float16))

    layers = [{name: make(k, n, K_LAYER, kf) for name, k, n, kf in layer_shapes} for _ in range(LAYERS)]
    head = make(head_shape[0], head_shape[1], K_HEAD)
    return layers, head


def run_gpu(args):
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

    m = 1
    tp = world if (world > 1 and args.mode == "tp") else 1
    if tp > 1 and ((HIDDEN // tp) % 128 or (KV // tp) % 128 or (FFN // tp) % 128):
        raise SystemExit("bench.py: the stack does not shard %d ways in multiples of 128" % tp)
    shapes = tp_shapes(rank, tp) if tp > 1 else None
    layers, head = build_stack(torch, device, seed=1234 + rank, shapes=shapes)
    vocab_local = head.out_features
    f16 = dict(dtype=torch.float16, device=device)
    h_in = torch.empty((1, m, HIDDEN), **f16)
    bufs = {"q": torch.empty((1, m, HIDDEN // tp), **f16), "k": torch.empty((1, m, KV // tp), **f16),
            "v": torch.empty((1, m, KV // tp), **f16), "a": torch.empty((1, m, HIDDEN), **f16),
            "gu": torch.empty((2, m, FFN // tp), **f16), "h": torch.empty((1, m, HIDDEN), **f16),
            "logits": torch.empty((m, vocab_local), **f16)}
    comm = None
    if tp > 1:
        # partial sums of the row-parallel o / down, all-reduced over NVLink inside the graph
        from ampstein_b200.comm import P2PComm
        bufs["a_part"] = torch.empty((1, m, HIDDEN), **f16)
        bufs["h_part"] = torch.empty((1, m, HIDDEN), **f16)
        comm = P2PComm.from_process_group(cap=m * HIDDEN)
    # the reference's decode step runs q|k|v as one sliced bundle and gate|up as one stacked bundle
    # (src/ucode/ampstein/graphdec.uc:163-210): four launches per layer
    qkv = [Sliced([L["q"], L["k"], L["v"]], [bufs["q"], bufs["k"], bufs["v"]]) for L in layers]
    gu = [Multi([L["gate"], L["up"]], bufs["gu"]) for L in layers]
    launches = [0]

    def step(stub=False):
        # stub: the row-parallel linears without their all-reduce (to price the exchange)
        x = h_in
        n = 0
        for i, L in enumerate(layers):
            qkv[i].run(x)
            if comm is None:
                L["o"].forward(bufs["q"][0], bufs["a"][0])    # attention itself is outside the path
                gu[i].run(bufs["a"])
                L["down"].forward(bufs["gu"][0], bufs["h"][0])
                n += 4
            else:
                if stub:
                    L["o"].forward(bufs["q"][0], bufs["a"][0])
                elif args.unfused:
                    L["o"].forward(bufs["q"][0], bufs["a_part"][0])
                    comm.allreduce(bufs["a_part"], out=bufs["a"])
                else:
                    comm.linear_allreduce(L["o"], bufs["q"][0], bufs["a"][0])
                gu[i].run(bufs["a"])
                if stub:
                    L["down"].forward(bufs["gu"][0], bufs["h"][0])
                elif args.unfused:
                    L["down"].forward(bufs["gu"][0], bufs["h_part"][0])
                    comm.allreduce(bufs["h_part"], out=bufs["h"])
                else:
                    comm.linear_allreduce(L["down"], bufs["gu"][0], bufs["h"][0])
                n += 6 if args.unfused else 4
            x = bufs["h"]
        head.forward(x[0], bufs["logits"])
        if not stub:
            launches[0] = n + 1

    host_x = torch.randn((m, HIDDEN), dtype=torch.float16).pin_memory()
    host_logits = torch.empty((m, vocab_local), dtype=torch.float16).pin_memory()
    h_in.copy_(host_x.view(1, m, HIDDEN))
    graph = DecodeGraph(step, warmup=2)
    stream = graph.stream

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def resident_step():
        graph.replay()

    def e2e_step():
        h_in.copy_(host_x.view(1, m, HIDDEN), non_blocking=True)
        graph.replay()
        host_logits.copy_(bufs["logits"], non_blocking=True)

    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            e2e_step()
    sampler = ClockSampler(local) if rank == 0 else None
    t0 = time.time()
    ms = timed(resident_step, args.steps)
    ms_e2e = timed(e2e_step, args.steps)
    t1 = time.time()
    ms_stub = None
    if comm is not None:
        # the same graph without the exchange: the difference is what the all-reduces cost
        # (values diverge between ranks here; only the time is used)
        stub_graph = DecodeGraph(lambda: step(stub=True), warmup=1, stream=stream)
        ms_stub = timed(stub_graph.replay, args.steps)
    clocks = sampler.stop(t0, t1) if sampler else None

    logits = host_logits.float()
    if not torch.isfinite(logits).all() or float(logits.abs().max()) == 0.0:
        raise SystemExit("bench.py: step produced non-finite or all-zero logits")

    comm_status = 0
    if comm is not None:
        comm_status = comm.status()
        t = torch.tensor([comm_status], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        comm_status = int(t.item())
        if comm_status:
            raise SystemExit("bench.py: an all-reduce gave up waiting for a peer (status %d)" % comm_status)
    if rank != 0:
        return
    ms_step = ms / args.steps
    # tensor parallel: every rank decodes the same token; replicas: one token per rank
    streams = 1 if tp > 1 else world
    tok_s = streams * m * 1000.0 / ms_step
    tok_s_e2e = streams * m * 1000.0 / (ms_e2e / args.steps)
    gemv_launches = 4 * LAYERS + 1
    # per GPU: a rank streams 1/tp of the weights (+ the unsharded vectors)
    bytes_step = algorithmic_bytes(m) if tp == 1 else algorithmic_bytes(m) // tp
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = bytes_step / (ms_step * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": round(tok_s, 2), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "strong" if tp > 1 else "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": "llama3-8b-shaped decode step, batch 1, EXL3 4.0 bpw x%d layers + 6 bpw lm_head, one CUDA graph" % LAYERS,
                   "l2": "inputs larger than L2 (%.2f GB of weights streamed per step and GPU)" % (bytes_step / 1e9),
                   "parallelism": ("tp%d: column-parallel q|k|v, gate|up; row-parallel o, down with the fp16 all-reduce (%d per step) over NVLink %s; lm_head by vocabulary"
                                   % (tp, 2 * LAYERS, "as separate launches" if args.unfused else "fused into the GEMV epilogue")) if tp > 1 else ("replicas x%d" % world)},
        "e2e": {"value": round(tok_s_e2e, 2), "unit": UNIT,
                "h2d_bytes_per_step": host_x.numel() * 2, "d2h_bytes_per_step": host_logits.numel() * 2},
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
        line["allreduce"] = {"per_step": 2 * LAYERS, "bytes": m * HIDDEN * 2,
                             "ms_per_step_without": round(ms_stub / args.steps, 4),
                             "share_of_step": round(max(0.0, 1.0 - ms_stub / ms), 4),
                             "us_each": round(max(0.0, ms - ms_stub) / args.steps / (2 * LAYERS) * 1e3, 2)}
    if world == 1:
        line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# secondary workloads (one GPU): the prefill GEMM and the fused decode MoE
# ------------------------------------------------------------------------------------------

def _peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        return {}


def run_prefill(args):
    """One decoder layer's seven linears at M = 2048 tokens, bf16 activations, mixed bit widths
    (attention K=5, gate/up K=3, down K=4): the tensor-core (tcgen05) trellis-decode GEMM,
    including the input rotation kernel. One step = the seven GEMMs."""
    import torch
    import ampstein_b200 as amp
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the path has no CPU fallback)")
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    M = 2048
    bits = {"q": 5, "k": 5, "v": 5, "o": 5, "gate": 3, "up": 3, "down": 4}
    ops = []
    for name, k, n in LAYER_LINEARS:
        K = bits[name]
        t = torch.randint(-32768, 32768, (k // 16, n // 16, 16 * K), dtype=torch.int16, device=dev, generator=g)
        sgn = lambda c: (torch.randint(0, 2, (c,), device=dev, generator=g).to(torch.float16) * 2 - 1)
        svh = (sgn(n) * (1.0 / (1.2437 * math.sqrt(k)))).to(torch.float16)
        x = torch.randn((M, k), device=dev, generator=g).to(torch.bfloat16)
        ops.append((x, t, torch.empty((M, n), dtype=torch.float16, device=dev), sgn(k), svh))
    flops = sum(2.0 * M * k * n for _, k, n in LAYER_LINEARS)

    def step():
        for x, t, y, suh, svh in ops:
            amp.exl3_gemm(x, t, y, suh, svh)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    t0 = time.time()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop(t0, time.time())
    ms = e0.elapsed_time(e1) / args.steps
    if not all(torch.isfinite(o[2].float()).all() for o in ops):
        raise SystemExit("bench.py: prefill produced non-finite outputs")
    peaks = _peaks()
    peak = float(peaks.get("bf16_tflops", 1590.0))
    tf = flops / ms / 1e9
    print(json.dumps({
        "metric": "prefill TFLOP/s (one 8B-shaped layer, M=2048, EXL3 K=5/3/4)", "value": round(tf, 1), "unit": "TFLOP/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "prefill: 7 linears of one llama3-8b-shaped layer, M=2048 bf16 tokens, K=5 attention / 3 gate,up / 4 down",
                   "l2": "operands of a step: 0.23 GB (weights read once per GEMM)"},
        "gpu_launches": 14 * args.steps, "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": round(tf, 1), "peak": peak, "unit": "TFLOP/s", "frac": round(tf / peak, 4),
                     "peak_source": "measured burst (MEASURED_PEAKS.json)" if "bf16_tflops" in peaks else "fallback",
                     "kernel": "exl3_gemm_tc2_kernel", "traffic": None}}), flush=True)


def run_moe(args):
    """Fused decode MoE: 128 experts 2048 -> 768 -> 2048 at K=3, top-8 routing from fp32 router
    logits ~ N(0,1), T tokens per step (--tokens 1, 4 or 16). Eight different routings are
    captured in one CUDA graph so that successive layers hit different experts; one step = one
    MoE layer."""
    import numpy as np
    import torch
    import ampstein_b200 as amp
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the path has no CPU fallback)")
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(11)
    E, Hi, I, Ho, K, topk, T = 128, 2048, 768, 2048, 3, 8, args.tokens
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
               ctr=torch.zeros(amp.moe_coop_ctr_len(slots), dtype=torch.int32, device=dev),
               out=torch.zeros(T, Hi, dtype=torch.float32, device=dev), Hi=Hi, Kg=K, Ku=K, Kd=K, act=0, act_limit=0.0)
    sets = []
    for _ in range(8):
        w, sel = torch.topk(torch.randn(T, E, device=dev, generator=g), topk, dim=1)
        sets.append((torch.randn(T, Hi, device=dev, generator=g).to(torch.float16), sel.contiguous(),
                     torch.softmax(w, 1).to(torch.float16).contiguous()))
    distinct = float(np.mean([len(torch.unique(s[1])) for s in sets]))
    for x, sel, rw in sets:
        amp.moe_coop(x, sel, rw, cfg)
    torch.cuda.synchronize()
    gr, st = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(st), torch.cuda.graph(gr, stream=st):
        for x, sel, rw in sets:
            amp.moe_coop(x, sel, rw, cfg)
    for _ in range(max(args.warmup, 3)):
        gr.replay()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    t0 = time.time()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        gr.replay()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop(t0, time.time())
    us = e0.elapsed_time(e1) * 1e3 / (args.steps * len(sets))
    if not torch.isfinite(cfg["out"]).all():
        raise SystemExit("bench.py: MoE produced non-finite outputs")
    byt = distinct * 3 * Hi * I * K // 8
    peaks = _peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    gbs = byt / us / 1e3
    print(json.dumps({
        "metric": "fused decode MoE layer time (128 experts, top-8, K=3)", "value": round(us, 2), "unit": "us/layer",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(us * len(sets) / 1e3, 4),
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "moe decode: 128 experts 2048->768->2048 K=3, top-8, %d token(s), 8 routings per graph" % T,
                   "distinct_experts_per_layer": round(distinct, 1),
                   "l2": "expert weights in total 226 MB (larger than L2); each layer touches %.1f MB" % (byt / 1e6)},
        "gpu_launches": 4 * len(sets) * args.steps, "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(gbs / peak, 4),
                     "peak_source": "measured (MEASURED_PEAKS.json)" if "hbm_gbs" in peaks else "fallback",
                     "kernel": "exl3_gemv_kernel (grouped modes)", "bytes_per_launch": int(byt) // 2, "traffic": None}}), flush=True)


# ------------------------------------------------------------------------------------------
# CPU legs (the oracle as the timed thing: allowed only here)
# ------------------------------------------------------------------------------------------

def cpu_sample_seconds(repeats=1):
    """One layer of the stack (7 linears, 218 M weights) through the CPU restatement of
    reconstruct-then-matmul; returns (seconds per layer, threads)."""
    import numpy as np
    from oracle import exl3_oracle as o
    rng = np.random.default_rng(0)
    mats = []
    for _, k, n in LAYER_LINEARS:
        trellis = rng.integers(0, 65536, size=(k // 16, n // 16, 16 * K_LAYER), dtype=np.uint16)
        suh = rng.choice(np.array([-1.0, 1.0], np.float16), k)
        svh = rng.choice(np.array([-1.0, 1.0], np.float16), n)
        x = rng.standard_normal((1, k)).astype(np.float16)
        mats.append((x, trellis, suh, svh))
    best = None
    for _ in range(repeats):
        t = time.time()
        for x, trellis, suh, svh in mats:
            o.linear(x, trellis, suh, svh, 0)
        dt = time.time() - t
        best = dt if best is None else min(best, dt)
    return best, o.num_threads()


def cpu_baseline(repeats=2):
    sec_layer, threads = cpu_sample_seconds(repeats)
    layer_weights = sum(k * n for _, k, n in LAYER_LINEARS)
    sec_step = sec_layer * total_weights() / layer_weights
    return {"value": round(1.0 / sec_step, 5), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": "one of 32 layers (7 linears, 218M weights) reconstructed and multiplied, "
                      "best of %d, scaled by weight count to the full step" % repeats}


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
    sec_layer = sum(t for t, _ in t_all) / len(t_all)
    threads = t_all[0][1]
    layer_weights = sum(k * n for _, k, n in LAYER_LINEARS)
    sec_step = sec_layer * total_weights() / layer_weights
    val = round(1.0 / sec_step, 5)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT,
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(sec_step * 1e3, 1), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "llama3-8b-shaped decode step, batch 1, EXL3 4.0 bpw x%d layers + 6 bpw lm_head" % LAYERS,
                   "note": "CPU reconstruct-then-matmul; the reference ships no CPU code for this codebook, "
                           "so the timed code is the CPU restatement (oracle port)"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "each step = one of 32 layers (7 linears, 218M weights), scaled by weight count"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": round(time.time() - t0, 1),
    }
    print(json.dumps(line), flush=True)


def main():
    global LAYERS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--mode", default="tp", choices=["tp", "replicas"],
                    help="with --gpus N > 1: tensor-parallel decode of one stack (default) or N independent replicas")
    ap.add_argument("--unfused", action="store_true",
                    help="tensor-parallel mode: separate all-reduce launches instead of the GEMV's fused exchange")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "moe"],
                    help="decode (default, the headline step) or a secondary one-GPU workload: the prefill GEMM / the fused decode MoE")
    ap.add_argument("--tokens", type=int, default=1, choices=[1, 4, 16], help="tokens per step of --workload moe")
    ap.add_argument("--tmem-gemv", action="store_true",
                    help="A/B: run the decode GEMVs on the tensor-memory (tcgen05) kernel instead of the mma.sync kernel")
    ap.add_argument("--layers", type=int, default=LAYERS,
                    help="layers of the stack (default: the full 32; fewer only for a small profiler capture)")
    args = ap.parse_args()
    LAYERS = args.layers
    if args.tmem_gemv and args.impl != "reference":
        from ampstein_b200 import _lib
        _lib.lib().amp_exl3_set_gemv_tc(1)
    if args.impl == "reference":
        if args.steps > 5:
            args.steps = 5                 # each step is seconds of CPU work
        args.warmup = min(args.warmup, 1)
        run_reference(args)
    elif args.workload == "prefill":
        run_prefill(args)
    elif args.workload == "moe":
        run_moe(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
