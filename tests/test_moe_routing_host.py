"""Host side of the token-sorted MoE (no GPU): the routing sort that feeds moe_fused, its expert-parallel
partition over two ranks (gloo), and the argument errors of the wrappers, which must refuse host
tensors instead of computing anything on the CPU."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.multiprocessing as mp  # noqa: E402


def _routing(T, K, E, seed):
    g = torch.Generator().manual_seed(seed)
    sel = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int64)
    rw = torch.rand((T, K), generator=g)
    return sel, rw


def test_sort_routing_is_a_stable_sort_by_local_expert():
    from ampstein_b200 import moe_sort_routing
    T, K, E, e0 = 50, 4, 6, 3
    sel, rw = _routing(T, K, 12, 1)
    count, tok, wts, fe, inv, start = moe_sort_routing(sel, rw, E, e0, with_inverse=True)
    loc = sel.reshape(-1).numpy() - e0
    want_fe = np.where((loc >= 0) & (loc < E), loc, E)
    order = np.argsort(want_fe, kind="stable")
    assert np.array_equal(fe.numpy(), want_fe)
    assert np.array_equal(tok.numpy(), order // K)
    assert np.array_equal(wts.numpy().view(np.uint16), rw.reshape(-1).numpy()[order].astype(np.float16).view(np.uint16))
    assert np.array_equal(count.numpy(), np.bincount(want_fe, minlength=E + 1))
    assert np.array_equal(start.numpy(), np.cumsum(count.numpy()) - count.numpy())
    assert np.array_equal(inv.numpy()[order], np.arange(T * K))
    assert count.sum().item() == T * K and count.dtype == torch.int64 and wts.dtype == torch.float16


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    import torch.distributed as dist
    from ampstein_b200 import moe_sort_routing
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        T, K, E = 64, 4, 16
        sel, rw = _routing(T, K, E, 7)                     # every rank sees the same router output
        per = E // world
        count, tok, wts = moe_sort_routing(sel, rw, per, rank * per)
        mine = torch.zeros(E + 1, dtype=torch.int64)
        mine[rank * per:(rank + 1) * per] = count[:per]
        mine[E] = count[per]                               # picks that belong to another rank
        dist.all_reduce(mine)
        # the rows this rank would process, as (token, global expert) pairs
        owned = int(count[:per].sum())
        fe = sel.reshape(-1) - rank * per
        pairs = sorted((int(t), int(e)) for t, e in zip(torch.arange(T * K) // K, sel.reshape(-1)) if 0 <= int(e) - rank * per < per)
        got = sorted((int(t), -1) for t in tok[:owned])
        q.put((rank, mine.tolist(), owned, [p[0] for p in pairs] == [g[0] for g in got], int((fe < 0).sum() + (fe >= per).sum())))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_partition_gloo_world2():
    """Two ranks, each owning half of the experts: the shards' counts tile the global histogram, every
    pick is processed by exactly one rank, and the foreign picks sit in each rank's sentinel bin."""
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
    T, K, E = 64, 4, 16
    sel, _ = _routing(T, K, E, 7)
    hist = np.bincount(sel.reshape(-1).numpy(), minlength=E)
    total_owned = 0
    for rank, summed, owned, tokens_match, foreign in res:
        assert summed[:E] == hist.tolist()                 # the shards tile the global histogram
        assert summed[E] == T * K                          # every pick is foreign to exactly one of two ranks
        assert tokens_match and owned + foreign == T * K
        total_owned += owned
    assert total_owned == T * K


def test_wrappers_refuse_host_tensors_and_bad_shapes():
    import ampstein_b200 as amp
    y = torch.zeros((4, 128), dtype=torch.float16)
    out = torch.zeros((4, 128), dtype=torch.float32)
    cnt = torch.zeros(3, dtype=torch.int64)
    tok = torch.zeros(4, dtype=torch.int64)
    w = torch.zeros(4, dtype=torch.float16)
    table = torch.zeros(2, dtype=torch.int64)
    cfg = {n: table for n in ("g_trellis", "g_suh", "g_svh", "u_trellis", "u_suh", "u_svh", "d_trellis", "d_suh", "d_svh")}
    cfg.update(I=128, Kg=3, Ku=3, Kd=3)
    with pytest.raises(RuntimeError):
        amp.moe_fused(y, out, cnt, tok, w, cfg)            # no CPU path
    with pytest.raises(TypeError):
        amp.moe_fused(y, out, cnt, tok, w, [])             # cfg must be an object
    bad = dict(cfg)
    bad["u_suh"] = table.to(torch.int32)
    with pytest.raises(TypeError):
        amp.moe_fused(y, out, cnt, tok, w, bad)
    with pytest.raises(RuntimeError):
        amp.moe_prep(torch.zeros((4, 2), dtype=torch.int64), torch.zeros((4, 2)), 8)
    with pytest.raises(RuntimeError):
        amp.moe_gather(out, out, tok, tok, cnt, cnt, cnt, w)
    with pytest.raises(RuntimeError):
        amp.exl3_shard_cols(torch.zeros((8, 8, 64), dtype=torch.int16), torch.zeros(128, dtype=torch.float16), [(0, 128)])
