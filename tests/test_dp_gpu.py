"""Two-GPU data-parallel step: bucketed NCCL all-reduce overlapped with the backward pass.

The reduced gradient of two ranks (one micro-batch each) must equal the gradient one rank
accumulates over both micro-batches (a sum: the w-rank result equals the 1-rank result with accum = w).
Skipped when fewer than two GPUs are visible.
"""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

CFG = dict(vocab=1024, hidden=256, heads=4, kv=2, ffn=512, layers=3)
B, S = 2, 256


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _batch(rank):
    rng = np.random.default_rng(7 + rank)
    return rng.integers(0, CFG["vocab"], (B, S)).astype(np.int32), rng.integers(0, CFG["vocab"], B * S)


def _build(dev):
    from eisen_b200.graph import BF16_MIXED, Graph, TransformerLM

    stream = torch.cuda.Stream(device=dev)
    g = Graph(BF16_MIXED, stream.cuda_stream)
    lm = TransformerLM(g, CFG["vocab"], CFG["hidden"], CFG["heads"], CFG["kv"], CFG["ffn"], CFG["layers"], False)
    g.mark_params()
    rng = np.random.default_rng(0)
    for p in lm.params():
        shp = g.shape(p)
        if len(shp) == 2:
            g.load_tensor_data(p, (rng.standard_normal(int(np.prod(shp))) * 0.02).astype(np.float32))
    return g, lm, stream


def _worker(rank, world, port, out):
    import torch.distributed as dist

    from eisen_b200 import dp as edp
    from eisen_b200.graph import AdamW

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    g, lm, stream = _build(dev)
    opt = AdamW(g, lm.params(), 3e-4)
    opt.zero_grad()
    _, _, gptr, n = g.param_arena()
    flat = edp.device_view(gptr, n, dev)
    offs, total = edp.param_offsets([g.shape(p) for p in sorted(lm.params())])
    assert total == n
    red = edp.BucketedAllReduce(flat, edp.plan_buckets(offs, CFG["layers"], total, min_bucket_elems=1 << 18))
    ids, tg = _batch(rank)
    x = g.alloc_ids([B, S], ids)
    lm.train_micro_step(x, tg.tolist(), checkpoint=True, after_block=lambda l: red.on_block_done(l, stream))
    red.finish(stream)
    g.clear_activations()
    g.synchronize()
    reduced = flat.detach().cpu().numpy().copy()
    opt.step_fused(1.0, red.grad_scale())
    g.synchronize()
    if rank == 0:
        out.put(reduced)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_step_equals_accumulated_single_gpu():
    import torch.multiprocessing as mp

    from eisen_b200 import dp as edp
    from eisen_b200.graph import AdamW

    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    reduced = out.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    g, lm, stream = _build(dev)
    opt = AdamW(g, lm.params(), 3e-4)
    opt.zero_grad()
    for r in range(2):
        ids, tg = _batch(r)
        x = g.alloc_ids([B, S], ids)
        lm.train_micro_step(x, tg.tolist(), checkpoint=True)
        g.clear_activations()
    g.synchronize()
    _, _, gptr, n = g.param_arena()
    ref = edp.device_view(gptr, n, dev).cpu().numpy()
    err = np.linalg.norm(reduced - ref) / np.linalg.norm(ref)
    assert err < 1e-4, err


# ------------------------------------------------------------------ the eisen_dp_* C ABI over NCCL
def test_dp_abi_single_rank_collectives():
    """One rank, one GPU: every eisen_dp_* entry point runs through NCCL (bound at run time) and
    leaves the data as a one-rank collective must; wait returns within its deadline."""
    import ctypes as C

    import eisen_b200 as eb

    L = eb.lib()
    assert L.eisen_dp_available() == 1
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    s = torch.cuda.Stream(device=dev)
    uid = (C.c_char * 128)()
    eb.call("eisen_dp_unique_id", uid)
    h = C.c_void_p()
    eb.call("eisen_dp_init", 0, 1, uid, C.byref(h))
    try:
        x = torch.arange(4096, dtype=torch.float32, device=dev)
        y = torch.zeros(4096, dtype=torch.float32, device=dev)
        hb = torch.arange(4096, dtype=torch.float32, device=dev).to(torch.bfloat16)
        d = torch.full((1,), 2.5, dtype=torch.float64, device=dev)
        torch.cuda.synchronize()
        eb.call("eisen_dp_allreduce_bucket", h, x.data_ptr(), 4096, eb.F32, s.cuda_stream)
        eb.call("eisen_dp_reduce_scatter", h, x.data_ptr(), y.data_ptr(), 4096, eb.F32, s.cuda_stream)
        eb.call("eisen_dp_all_gather", h, hb.data_ptr(), hb.data_ptr(), 4096, eb.BF16, s.cuda_stream)
        eb.call("eisen_dp_allreduce_bucket", h, d.data_ptr(), 1, 3, s.cuda_stream)
        eb.call("eisen_dp_group_begin")
        eb.call("eisen_dp_broadcast", h, x.data_ptr(), 16, eb.F32, 0, s.cuda_stream)
        eb.call("eisen_dp_broadcast", h, x.data_ptr() + 64, 16, eb.F32, 0, s.cuda_stream)
        eb.call("eisen_dp_group_end")
        eb.call("eisen_dp_wait", h, s.cuda_stream, 20000)
        eb.call("eisen_dp_poll_error", h)
        n = C.c_longlong()
        r, w = C.c_int(), C.c_int()
        eb.call("eisen_dp_rank_world", h, C.byref(r), C.byref(w), C.byref(n))
        assert (r.value, w.value, n.value) == (0, 1, 6)
        assert torch.equal(x.cpu(), torch.arange(4096, dtype=torch.float32)) and torch.equal(y.cpu(), x.cpu())
        assert d.item() == 2.5
        assert L.eisen_dp_broadcast(h, x.data_ptr(), 16, eb.F32, 3, s.cuda_stream) == 1  # root out of range
        assert L.eisen_dp_allreduce_bucket(h, x.data_ptr(), 16, 2, s.cuda_stream) == 1  # not a collective dtype
        # after an abort every call on the handle fails with EISEN_ERR_COMM (6) instead of hanging
        eb.call("eisen_dp_abort", h)
        assert L.eisen_dp_allreduce_bucket(h, x.data_ptr(), 16, eb.F32, s.cuda_stream) == 6
    finally:
        L.eisen_dp_destroy(h)


def _zero_worker(rank, world, port, out):
    import torch.distributed as dist

    from eisen_b200 import dp as edp
    from eisen_b200.graph import AdamW, ShardedAdamW

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)  # control plane only: carries the NCCL id

    def exchange_id(raw):
        box = [raw]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    comm = torch.cuda.Stream(device=dev)
    backend = edp.NcclAbiBackend(rank, world, comm, exchange_id)
    # two identical models: A takes the replicated step, B the sharded one, on the same local gradients
    ga, lma, sa = _build(dev)
    gb, lmb, sb = _build(dev)
    views = {}
    for name, g in (("a", ga), ("b", gb)):
        wptr, sptr, gptr, n = g.param_arena()
        views[name] = (edp.device_view(wptr, n, dev), edp.device_view(sptr, n, dev, torch.bfloat16), edp.device_view(gptr, n, dev))
    shapes = [ga.shape(p) for p in sorted(lma.params())]
    offs, total = edp.param_offsets(shapes)
    buckets = edp.plan_buckets(offs, CFG["layers"], total, min_bucket_elems=1 << 18)
    exact = [(o, o + s[0]) for o, s in zip(offs, shapes) if len(s) == 1]  # norm weights are read in f32
    store = dist.distributed_c10d._get_default_store()
    red = edp.BucketedAllReduce(views["a"][2], buckets, backend=backend, handshake=edp.StepHandshake(store, rank, world, 60.0, "hs/a"))
    zex = edp.ShardedExchange(views["b"][2], buckets, gather=views["b"][1], flat_w=views["b"][0], exact_ranges=exact,
                              backend=backend, handshake=edp.StepHandshake(store, rank, world, 60.0, "hs/b"))
    opta = AdamW(ga, lma.params(), 1e-3)
    optb = ShardedAdamW(gb, lmb.params(), 1e-3, zex.pieces())
    for o in (opta, optb):
        o.config(1e-3, 0.9, 0.95, 1e-8, 0.1)
    order = [CFG["layers"]] + list(range(CFG["layers"] - 1, -1, -1)) + [-1]
    for step in range(2):
        opta.zero_grad()
        ids, tg = _batch(rank + 10 * step)
        x = ga.alloc_ids([B, S], ids)
        lma.train_micro_step(x, tg.tolist(), checkpoint=True)
        ga.clear_activations()
        ga.synchronize()
        views["b"][2].copy_(views["a"][2])  # same local gradient on both models
        torch.cuda.synchronize()
        for k in order:
            red.on_block_done(k, sa)
        red.finish(sa, deadline_s=60.0)
        opta.step_fused(0.5, red.grad_scale())
        for k in order:
            zex.on_block_done(k, sb, optimizer=optb)
        zex.finish_and_step(optb, 0.5, sb, deadline_s=60.0)
        ga.synchronize()
        gb.synchronize()
    zex.gather_master(sb)
    gb.synchronize()
    torch.cuda.synchronize()
    wa, sha = views["a"][0].cpu().numpy(), views["a"][1].float().cpu().numpy()
    wb, shb = views["b"][0].cpu().numpy(), views["b"][1].float().cpu().numpy()
    out.put((rank, float(np.linalg.norm(wa - wb) / np.linalg.norm(wa)), float((sha != shb).mean()),
             float(np.abs(wa - np.float32(0)).sum())))
    backend.close()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_sharded_step_equals_replicated_step():
    """ZeRO-1 (reduce-scatter, AdamW on the rank's pieces, all-gather of the bf16 weights, f32
    broadcast of the norm weights) through the eisen_dp_* C ABI against the replicated step
    (all-reduce, AdamW everywhere) on the same gradients, two optimizer steps with clipping."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_zero_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = [out.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, w_err, shadow_mismatch, wsum in got:
        assert w_err < 1e-6, (rank, w_err)
        assert shadow_mismatch < 1e-5, (rank, shadow_mismatch)
    assert got[0][3] == got[1][3]  # both ranks hold the same master weights after gather_master
