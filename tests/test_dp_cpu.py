"""Data-parallel host logic on CPU: two gloo ranks, gradients from the CPU oracle.

Checks the bucket plan over the flat gradient layout and that the bucketed all-reduce of the
per-rank gradients equals the single-process gradient accumulated over both micro-batches
(a sum, as the reference accumulates: tests/test_grad_accum.rs:108-166).
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from eisen_b200 import dp as edp
from oracle_binding import OracleGraph, OracleLM

CFG = dict(vocab=64, hidden=32, heads=2, kv=1, ffn=64, layers=3)
B, S = 2, 8


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _model(seed=0):
    og = OracleGraph()
    lm = OracleLM(og, CFG["vocab"], CFG["hidden"], CFG["heads"], CFG["kv"], CFG["ffn"], CFG["layers"], False)
    og.mark_params()
    rng = np.random.default_rng(seed)
    for p in lm.params():
        shp = og.shape(p)
        if len(shp) == 2:
            og.load_tensor_data(p, (rng.standard_normal(int(np.prod(shp))) * 0.02).astype(np.float32))
    return og, lm


def _micro_batch(rank):
    rng = np.random.default_rng(100 + rank)  # per-rank seed
    return rng.integers(0, CFG["vocab"], (B, S)), rng.integers(0, CFG["vocab"], B * S)


def _grads_flat(og, lm, batches):
    for ids, tg in batches:
        x = og.alloc([B, S], ids.astype(np.float32))
        lg = lm.forward(x)
        og.reinterpret_shape(lg, [B * S, CFG["vocab"]])
        og.backward(og.cross_entropy(lg, tg.tolist()))
        og.clear_activations()
    ids_sorted = sorted(lm.params())  # creation order == arena order
    offs, total = edp.param_offsets([og.shape(p) for p in ids_sorted])
    flat = torch.zeros(total, dtype=torch.float32)
    for p, o in zip(ids_sorted, offs):
        g = og.grad(p)
        flat[o:o + g.size] = torch.from_numpy(g)
    return flat, offs, total


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    og, lm = _model()
    flat, offs, total = _grads_flat(og, lm, [_micro_batch(rank)])
    buckets = edp.plan_buckets(offs, CFG["layers"], total, min_bucket_elems=0)
    red = edp.BucketedAllReduce(flat, buckets)
    # the backward pass reports: head/final norm, blocks last to first, embedding
    for key in [CFG["layers"]] + list(range(CFG["layers"] - 1, -1, -1)) + [-1]:
        red.on_block_done(key)
    red.finish()
    assert abs(red.grad_scale() - 1.0 / world) < 1e-12
    if rank == 0:
        out.put(flat.numpy().copy())
    dist.barrier()
    dist.destroy_process_group()


def test_bucket_plan_covers_arena_once():
    og, lm = _model()
    ids_sorted = sorted(lm.params())
    offs, total = edp.param_offsets([og.shape(p) for p in ids_sorted])
    for min_elems in (0, 5000, 10 ** 9):
        b = edp.plan_buckets(offs, CFG["layers"], total, min_bucket_elems=min_elems)
        spans = sorted((a, e) for _, a, e in b)
        assert spans[0][0] == 0 and spans[-1][1] == total
        for (a0, e0), (a1, e1) in zip(spans, spans[1:]):
            assert e0 == a1  # contiguous, no overlap
        keys = [k for k, _, _ in b]
        assert keys[0] == CFG["layers"] and keys[-1] == -1  # backward order
        assert keys[1:-1] == sorted(keys[1:-1], reverse=True)
    # with a huge minimum all blocks share one bucket that completes with block 0
    assert [k for k, _, _ in edp.plan_buckets(offs, CFG["layers"], total, 10 ** 9)] == [CFG["layers"], 0, -1]


@pytest.mark.timeout(300)
def test_two_rank_allreduce_equals_accumulated_single_process():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    reduced = out.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    og, lm = _model()
    ref, _, _ = _grads_flat(og, lm, [_micro_batch(0), _micro_batch(1)])
    num = np.linalg.norm(reduced - ref.numpy())
    assert num / np.linalg.norm(ref.numpy()) < 1e-6


# ------------------------------------------------------------------------------ ZeRO-1 host logic
class _NumpyAdamW:
    """AdamW of src/nn/optim.rs:523-543 on flat CPU tensors, whole buffer or pieces of it."""

    def __init__(self, w, g, pieces, lr=1e-2, b1=0.9, b2=0.95, eps=1e-8, wd=0.1):
        self.w, self.g, self.pieces = w, g, pieces
        self.lr, self.b1, self.b2, self.eps, self.wd = lr, b1, b2, eps, wd
        self.m = [torch.zeros(b - a) for a, b in pieces]
        self.v = [torch.zeros(b - a) for a, b in pieces]
        self.sumsq = torch.zeros(1, dtype=torch.float64)
        self.t = 0

    def begin_step(self):
        self.t += 1

    def sumsq_piece(self, i, accumulate, stream=None):
        a, b = self.pieces[i]
        s = (self.g[a:b].double() ** 2).sum()
        self.sumsq[0] = self.sumsq[0] + s if accumulate else s

    def step_piece(self, i, max_norm, grad_scale):
        a, b = self.pieces[i]
        gs = grad_scale
        if max_norm > 0:
            norm = float(self.sumsq[0].sqrt()) * abs(grad_scale)
            if norm > 0:
                gs *= min(max_norm / (norm + 1e-6), 1.0)
        g = self.g[a:b] * gs
        w = self.w[a:b]
        w.mul_(1.0 - self.lr * self.wd)
        self.m[i].mul_(self.b1).add_(g, alpha=1 - self.b1)
        self.v[i].mul_(self.b2).addcmul_(g, g, value=1 - self.b2)
        bc1, bc2 = 1.0 / (1.0 - self.b1 ** self.t), 1.0 / (1.0 - self.b2 ** self.t)
        w.sub_(self.lr * (self.m[i] * bc1) / ((self.v[i] * bc2).sqrt() + self.eps))


def _grads_for(rank, step):
    og, lm = _model()
    rng = np.random.default_rng(1000 * step + rank)
    batch = (rng.integers(0, CFG["vocab"], (B, S)), rng.integers(0, CFG["vocab"], B * S))
    return _grads_flat(og, lm, [batch])


def _weights_flat(total):
    return torch.from_numpy(np.random.default_rng(5).standard_normal(total).astype(np.float32))


BACKWARD_ORDER = [CFG["layers"]] + list(range(CFG["layers"] - 1, -1, -1)) + [-1]


def _zero_worker(rank, world, port, out, steps):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    flat, offs, total = _grads_for(rank, 0)
    buckets = edp.plan_buckets(offs, CFG["layers"], total, min_bucket_elems=0)
    w = _weights_flat(total)
    store = dist.distributed_c10d._get_default_store()
    ex = edp.ShardedExchange(flat, buckets, gather=w, handshake=edp.StepHandshake(store, rank, world, timeout_s=20.0))
    opt = _NumpyAdamW(w, flat, ex.pieces())
    for step in range(steps):
        flat.copy_(_grads_for(rank, step)[0])
        for key in BACKWARD_ORDER:
            ex.on_block_done(key, optimizer=opt)
        ex.finish_and_step(opt, max_norm=0.05)
    out.put((rank, w.numpy().copy()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_sharded_step_equals_replicated_step():
    """reduce-scatter -> AdamW on each rank's pieces -> all-gather == all-reduce -> AdamW everywhere,
    over two optimizer steps with clipping (the clip needs the norm summed over the shards)."""
    world, steps = 2, 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_zero_worker, args=(r, world, port, out, steps)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(out.get(timeout=240) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # replicated reference in this process
    _, offs, total = _grads_for(0, 0)
    w = _weights_flat(total)
    g = torch.zeros(total)
    ref = _NumpyAdamW(w, g, [(0, total)])
    for step in range(steps):
        g.copy_(_grads_for(0, step)[0] + _grads_for(1, step)[0])
        ref.begin_step()
        ref.sumsq_piece(0, False)
        ref.step_piece(0, 0.05, 1.0 / world)
    for r in range(world):
        assert np.linalg.norm(got[r] - w.numpy()) / np.linalg.norm(w.numpy()) < 1e-6
    assert (got[0] == got[1]).all()  # the replicas agree bit for bit after the gather


def test_sharded_exchange_exact_ranges_and_pieces():
    flat = torch.zeros(64 * 6)
    buckets = [(1, 128, 384), (0, 0, 128)]

    class _B:  # two ranks without a process group
        world, rank, launched, comm_stream = 2, 1, 0, None

    ex = edp.ShardedExchange(flat, buckets, gather=flat, flat_w=flat, exact_ranges=[(120, 136), (250, 262)], backend=_B())
    assert ex.pieces() == [(256, 384), (64, 128)]
    assert ex.exact == [(128, 136, 0), (120, 128, 1), (250, 256, 0), (256, 262, 1)] or sorted(ex.exact) == sorted(
        [(128, 136, 0), (120, 128, 1), (250, 256, 0), (256, 262, 1)])
    with pytest.raises(edp.EisenError):
        edp.ShardedExchange(torch.zeros(24), [(0, 0, 24)], gather=flat, backend=_B())  # 24 elements do not split into 2 x 8k


# ------------------------------------------------------------------------------ failure handling
def _put_and_exit(out, item):
    out.put(item)
    out.close()
    out.join_thread()  # the queue's feeder thread has written the item before the process goes
    os._exit(0)


def _failing_worker(rank, world, port, out, mode):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    flat, offs, total = _grads_for(rank, 0)
    buckets = edp.plan_buckets(offs, CFG["layers"], total, min_bucket_elems=0)
    store = dist.distributed_c10d._get_default_store()
    red = edp.BucketedAllReduce(flat, buckets, handshake=edp.StepHandshake(store, rank, world, timeout_s=3.0))
    result = "ok"
    try:
        for step in range(2):
            if mode == "leave" and rank == 1 and step == 1:
                # the rank leaves between steps, with nothing of its own in flight
                _put_and_exit(out, (rank, "left"))
            if mode == "skip" and rank == 1 and step == 1:
                # host-side fault: this rank forgets its last bucket (the embedding's), so the peer is
                # left with one all-reduce that nobody answers
                red.skip_keys = {-1}
            for key in BACKWARD_ORDER:
                red.on_block_done(key)
            t0 = __import__("time").monotonic()
            red.finish(deadline_s=10.0)
    except edp.EisenError as e:
        result = "error after %.1f s: %s" % (__import__("time").monotonic() - t0, e)
    _put_and_exit(out, (rank, result))  # no teardown: collectives of a broken step may still be pending


@pytest.mark.timeout(120)
@pytest.mark.parametrize("mode", ["leave", "skip"])
def test_survivor_gets_an_error_not_a_hang(mode):
    """A rank that leaves between steps, or that skips a bucket, is detected on the host (step
    handshake through the store) within the deadline; nobody blocks on the broken collective."""
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, world, port, out, mode)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(out.get(timeout=60) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
    assert got[0].startswith("error"), got
    if mode == "leave":
        assert got[1] == "left" and "did not reach step 1" in got[0]
    else:
        assert got[1].startswith("error") and "out of step" in got[0] and "out of step" in got[1]
