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
