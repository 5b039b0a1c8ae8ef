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
