"""VRAM budget and parameter streaming: the residency plan against its restatement (integer
bookkeeping: exact), and a training step with streamed weights against the same step with
everything resident."""
import os
import sys

import numpy as np
import pytest

from conftest import rel_l2

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))

import eisen_b200 as eb  # noqa: E402
from eisen_b200.graph import AdamW, BF16_MIXED, FP32, Graph, TransformerLM  # noqa: E402
from streaming_oracle import plan_streaming_layout  # noqa: E402

CFG = dict(vocab=512, hidden=256, heads=4, kv=2, ffn=512, layers=3)


def _build(precision, budget=None, seed=0):
    g = Graph(precision, torch.cuda.current_stream().cuda_stream)
    if budget is not None:
        g.set_vram_budget(budget, 1 << 20)
    lm = TransformerLM(g, CFG["vocab"], CFG["hidden"], CFG["heads"], CFG["kv"], CFG["ffn"], CFG["layers"], False)
    g.mark_params()
    rng = np.random.default_rng(seed)
    for p in lm.params():
        shp = g.shape(p)
        if len(shp) == 2:
            g.load_tensor_data(p, (rng.standard_normal(int(np.prod(shp))) * 0.02).astype(np.float32))
    return g, lm


def _pinned(lm):
    ps = sorted(lm.params())
    return [ps[0], ps[-2], ps[-1]]  # embedding, final norm, head (examples/train_llm.rs:245-251)


@pytest.mark.parametrize("budget_mb,reserve_mb", [(1 << 12, 1), (40, 1), (30, 4), (22, 1), (16, 2), (9, 1), (0, 0)])
def test_streaming_plan_matches_restatement(budget_mb, reserve_mb):
    g, lm = _build(FP32)
    n = g.counts()[2]
    sizes = [int(np.prod(g.shape(i))) for i in range(n)]
    got = g.plan_streaming(budget_mb << 20, reserve_mb << 20, _pinned(lm), apply=False)
    want = plan_streaming_layout(sizes, budget_mb << 20, reserve_mb << 20, _pinned(lm))
    assert got == want
    assert sorted(got["resident_param_ids"] + got["streamed_param_ids"]) == list(range(n))


def test_budget_makes_activation_allocation_fail_cleanly():
    g, lm = _build(FP32)
    used, _ = g.vram_usage()
    g.set_vram_budget(used + (1 << 20), 0)
    with pytest.raises(eb.EisenError, match="budget"):
        g.alloc_pooled([1 << 20])  # 4 MB of f32 against 1 MB of room
    small = g.alloc_pooled([1 << 10])  # still usable afterwards
    assert g.shape(small) == [1 << 10]


@pytest.mark.parametrize("precision,tol", [(FP32, 1e-5), (BF16_MIXED, 2e-2)])
def test_step_with_streamed_weights_matches_resident_step(precision, tol):
    """Two optimizer steps of a model whose block weights are partly streamed from host memory
    (staged through the copy stream, gradients and moments on the host) against the same steps with
    every parameter resident."""
    rng = np.random.default_rng(5)
    batches = [(rng.integers(0, CFG["vocab"], (2, 128)).astype(np.int32), rng.integers(0, CFG["vocab"], 256)) for _ in range(2)]

    reserve = 0

    def run(budget):
        g, lm = _build(precision, budget)
        rep = None
        if budget is not None:
            rep = g.plan_streaming(budget, reserve, _pinned(lm))
        opt = AdamW(g, lm.params(), 1e-3)
        opt.config(1e-3, 0.9, 0.95, 1e-8, 0.1)
        losses = []
        for ids, tg in batches:
            opt.zero_grad()
            loss = lm.train_micro_step(g.alloc_ids([2, 128], ids), tg.tolist(), checkpoint=True)
            losses.append(float(g.data(loss)[0]))
            g.clear_activations()
            opt.step_fused(1.0, 1.0)
        g.synchronize()
        return [g.data(p) for p in lm.params()], losses, rep, opt.is_flat()

    full, full_loss, _, full_flat = run(None)
    # 16 bytes per element: of 64 MB, 55 MB are reserved for activations and staging, 4 MB hold the pinned
    # embedding and head; the 5 MB left keep a few block matrices resident, the other ones stream
    reserve = 55 << 20
    part, part_loss, rep, part_flat = run(64 << 20)
    used, budget = 0, 0
    assert full_flat and not part_flat
    assert len(rep["streamed_param_ids"]) >= 8 and len(rep["resident_param_ids"]) >= 4
    for a, b in zip(full_loss, part_loss):
        assert abs(a - b) < (1e-5 if precision == FP32 else 1e-3) * max(1.0, abs(a))
    for a, b in zip(full, part):
        assert rel_l2(b, a) < tol
