"""Greedy generation: the KV-cached path against the reference's loop (the whole context through
the forward pass for every token, examples/train_llm.rs:560-584) and against the CPU oracle."""
import numpy as np
import pytest

from conftest import rel_l2

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import eisen_b200 as eb  # noqa: E402
from eisen_b200.graph import BF16_MIXED, FP32, Graph, TransformerLM  # noqa: E402
from oracle_binding import OracleGraph, OracleLM  # noqa: E402


def _build(cfg, precision, seed, std, with_oracle=False):
    g = Graph(precision, torch.cuda.current_stream().cuda_stream)
    lm = TransformerLM(g, cfg["vocab"], cfg["hidden"], cfg["heads"], cfg["kv"], cfg["ffn"], cfg["layers"], cfg["tie"])
    g.mark_params()
    og = olm = None
    if with_oracle:
        og = OracleGraph()
        olm = OracleLM(og, cfg["vocab"], cfg["hidden"], cfg["heads"], cfg["kv"], cfg["ffn"], cfg["layers"], cfg["tie"])
        og.mark_params()
    rng = np.random.default_rng(seed)
    for p in lm.params():
        shp = g.shape(p)
        if len(shp) == 2:
            w = (rng.standard_normal(int(np.prod(shp))) * std).astype(np.float32)
            g.load_tensor_data(p, w)
            if og:
                og.load_tensor_data(p, w)
    return g, lm, og, olm


def _last_logits_full_forward(g, lm, tokens):
    g.set_no_grad(True)
    x = g.alloc_ids([1, len(tokens)], np.asarray(tokens, np.int32))
    lg = g.data(lm.forward(x)).reshape(len(tokens), -1)[-1].copy()
    g.clear_activations()
    g.set_no_grad(False)
    return lg


def _margin(lg):
    top = np.sort(lg)[-2:]
    return float(top[1] - top[0])


@pytest.mark.parametrize("tie", [False, True])
def test_kv_cached_generation_f32_matches_reference_loop_and_oracle(tie):
    cfg = dict(vocab=96, hidden=64, heads=4, kv=2, ffn=96, layers=2, tie=tie)
    g, lm, og, olm = _build(cfg, FP32, 3, 0.15, with_oracle=True)
    prompt = np.random.default_rng(1).integers(0, cfg["vocab"], 9).astype(np.int32)
    n_new = 7
    slow, slow_lg = lm.generate(prompt, n_new, 64, kv_cache=False, return_logits=True)
    fast, fast_lg = lm.generate(prompt, n_new, 64, kv_cache=True, return_logits=True)
    assert rel_l2(fast_lg, slow_lg) < 1e-4
    assert (slow == fast).all()
    # the oracle's forward over prompt + generated prefix gives the same last-position logits
    ctx = list(prompt) + list(fast[:-1])
    ox = og.alloc([1, len(ctx)], np.asarray(ctx, np.float32))
    og.set_no_grad(True)
    ol = og.data(olm.forward(ox)).reshape(len(ctx), -1)
    assert rel_l2(fast_lg, ol[-1]) < 1e-4
    for i in range(n_new):  # every generated token is the oracle's argmax where that is not a near tie
        row = ol[len(prompt) - 1 + i]
        if _margin(row) > 1e-3:
            assert fast[i] == int(np.argmax(row))


@pytest.mark.parametrize("hd_heads", [(64, 4, 2), (128, 2, 1)])
def test_kv_cached_generation_bf16(hd_heads):
    hd, heads, kv = hd_heads
    cfg = dict(vocab=512, hidden=hd * heads, heads=heads, kv=kv, ffn=512, layers=2, tie=False)
    g, lm, _, _ = _build(cfg, BF16_MIXED, 4, 0.05)
    prompt = np.random.default_rng(2).integers(0, cfg["vocab"], 150).astype(np.int32)  # ragged against the 128-row tiles
    prev = None
    for k in (1, 3, 6):
        toks, lg = lm.generate(prompt, k, 256, kv_cache=True, return_logits=True)
        if prev is not None:
            assert (toks[: len(prev)] == prev).all()  # deterministic: a longer run extends a shorter one
        prev = toks
        ref = _last_logits_full_forward(g, lm, list(prompt) + list(toks[:-1]))
        assert rel_l2(lg, ref) < 2e-2
        if _margin(ref) > 0.05 * float(np.abs(ref).max()):
            assert toks[-1] == int(np.argmax(ref))


def test_generation_window_rules():
    cfg = dict(vocab=64, hidden=32, heads=2, kv=1, ffn=64, layers=1, tie=False)
    g, lm, _, _ = _build(cfg, FP32, 5, 0.2)
    prompt = np.arange(10, dtype=np.int32)
    with pytest.raises(eb.EisenError, match="max_context"):
        lm.generate(prompt, 8, 12, kv_cache=True)  # 10 + 8 > 12: the window would slide
    out = lm.generate(prompt, 8, 12, kv_cache=False)  # the reference's sliding window
    assert out.shape == (8,) and (out >= 0).all() and (out < cfg["vocab"]).all()
    with pytest.raises(eb.EisenError):
        lm.generate(np.array([999], np.int32), 1, 8)
    # the no_grad flag is restored and training still works afterwards
    x = g.alloc_ids([1, 10], prompt)
    loss = lm.train_micro_step(x, list(range(10)))
    assert np.isfinite(g.data(loss)[0])
