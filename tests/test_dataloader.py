"""Input side (u16 token files -> int32 batches, fill-in-the-middle): the library's loader against the
CPU restatement of src/data/dataloader.rs / src/data/fim.rs, bit for bit.  CPU only."""
import importlib.util
import os

import numpy as np
import pytest

import eisen_b200 as eb
from eisen_b200.data import BinaryDataLoader

_spec = importlib.util.spec_from_file_location(
    "dataloader_oracle", os.path.join(os.path.dirname(__file__), "..", "oracle", "dataloader_oracle.py"))
orc = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(orc)


def _token_file(tmp_path, n_tokens, vocab, seed):
    rng = np.random.default_rng(seed)
    toks = rng.integers(0, vocab, n_tokens).astype("<u2")
    path = tmp_path / ("tokens_%d.bin" % seed)
    toks.tofile(path)
    return str(path), toks.astype(np.int64)


def test_plain_batches_are_consecutive_windows(tmp_path):
    S, B = 16, 3
    path, toks = _token_file(tmp_path, 1000, 5000, 1)
    ld = BinaryDataLoader(path, S, B)
    assert ld.total_batches == 1000 // (B * (S + 1))
    n = 0
    while True:
        got = ld.next_batch()
        if got is None:
            break
        x, t, masked = got
        base = n * B * (S + 1)
        for b in range(B):
            w = toks[base + b * (S + 1): base + (b + 1) * (S + 1)]
            assert (x[b * S:(b + 1) * S] == w[:S]).all()
            assert (t[b * S:(b + 1) * S] == w[1:]).all()
        assert masked is False
        n += 1
    assert n == ld.total_batches  # the trailing partial batch is dropped
    ld.reset()
    x0, _, _ = ld.next_batch()
    assert (x0[:S] == toks[:S]).all()


@pytest.mark.parametrize("S,B,rate,spm,seed", [(32, 4, 0.5, 0.5, 1337), (7, 2, 1.0, 0.0, 5), (64, 1, 0.9, 1.0, 123456789),
                                              (3, 2, 1.0, 0.5, 9), (128, 3, 0.3, 0.7, 42)])
def test_fim_matches_oracle_bit_for_bit(tmp_path, S, B, rate, spm, seed):
    vocab = 1000
    path, _ = _token_file(tmp_path, 20000, vocab, seed)
    ld = BinaryDataLoader(path, S, B, fim=(vocab, rate, spm), seed=seed)
    ref = orc.BinaryDataLoaderOracle(path, S, B, fim=(vocab, rate, spm), seed=seed)
    assert ld.total_batches == ref.total_batches
    seen_masked = False
    for _ in range(min(ref.total_batches, 40)):
        got, exp = ld.next_batch(), ref.next_batch()
        assert (got is None) == (exp is None)
        if got is None:
            break
        assert (got[0] == exp[0]).all()
        assert (got[1] == exp[1]).all()
        assert got[2] == exp[2]
        seen_masked |= got[2]
        if got[2]:
            # trained positions follow the <fim_middle> sentinel only; control tokens are never targets to learn from
            x, t = got[0].reshape(B, S), got[1].reshape(B, S)
            for b in range(B):
                if t[b, -1] != -1 or (t[b] == -1).all() or S < 4:  # untransformed, or the middle was cut off
                    continue
                first = int(np.argmax(t[b] != -1))
                assert (x[b, :first + 1] == vocab + 2).any()
    assert seen_masked or rate < 1.0


def test_fim_off_still_advances_generator_identically(tmp_path):
    # the reference draws one number per sequence even without FIM (dataloader.rs:162): switching
    # FIM on later in a run sees the generator where the reference would have it
    S, B = 8, 2
    path, _ = _token_file(tmp_path, 4000, 300, 7)
    a = orc.BinaryDataLoaderOracle(path, S, B, fim=None, seed=11)
    for _ in range(5):
        a.next_batch()
    assert a.rng.s != 11


def test_loader_errors():
    with pytest.raises(eb.EisenError):
        BinaryDataLoader("/nonexistent/file.bin", 8, 2)


@pytest.mark.gpu
def test_pinned_feeder_drives_training_steps(tmp_path):
    """Batches that reach the device through the double-buffered pinned feeder give the same losses
    as the same batches (from the oracle loader) uploaded one by one."""
    import torch
    from eisen_b200.data import PinnedBatchFeeder
    from eisen_b200.graph import BF16_MIXED, Graph, TransformerLM

    vocab, S, B = 508, 128, 2  # + 4 control tokens = 512 rows (the bf16 GEMM wants multiples of 8)
    path, _ = _token_file(tmp_path, 6000, vocab, 3)
    dev = torch.device("cuda:0")
    losses = []
    for use_feeder in (True, False):
        stream = torch.cuda.Stream(device=dev)
        g = Graph(BF16_MIXED, stream.cuda_stream)
        lm = TransformerLM(g, vocab + 4, 128, 2, 2, 256, 1, False)
        g.mark_params()
        rng = np.random.default_rng(0)
        for p in lm.params():
            shp = g.shape(p)
            if len(shp) == 2:
                g.load_tensor_data(p, (rng.standard_normal(int(np.prod(shp))) * 0.02).astype(np.float32))
        out = []
        if use_feeder:
            feeder = PinnedBatchFeeder(BinaryDataLoader(path, S, B, fim=(vocab, 0.5, 0.5), seed=77), g, stream)
            for _ in range(4):
                ids, tgt, masked, n_valid = feeder.next()
                loss = lm.train_micro_step_dev(ids, tgt, n_valid)
                out.append(float(g.data(loss)[0]))
                g.clear_activations()
        else:
            ref = orc.BinaryDataLoaderOracle(path, S, B, fim=(vocab, 0.5, 0.5), seed=77)
            for _ in range(4):
                x, t, masked = ref.next_batch()
                ids = g.alloc_ids([B, S], x)
                tgt = g.alloc_ids([B * S], t)
                loss = lm.train_micro_step_dev(ids, tgt, int((t != -1).sum()))
                out.append(float(g.data(loss)[0]))
                g.clear_activations()
        losses.append(out)
    assert losses[0] == losses[1]
    assert all(np.isfinite(v) for v in losses[0])
