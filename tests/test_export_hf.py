"""Hugging Face export: the safetensors file against a numpy restatement of the reference exporter
(examples/export_hf_pipeline.rs:24-55, 200-260), and the exported model against this engine's own
forward pass when loaded into transformers' LlamaForCausalLM (which rotates half-split pairs: the
q / k row permutation is what makes the two agree)."""
import json
import math

import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu


def _permute_rope_hf(w_out_in, heads, hd):
    out = np.zeros_like(w_out_in)
    for h in range(heads):
        for p in range(hd // 2):
            out[h * hd + p] = w_out_in[h * hd + 2 * p]
            out[h * hd + hd // 2 + p] = w_out_in[h * hd + 2 * p + 1]
    return out


def _build(tie):
    import torch
    from eisen_b200.graph import FP32, Graph, TransformerLM

    cfg = dict(vocab=96, hidden=64, heads=4, kv=2, ffn=160, layers=2)
    stream = torch.cuda.Stream()
    g = Graph(FP32, stream.cuda_stream)
    lm = TransformerLM(g, cfg["vocab"], cfg["hidden"], cfg["heads"], cfg["kv"], cfg["ffn"], cfg["layers"], tie)
    g.mark_params()
    rng = np.random.default_rng(1)
    for p in lm.params():
        shp = g.shape(p)
        scale = 0.1 if len(shp) == 2 else 0.2
        base = 0.0 if len(shp) == 2 else 1.0
        g.load_tensor_data(p, (base + rng.standard_normal(int(np.prod(shp))) * scale).astype(np.float32))
    return cfg, g, lm, stream


@pytest.mark.parametrize("tie", [False, True])
def test_safetensors_file_matches_restated_exporter(tmp_path, tie):
    from safetensors.numpy import load_file

    cfg, g, lm, _ = _build(tie)
    st, cj = tmp_path / "model.safetensors", tmp_path / "config.json"
    lm.export_hf(st, cj, max_position_embeddings=128)
    tensors = load_file(str(st))
    hd = cfg["hidden"] // cfg["heads"]
    params = lm.params()  # emb, per block [norm1, q, k, v, o, norm2, up, down, gate], norm_f, [head]
    expect = {"model.embed_tokens.weight": g.data(params[0]).reshape(g.shape(params[0]))}
    for i in range(cfg["layers"]):
        n1, q, k, v, o, n2, up, down, gate = params[1 + 9 * i: 10 + 9 * i]
        pre = "model.layers.%d." % i
        W = lambda t: g.data(t).reshape(g.shape(t)).T.copy()  # noqa: E731  [in,out] -> [out,in]
        expect[pre + "input_layernorm.weight"] = g.data(n1)
        expect[pre + "post_attention_layernorm.weight"] = g.data(n2)
        expect[pre + "self_attn.q_proj.weight"] = _permute_rope_hf(W(q), cfg["heads"], hd)
        expect[pre + "self_attn.k_proj.weight"] = _permute_rope_hf(W(k), cfg["kv"], hd)
        expect[pre + "self_attn.v_proj.weight"] = W(v)
        expect[pre + "self_attn.o_proj.weight"] = W(o)
        expect[pre + "mlp.gate_proj.weight"] = W(gate)
        expect[pre + "mlp.up_proj.weight"] = W(up)
        expect[pre + "mlp.down_proj.weight"] = W(down)
    expect["model.norm.weight"] = g.data(params[1 + 9 * cfg["layers"]])
    if not tie:
        t = params[2 + 9 * cfg["layers"]]
        expect["lm_head.weight"] = g.data(t).reshape(g.shape(t)).T.copy()
    assert sorted(tensors) == sorted(expect)
    for name, ref in expect.items():
        assert tensors[name].shape == ref.shape, name
        assert np.array_equal(tensors[name], ref), name
    # header: 8-byte length, JSON padded with spaces to a multiple of 8, names in sorted order
    raw = open(st, "rb").read()
    hl = int.from_bytes(raw[:8], "little")
    assert hl % 8 == 0
    header = json.loads(raw[8:8 + hl].decode())
    assert list(header) == sorted(header)
    conf = json.load(open(cj))
    assert conf["num_key_value_heads"] == cfg["kv"] and conf["num_attention_heads"] == cfg["heads"]
    assert conf["tie_word_embeddings"] is tie and conf["rms_norm_eps"] == 1e-5 and conf["rope_theta"] == 10000.0


def test_exported_model_reproduces_logits_in_transformers(tmp_path):
    torch = pytest.importorskip("torch")
    transformers = pytest.importorskip("transformers")
    from safetensors.torch import load_file

    cfg, g, lm, _ = _build(False)
    st, cj = tmp_path / "model.safetensors", tmp_path / "config.json"
    lm.export_hf(st, cj, max_position_embeddings=128)
    B, S = 2, 24
    ids = np.random.default_rng(2).integers(0, cfg["vocab"], (B, S)).astype(np.int32)
    g.set_no_grad(True)
    logits = g.data(lm.forward(g.alloc_ids([B, S], ids))).reshape(B, S, cfg["vocab"])
    hf_cfg = transformers.LlamaConfig.from_json_file(str(cj))
    hf_cfg._attn_implementation = "eager"
    model = transformers.LlamaForCausalLM(hf_cfg).float().eval()
    missing, unexpected = model.load_state_dict(load_file(str(st)), strict=False)
    assert not unexpected and all("rotary" in m or "inv_freq" in m for m in missing), (missing, unexpected)
    with torch.no_grad():
        ref = model(torch.from_numpy(ids.astype(np.int64))).logits.numpy()
    assert rel_l2(logits, ref) < 1e-4
    assert math.isfinite(float(ref.sum()))


def test_weights_checkpoint_round_trip(tmp_path):
    """save_weights writes the parameters back to back in id order (the reference's eisen_model.bin);
    load_weights restores them bit for bit into a second, identically built model (bf16 copies included)."""
    import torch
    from eisen_b200.graph import BF16_MIXED, Graph, TransformerLM

    def build(seed):
        stream = torch.cuda.Stream()
        g = Graph(BF16_MIXED, stream.cuda_stream)
        lm = TransformerLM(g, 256, 128, 2, 1, 256, 2, False)
        g.mark_params()
        rng = np.random.default_rng(seed)
        for p in lm.params():
            shp = g.shape(p)
            if len(shp) == 2:
                g.load_tensor_data(p, (rng.standard_normal(int(np.prod(shp))) * 0.02).astype(np.float32))
        return g, lm, stream

    g1, lm1, _ = build(1)
    path = tmp_path / "eisen_model.bin"
    g1.save_weights(path)
    flat = np.fromfile(path, dtype="<f4")
    expect = np.concatenate([g1.data(p).reshape(-1) for p in sorted(lm1.params())])
    assert np.array_equal(flat, expect)
    g2, lm2, _ = build(2)
    assert not np.array_equal(g2.data(lm2.params()[1 + 1]), g1.data(lm1.params()[1 + 1]))
    g2.load_weights(path)
    for a, b in zip(lm1.params(), lm2.params()):
        assert np.array_equal(g1.data(a), g2.data(b))
    ids = np.random.default_rng(3).integers(0, 256, (2, 128)).astype(np.int32)
    outs = []
    for g, lm in ((g1, lm1), (g2, lm2)):
        g.set_no_grad(True)
        outs.append(g.data(lm.forward(g.alloc_ids([2, 128], ids))))
    assert np.array_equal(outs[0], outs[1])  # the bf16 shadows were refreshed as well
    with pytest.raises(Exception):
        open(tmp_path / "short.bin", "wb").write(b"1234")
        g2.load_weights(tmp_path / "short.bin")


def test_resume_from_weights_and_optimizer_state_is_bit_exact(tmp_path):
    """Two optimizer steps == one step, save (weights + optimizer state), load into a freshly built
    model and optimizer, one more step: bit for bit in the f32 graph (whose kernels use no atomics)."""
    import torch
    from eisen_b200.graph import AdamW, FP32, Graph, TransformerLM

    cfg = dict(vocab=128, hidden=64, heads=2, kv=1, ffn=128, layers=2)
    rng = np.random.default_rng(9)
    batches = [(rng.integers(0, cfg["vocab"], (2, 16)).astype(np.int32), rng.integers(0, cfg["vocab"], 32)) for _ in range(2)]

    def build(seed):
        g = Graph(FP32, torch.cuda.current_stream().cuda_stream)
        lm = TransformerLM(g, cfg["vocab"], cfg["hidden"], cfg["heads"], cfg["kv"], cfg["ffn"], cfg["layers"], False)
        g.mark_params()
        r = np.random.default_rng(seed)
        for p in lm.params():
            shp = g.shape(p)
            if len(shp) == 2:
                g.load_tensor_data(p, (r.standard_normal(int(np.prod(shp))) * 0.02).astype(np.float32))
        opt = AdamW(g, lm.params(), 1e-2)
        opt.config(1e-2, 0.9, 0.95, 1e-8, 0.1)
        return g, lm, opt

    def step(g, lm, opt, b):
        opt.zero_grad()
        lm.train_micro_step(g.alloc_ids([2, 16], b[0]), b[1].tolist())
        g.clear_activations()
        opt.step_fused(1.0, 1.0)
        g.synchronize()

    g1, lm1, o1 = build(1)
    step(g1, lm1, o1, batches[0])
    g1.save_weights(tmp_path / "w.bin")
    o1.save_state(tmp_path / "opt.bin")
    step(g1, lm1, o1, batches[1])

    g2, lm2, o2 = build(2)  # other initial weights, fresh moments, t = 0
    g2.load_weights(tmp_path / "w.bin")
    o2.load_state(tmp_path / "opt.bin")
    step(g2, lm2, o2, batches[1])
    for a, b in zip(lm1.params(), lm2.params()):
        assert np.array_equal(g1.data(a), g2.data(b))

    # without the optimizer state the resumed step differs (moments and bias correction restart)
    g3, lm3, o3 = build(2)
    g3.load_weights(tmp_path / "w.bin")
    step(g3, lm3, o3, batches[1])
    assert not np.array_equal(g1.data(lm1.params()[1]), g3.data(lm3.params()[1]))
    # a state file of another model is rejected
    gs = Graph(FP32, torch.cuda.current_stream().cuda_stream)
    lms = TransformerLM(gs, 64, 32, 2, 1, 64, 1, False)
    gs.mark_params()
    with pytest.raises(Exception, match="another model"):
        AdamW(gs, lms.params(), 1e-2).load_state(tmp_path / "opt.bin")
