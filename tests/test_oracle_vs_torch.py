"""Independent cross-check of the CPU oracle's whole model against PyTorch autograd (CPU).

The oracle restates the reference's CPU arms; nothing in the reference's own tests pins a
whole-model gradient, GQA with repeats > 1, masked cross-entropy, the tied head or AdamW values.
This test evaluates the same model with an implementation that shares no code with the oracle:
a float64 PyTorch module written from the formulas (interleaved-pair RoPE with
theta = pos / 10000^(2p/D) (src/graph/ops/transform.rs:559-565), RMSNorm 1/sqrt(mean(x^2) + eps)
(src/graph/ops/normalization.rs:141-152), additive -1e20 causal mask (src/nn/attention.rs:354),
loss -ln(p + 1e-8) whose epsilon is not differentiated (src/graph/ops/reduction.rs:690-708), mean over
the valid rows (reduction.rs:737), AdamW with decay on every parameter and reciprocal bias
corrections (src/nn/optim.rs:336-338, 537-542)) and compares loss, logits, every parameter
gradient and the parameters after one AdamW step.
"""
import math

import numpy as np
import pytest

from oracle_binding import OracleAdamW, OracleGraph, OracleLM

torch = pytest.importorskip("torch")


def rel_l2(a, b):
    a = np.asarray(a, np.float64).reshape(-1)
    b = np.asarray(b, np.float64).reshape(-1)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


def rope_interleaved(x, head_dim):
    """x: [B, S, H*D]; pairs (2p, 2p+1) inside each head rotate by pos / 10000^(2p/D)."""
    B, S, W = x.shape
    xh = x.reshape(B, S, W // head_dim, head_dim // 2, 2)
    p = torch.arange(head_dim // 2, dtype=torch.float64)
    # the reference forms the angle in f32: theta = pos / powf(10000, 2p/D)
    freq = torch.pow(torch.tensor(10000.0, dtype=torch.float32), (2.0 * p / head_dim).to(torch.float32))
    theta = (torch.arange(S, dtype=torch.float32)[:, None] / freq[None, :]).to(torch.float32)
    c = torch.cos(theta).to(torch.float64)[None, :, None, :]
    s = torch.sin(theta).to(torch.float64)[None, :, None, :]
    x0, x1 = xh[..., 0], xh[..., 1]
    return torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1).reshape(B, S, W)


def rms_norm(x, w, eps=1e-5):
    return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


class TorchLM:
    def __init__(self, cfg, tie, weights):
        """weights: list of float32 arrays in the reference's params() order."""
        self.cfg, self.tie = cfg, tie
        self.p = [torch.tensor(np.asarray(w, np.float64), requires_grad=True) for w in weights]

    def forward(self, ids):
        c = self.cfg
        H, KV, d = c["heads"], c["kv"], c["hidden"]
        hd = d // H
        it = iter(self.p)
        emb = next(it)
        x = emb[torch.as_tensor(ids)]  # [B,S,d]
        B, S, _ = x.shape
        mask = torch.triu(torch.full((S, S), -1e20, dtype=torch.float64), diagonal=1)
        for _ in range(c["layers"]):
            # params(): norm1, q, k, v, o, norm2, up, down, gate (src/nn/transformer.rs:57-66)
            n1, wq, wk, wv, wo, n2, wup, wdown, wgate = (next(it) for _ in range(9))
            h = rms_norm(x, n1)
            q = rope_interleaved(h @ wq, hd).reshape(B, S, H, hd).transpose(1, 2)
            k = rope_interleaved(h @ wk, hd).reshape(B, S, KV, hd).transpose(1, 2)
            v = (h @ wv).reshape(B, S, KV, hd).transpose(1, 2)
            k = k.repeat_interleave(H // KV, dim=1)  # query head h reads kv head h / r (src/graph/ops/gqa.rs:148-157)
            v = v.repeat_interleave(H // KV, dim=1)
            s = (q @ k.transpose(-1, -2)) * (1.0 / math.sqrt(hd)) + mask
            ctx = (torch.softmax(s, dim=-1) @ v).transpose(1, 2).reshape(B, S, d)
            x = x + ctx @ wo
            h2 = rms_norm(x, n2)
            x = x + (torch.nn.functional.silu(h2 @ wgate) * (h2 @ wup)) @ wdown
        nf = next(it)
        x = rms_norm(x, nf)
        if self.tie:
            return x @ emb.t()
        return x @ next(it)


def loss_and_backward(logits, targets):
    """Value: mean over valid rows of -ln(p_t + 1e-8); gradient: that of the plain cross-entropy."""
    t = torch.as_tensor(targets)
    valid = t >= 0
    lg = logits.reshape(-1, logits.shape[-1])[valid]
    tv = t[valid]
    p = torch.softmax(lg.detach(), dim=-1).gather(1, tv[:, None]).squeeze(1)
    value = float((-(p + 1e-8).log()).mean())
    torch.nn.functional.cross_entropy(lg, tv, reduction="mean").backward()
    return value


@pytest.mark.parametrize("tie,masked", [(False, True), (True, False), (False, False)])
def test_whole_model_oracle_matches_torch_autograd(tie, masked):
    cfg = dict(vocab=96, hidden=48, heads=4, kv=2, ffn=80, layers=2, batch=2, seq=24)
    rng = np.random.default_rng(11 + tie + 2 * masked)
    og = OracleGraph()
    olm = OracleLM(og, cfg["vocab"], cfg["hidden"], cfg["heads"], cfg["kv"], cfg["ffn"], cfg["layers"], tie)
    og.mark_params()
    ps = olm.params()
    weights = []
    for p in ps:
        shp = og.shape(p)
        if len(shp) == 2:
            w = (rng.standard_normal(shp) * 0.05).astype(np.float32)
        else:
            w = (1.0 + 0.1 * rng.standard_normal(shp)).astype(np.float32)  # norm gains away from 1
        og.load_tensor_data(p, w)
        weights.append(w)
    ids = rng.integers(0, cfg["vocab"], (cfg["batch"], cfg["seq"]))
    tg = rng.integers(0, cfg["vocab"], cfg["batch"] * cfg["seq"])
    if masked:
        tg[rng.random(tg.size) < 0.25] = -1
        tg[0] = 3

    ox = og.alloc([cfg["batch"], cfg["seq"]], ids.astype(np.float32))
    ol = olm.forward(ox)
    og.reinterpret_shape(ol, [cfg["batch"] * cfg["seq"], cfg["vocab"]])
    oloss = og.cross_entropy_masked(ol, tg.tolist()) if masked else og.cross_entropy(ol, tg.tolist())
    og.backward(oloss)

    tm = TorchLM(cfg, tie, weights)
    logits = tm.forward(ids)
    value = loss_and_backward(logits, tg)

    assert abs(float(og.data(oloss)[0]) - value) <= 1e-5 * max(1.0, abs(value))
    assert rel_l2(og.data(ol), logits.detach().numpy()) < 1e-5
    for i, (p, tp) in enumerate(zip(ps, tm.p)):
        assert rel_l2(og.grad(p), tp.grad.numpy()) < 1e-5, ("gradient of parameter", i, og.shape(p))

    # one AdamW step (t = 1): w *= 1 - lr*wd; m, v EMA; w -= lr * m*bc1 / (sqrt(v*bc2) + eps)
    lr, b1, b2, eps, wd = 3e-3, 0.9, 0.95, 1e-8, 0.1
    oopt = OracleAdamW(og, ps, lr)
    oopt.config(lr, b1, b2, eps, wd)
    oopt.step()
    bc1, bc2 = 1.0 / (1.0 - b1), 1.0 / (1.0 - b2)
    for i, (p, tp) in enumerate(zip(ps, tm.p)):
        g = tp.grad.numpy()
        w = tp.detach().numpy() * (1.0 - lr * wd)
        m, v = (1.0 - b1) * g, (1.0 - b2) * g * g
        w = w - lr * (m * bc1) / (np.sqrt(v * bc2) + eps)
        assert rel_l2(og.data(p), w) < 1e-5, ("parameter after AdamW", i)
