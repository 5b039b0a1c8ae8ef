"""Checks at the full sizes of the benchmark configurations (run on a B200 with `-m gpu`).

The CPU oracle cannot produce these sizes in test time, so the checker is either an f32 evaluation
of the same bf16 inputs on the device (plain torch ops on sampled heads, rows or slices: the kernel
under test still runs on the whole problem), or a property that does not depend on the size
(attention rows that must average their values, a checkpointed step that must equal the plain one).
"""
import math

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import eisen_b200 as eb  # noqa: E402
from eisen_b200.graph import BF16_MIXED, Graph, TransformerLM  # noqa: E402


def dev():
    return torch.device("cuda:0")


def stream():
    return torch.cuda.current_stream().cuda_stream


def P(t):
    return t.data_ptr() if t is not None else None


def _rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def _attention(q, k, v, d_o, causal=True):
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    scale = 1.0 / math.sqrt(D)
    o = torch.full_like(q, float("nan"))
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device=dev())
    st = torch.zeros(1, dtype=torch.int32, device=dev())
    sq, sk = q.stride()[:3], k.stride()[:3]
    eb.call("eisen_attn_fwd", stream(), P(q), P(k), P(v), P(o), P(lse), B, S, Hq, Hkv, D, *sq, *sk, *sq, scale, int(causal), P(st))
    dq, dk, dv = torch.full_like(q, float("nan")), torch.full_like(k, float("nan")), torch.full_like(v, float("nan"))
    if d_o is not None:
        ws = torch.empty(eb.lib().eisen_attn_bwd_workspace_bytes(B, S, Hq, Hkv, D), dtype=torch.uint8, device=dev())
        eb.call("eisen_attn_bwd", stream(), P(q), P(k), P(v), P(o), P(lse), P(d_o), P(dq), P(dk), P(dv), P(ws),
                B, S, Hq, Hkv, D, *sq, *sk, *sq, scale, int(causal), P(st))
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    return o, lse, dq, dk, dv


@pytest.mark.parametrize("D", [128, 64])
def test_attention_full_geometry_sampled_groups(D):
    """Benchmark configs 3 and 5: batch 8, 32 query heads, 8 KV heads, seq 2048, causal.  Forward and
    backward run on the whole problem; two (batch, KV head) groups are checked against the materialised
    f32 chain of the same bf16 inputs (all four query heads of the group, since dK / dV sum over them)."""
    B, S, Hq, Hkv = 8, 2048, 32, 8
    g = torch.Generator(device=dev()).manual_seed(D)
    q, d_o = (torch.randn(B, S, Hq, D, generator=g, device=dev()).to(torch.bfloat16) for _ in range(2))
    k, v = (torch.randn(B, S, Hkv, D, generator=g, device=dev()).to(torch.bfloat16) for _ in range(2))
    o, lse, dq, dk, dv = _attention(q, k, v, d_o)
    assert torch.isfinite(o.float()).all() and torch.isfinite(dq.float()).all()
    assert torch.isfinite(dk.float()).all() and torch.isfinite(dv.float()).all()
    rep = Hq // Hkv
    scale = 1.0 / math.sqrt(D)
    mask = torch.triu(torch.full((S, S), float("-inf"), device=dev()), diagonal=1)
    for b, kvh in ((0, 0), (7, 5)):
        hs = slice(kvh * rep, (kvh + 1) * rep)
        qf = q[b, :, hs].float().requires_grad_(True)      # [S, rep, D]
        kf = k[b, :, kvh].float().requires_grad_(True)     # [S, D]
        vf = v[b, :, kvh].float().requires_grad_(True)
        s = torch.einsum("qhd,kd->hqk", qf, kf) * scale + mask
        p = torch.softmax(s, dim=-1)
        of = torch.einsum("hqk,kd->qhd", p, vf)
        of.backward(d_o[b, :, hs].float())
        assert _rel(o[b, :, hs].float(), of.detach()) < 1e-2
        assert (lse[b, hs].float() - torch.logsumexp(s, dim=-1).detach()).abs().max().item() < 2e-2
        assert _rel(dq[b, :, hs].float(), qf.grad) < 2e-2
        assert _rel(dk[b, :, kvh].float(), kf.grad) < 2e-2
        assert _rel(dv[b, :, kvh].float(), vf.grad) < 2e-2


def test_attention_full_geometry_zero_queries_average_the_values():
    """A property that needs no reference: with q = 0 every unmasked score is 0, so row s of the causal
    output is the mean of v[0..s] of its KV head and its log-sum-exp is ln(s + 1), at every one of the
    8 x 32 x 2048 rows."""
    B, S, Hq, Hkv, D = 8, 2048, 32, 8, 64
    g = torch.Generator(device=dev()).manual_seed(1)
    q = torch.zeros(B, S, Hq, D, dtype=torch.bfloat16, device=dev())
    k = torch.randn(B, S, Hkv, D, generator=g, device=dev()).to(torch.bfloat16)
    v = torch.randn(B, S, Hkv, D, generator=g, device=dev()).to(torch.bfloat16)
    o, lse, _, _, _ = _attention(q, k, v, None)
    counts = torch.arange(1, S + 1, device=dev(), dtype=torch.float32)
    mean_v = torch.cumsum(v.float(), dim=1) / counts.view(1, S, 1, 1)             # [B, S, Hkv, D]
    expect = mean_v.repeat_interleave(Hq // Hkv, dim=2)
    # P is rounded to bf16 before the P V product and O once more at the end
    assert (o.float() - expect).abs().max().item() < 2e-2
    assert _rel(o.float(), expect) < 6e-3
    assert (lse - torch.log(counts).view(1, 1, S)).abs().max().item() < 1e-3


def test_cross_entropy_and_head_gradient_full_size():
    """Benchmark config 4: 16384 tokens x vocab 32000 in bf16 with 5 % ignored targets: loss, dlogits (the
    two-kernel path and the fused in-place kernel) against f32 torch on the device, and the LM-head weight
    gradient X^T dlogits (2048 x 32000 x 16384, f32 atomic output, split left to the library)."""
    rows, vocab, d = 16384, 32000, 2048
    g = torch.Generator(device=dev()).manual_seed(4)
    logits = (1.5 * torch.randn(rows, vocab, generator=g, device=dev())).to(torch.bfloat16)
    t = torch.randint(0, vocab, (rows,), generator=g, device=dev(), dtype=torch.int32)
    t[torch.rand(rows, generator=g, device=dev()) < 0.05] = -1
    valid = int((t >= 0).sum().item())
    lf = logits.float()
    lse_ref = torch.logsumexp(lf, dim=-1)
    tl = t.clamp_min(0).long()
    picked = lf.gather(1, tl[:, None]).squeeze(1)
    prob_t = torch.exp(picked - lse_ref)
    row_ref = torch.where(t >= 0, -(prob_t + 1e-8).log(), torch.zeros_like(prob_t))   # -ln(p + 1e-8), src/graph/ops/reduction.rs:690
    loss_ref = row_ref.double().sum().item() / valid
    dl_ref = torch.softmax(lf, dim=-1)
    dl_ref[torch.arange(rows, device=dev()), tl] -= 1.0
    dl_ref *= (t >= 0).float()[:, None] / valid
    del lf
    loss = torch.zeros(1, device=dev())
    row_loss, lse = torch.empty(rows, device=dev()), torch.empty(rows, device=dev())
    flag = torch.zeros(1, dtype=torch.int32, device=dev())
    eb.call("eisen_ce_fwd", stream(), P(logits), P(t), P(loss), P(row_loss), P(lse), rows, vocab, -1, 1.0 / valid, eb.BF16, P(flag))
    dl = torch.empty_like(logits)
    eb.call("eisen_ce_bwd", stream(), P(logits), P(t), P(lse), P(dl), None, rows, vocab, -1, 1.0 / valid, eb.BF16, 0)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0
    assert abs(loss.item() - loss_ref) < 1e-3 * loss_ref
    assert (lse - lse_ref)[t >= 0].abs().max().item() < 2e-3  # ignored rows have no log-sum-exp
    assert _rel(dl.float(), dl_ref) < 1e-2
    assert (dl[t < 0].float() == 0).all()
    fused = logits.clone()
    row2 = torch.empty(rows, device=dev())
    eb.call("eisen_ce_fused", stream(), P(fused), P(t), None, P(row2), None, rows, vocab, -1, 1.0 / valid, 1.0, eb.BF16, P(flag))
    torch.cuda.synchronize()
    assert _rel(fused.float(), dl_ref) < 1e-2
    assert abs(row2.double().sum().item() - loss_ref) < 1e-3 * loss_ref
    del dl_ref, fused
    # head weight gradient from the bf16 dlogits: dW[d, vocab] += X^T dlogits
    x = torch.randn(rows, d, generator=g, device=dev()).to(torch.bfloat16)
    dw = torch.zeros(d, vocab, device=dev())
    st = torch.zeros(1, dtype=torch.int32, device=dev())
    eb.call("eisen_gemm_bf16", stream(), 1, 1, d, vocab, rows, P(x), d, P(dl), vocab, P(dw), vocab, 4, 0, 1.0, P(st))
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    ref = x.float().t() @ dl.float()
    assert _rel(dw, ref) < 1e-3  # the checker's f32 matmul may itself use reduced-precision accumulation paths


def test_rmsnorm_backward_full_size():
    """Benchmark config 4's side kernel: 16384 x 2048 in bf16, against f32 autograd on the device."""
    rows, dim = 16384, 2048
    g = torch.Generator(device=dev()).manual_seed(5)
    x = torch.randn(rows, dim, generator=g, device=dev()).to(torch.bfloat16)
    dy = torch.randn(rows, dim, generator=g, device=dev()).to(torch.bfloat16)
    w = 1.0 + 0.1 * torch.randn(dim, generator=g, device=dev())
    xf, wf = x.float().requires_grad_(True), w.clone().requires_grad_(True)
    y = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + 1e-5) * wf
    y.backward(dy.float())
    dx = torch.full_like(x, float("nan"))
    dw = torch.zeros(dim, device=dev())
    ws = torch.empty(eb.lib().eisen_rmsnorm_bwd_workspace_bytes(rows, dim), dtype=torch.uint8, device=dev())
    eb.call("eisen_rmsnorm_bwd", stream(), P(x), P(w), P(dy), P(dx), P(dw), P(ws), rows, dim, 1e-5, eb.BF16, 0)
    torch.cuda.synchronize()
    assert _rel(dx.float(), xf.grad) < 5e-3
    assert _rel(dw, wf.grad) < 1e-4


def test_adamw_full_size_flat_buffer():
    """Benchmark config 4's side kernel: one AdamW step over a 1.1e9-element f32 buffer (gradients N(0, 1e-3),
    clip coefficient from the fused squared norm); three slices of 4M elements (both ends and the middle,
    chosen to straddle 2^31 bytes of offset) are checked against the update formula in torch."""
    n = 1_100_000_000
    g = torch.Generator(device=dev()).manual_seed(6)
    w = torch.empty(n, device=dev()).normal_(0.0, 0.02, generator=g)
    gr = torch.empty(n, device=dev()).normal_(0.0, 1e-3, generator=g)
    m = torch.empty(n, device=dev()).normal_(0.0, 1e-4, generator=g)
    v = torch.empty(n, device=dev()).uniform_(0.0, 1e-6, generator=g)
    wb = torch.empty(n, dtype=torch.bfloat16, device=dev())
    ws = torch.empty(eb.lib().eisen_sumsq_workspace_bytes(n), dtype=torch.uint8, device=dev())
    ss = torch.zeros(1, dtype=torch.float64, device=dev())
    eb.call("eisen_sumsq", stream(), P(gr), n, P(ws), P(ss), 0)
    torch.cuda.synchronize()
    ref_ss = gr.double().pow(2).sum().item()
    assert abs(ss.item() - ref_ss) < 1e-9 * ref_ss
    lr, b1, b2, eps, wd, step, max_norm = 3e-4, 0.9, 0.95, 1e-8, 0.1, 7, 1.0
    bc1, bc2 = 1.0 / (1.0 - b1 ** step), 1.0 / (1.0 - b2 ** step)
    sl = [slice(0, 1 << 22), slice((1 << 29) - (1 << 21), (1 << 29) + (1 << 21)), slice(n - (1 << 22), n)]
    before = [(w[s].clone(), gr[s].clone(), m[s].clone(), v[s].clone()) for s in sl]
    eb.call("eisen_adamw_step", stream(), P(w), P(wb), P(gr), P(m), P(v), n, lr, b1, b2, eps, wd, bc1, bc2, 1.0, P(ss), max_norm)
    torch.cuda.synchronize()
    coef = min(max_norm / (math.sqrt(ref_ss) + 1e-6), 1.0)   # src/nn/optim.rs:283-287
    for s, (w0, g0, m0, v0) in zip(sl, before):
        g1 = g0 * coef
        m1 = b1 * m0 + (1 - b1) * g1
        v1 = b2 * v0 + (1 - b2) * g1 * g1
        w1 = w0 - lr * ((m1 * bc1) / (torch.sqrt(v1 * bc2) + eps) + wd * w0)
        assert _rel(m[s], m1) < 1e-6 and _rel(v[s], v1) < 1e-6
        assert _rel(w[s], w1) < 1e-6
        assert _rel(wb[s].float(), w1) < 4e-3


def test_headline_model_checkpointed_step_equals_plain_step():
    """Benchmark config 4's model (0.85B parameters, 16 blocks, 32 / 8 heads of 64, vocab 32000) on one
    2 x 2048 batch.  Per-block checkpointing re-runs each block's forward pass, which reproduces it bit for
    bit, so in the fixed-order mode the plain step, a second plain step, the checkpointed step and the variant
    that keeps the attention outputs all give identical gradient bits.  In the default mode (atomic adds in
    split-K weight gradients and in dQ) two runs of the very same step already differ: the 1e-6 differences
    of the last block are amplified by every bf16 rounding of an activation gradient on the way down, up to
    the size of the rounding error itself in the first blocks; the modes must agree within that."""
    B, S = 2, 2048
    rng = np.random.default_rng(8)
    ids = rng.integers(0, 32000, (B, S)).astype(np.int32)
    tg = rng.integers(0, 32000, B * S).tolist()
    g = Graph(BF16_MIXED, torch.cuda.current_stream().cuda_stream)
    lm = TransformerLM(g, 32000, 2048, 32, 8, 5632, 16, False)
    g.mark_params()
    ps = lm.params()
    probe = [ps[0], ps[2], ps[3], ps[1 + 9 * 7 + 4], ps[1 + 9 * 15 + 8], ps[-1]]  # embedding, q / k of block 0, o of block 7, gate of block 15, head

    def run(mode):
        for p in ps:
            g.zero_grad_tensor(p)
        lm.set_keep_attention(mode == "keep_attention")
        x = g.alloc_ids([B, S], ids)
        loss = lm.train_micro_step(x, tg, checkpoint=(mode != "plain"))
        out = (float(g.data(loss)[0]), [torch.from_numpy(g.grad(p)) for p in probe])
        g.clear_activations()
        lm.set_keep_attention(False)
        return out

    eb.call("eisen_set_deterministic", 1)
    try:
        l0, g0 = run("plain")
        assert math.isfinite(l0) and abs(l0 - math.log(32000)) < 0.5   # random weights: close to ln(vocab)
        for mode in ("plain", "checkpoint", "keep_attention"):
            l1, g1 = run(mode)
            assert l1 == l0
            for a, b in zip(g1, g0):
                assert torch.equal(a, b), mode
    finally:
        eb.call("eisen_set_deterministic", 0)
    for mode in ("plain", "checkpoint"):
        l1, g1 = run(mode)
        assert abs(l1 - l0) <= 1e-6 * abs(l0)
        for a, b in zip(g1, g0):
            assert torch.isfinite(a).all()
            assert _rel(a, b) < 2e-2
