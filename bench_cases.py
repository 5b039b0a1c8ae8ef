"""Single-kernel cases for timing and profiling one entry point of the C ABI at a time.

    python bench_cases.py gemm --m 8192 --n 5632 --k 2048 --a-mn 0 --b-mn 1 --out-mode 0
    python bench_cases.py gemm_swiglu --m 16384 --n 5632 --k 2048 --out-mode 1
    python bench_cases.py attn --batch 2 --seq 2048 --heads 8 --kv-heads 2 --head-dim 64
    python bench_cases.py ce --rows 4096 --vocab 32000
    python bench_cases.py rmsnorm --rows 16384 --dim 2048
    python bench_cases.py adamw --nelem 100000000

Each case allocates seeded inputs, runs `--iters` launches (default 3, so that a profiler capture
stays short) and returns / prints one JSON object with the CUDA-event time per launch and the
achieved algorithmic rate.  A case whose buffers would fit the 126 MB L2 rotates through several
buffer sets (`--sets`, default: enough sets to cover 3 x L2) so that no launch re-reads what the
one before left in the cache.  bench.py calls the same functions for the per-kernel entries of
its JSON line.
"""
import argparse
import json
import math
import sys
import os

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import eisen_b200 as eb  # noqa: E402

L2_BYTES = 126 * 1024 * 1024


def P(t):
    return t.data_ptr() if t is not None else None


def n_sets_for(bytes_per_set, requested=0):
    """Buffer sets to rotate through so that consecutive launches do not hit in L2."""
    if requested > 0:
        return requested
    if bytes_per_set >= 3 * L2_BYTES:
        return 1
    return max(2, min(12, math.ceil(3 * L2_BYTES / max(1, bytes_per_set))))


def timed(fns, iters, warmup=1):
    """fns: one callable or a list of callables (one per buffer set), called round-robin.
    Returns milliseconds per call (CUDA events on the current stream)."""
    if callable(fns):
        fns = [fns]
    for i in range(max(warmup, len(fns) if warmup else 0)):
        fns[i % len(fns)]()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fns[i % len(fns)]()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _ctx():
    dev = torch.device("cuda", torch.cuda.current_device())
    return dev, torch.cuda.current_stream().cuda_stream, torch.zeros(1, dtype=torch.int32, device=dev)


def case_gemm(M, N, K, a_mn=0, b_mn=1, out_mode=0, split_k=0, iters=3, sets=0):
    dev, s, st = _ctx()
    osz = 2 if out_mode < 2 else 4
    ns = n_sets_for(2 * (M * K + N * K) + osz * M * N, sets)
    fns = []
    keep = []
    for _ in range(ns):
        A = torch.randn((K, M) if a_mn else (M, K), device=dev).to(torch.bfloat16)
        B = torch.randn((K, N) if b_mn else (N, K), device=dev).to(torch.bfloat16)
        C = torch.zeros(M, N, device=dev, dtype=torch.bfloat16 if out_mode < 2 else torch.float32)
        keep.append((A, B, C))
        fns.append(lambda A=A, B=B, C=C: eb.call("eisen_gemm_bf16", s, a_mn, b_mn, M, N, K, P(A), A.stride(0), P(B),
                                                  B.stride(0), P(C), N, out_mode, split_k, 1.0, P(st)))
    ms = timed(fns, iters)
    return dict(ms=ms, tflops=2.0 * M * N * K / ms / 1e9, flops=2.0 * M * N * K, shape=[M, N, K], sets=ns, status=int(st.item()))


def case_gemm_swiglu(M, N, K, keep_gate_up=True, iters=3):
    # gate / up projections + SwiGLU in one launch; keep_gate_up keeps G and U (a pass that is
    # followed by a backward pass), otherwise H only is written
    dev, s, st = _ctx()
    A = torch.randn(M, K, device=dev).to(torch.bfloat16)
    Wg, Wu = ((torch.randn(K, N, device=dev) * 0.05).to(torch.bfloat16) for _ in range(2))
    G, U, H = (torch.empty(M, N, device=dev, dtype=torch.bfloat16) for _ in range(3))
    ms = timed(lambda: eb.call("eisen_gemm_bf16_swiglu", s, M, N, K, P(A), K, P(Wg), P(Wu), N,
                               P(G) if keep_gate_up else None, P(U) if keep_gate_up else None, P(H), N, P(st)), iters)
    return dict(ms=ms, tflops=4.0 * M * N * K / ms / 1e9, shape=[M, N, K], keep_gate_up=keep_gate_up, status=int(st.item()))


def case_gemm_rope(M, N, K, seq, head_dim, iters=3, sets=0):
    # q / k projection with the RoPE rotation in the epilogue, beside the plain projection of the same shape
    dev, s, st = _ctx()
    ns = n_sets_for(2 * (M * K + N * K + M * N), sets)
    tab = torch.empty(seq * (head_dim // 2) * 2, device=dev)
    eb.call("eisen_rope_table", s, P(tab), seq, head_dim, 10000.0)
    fr, fp, keep = [], [], []
    for _ in range(ns):
        A = torch.randn(M, K, device=dev).to(torch.bfloat16)
        B = (torch.randn(K, N, device=dev) * 0.05).to(torch.bfloat16)
        C = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        keep.append((A, B, C))
        fr.append(lambda A=A, B=B, C=C: eb.call("eisen_gemm_bf16_rope", s, M, N, K, P(A), K, P(B), N, P(C), N, P(tab), seq,
                                                head_dim, P(st)))
        fp.append(lambda A=A, B=B, C=C: eb.call("eisen_gemm_bf16", s, 0, 1, M, N, K, P(A), K, P(B), N, P(C), N, 0, 0, 1.0, P(st)))
    mr = timed(fr, iters)
    mp = timed(fp, iters)
    fl = 2.0 * M * N * K
    return dict(rope_ms=mr, rope_tflops=fl / mr / 1e9, plain_ms=mp, plain_tflops=fl / mp / 1e9, shape=[M, N, K], sets=ns,
                status=int(st.item()))


def case_qkv_bwd(M, d, nq, nkv, iters=3):
    # backward of the q / k / v projections of one input: three launches per product against the
    # K-segmented (dX) and N-segmented (dW) single launches
    import ctypes
    dev, s, st = _ctx()
    Ns = [nq, nkv, nkv]
    X = torch.randn(M, d, device=dev).to(torch.bfloat16)
    dYs = [torch.randn(M, n, device=dev).to(torch.bfloat16) for n in Ns]
    Ws = [(torch.randn(d, n, device=dev) * 0.05).to(torch.bfloat16) for n in Ns]
    dX = torch.empty(M, d, device=dev, dtype=torch.bfloat16)
    dWs = [torch.zeros(d, n, device=dev) for n in Ns]
    pa = lambda ts: (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
    la = lambda vs: (ctypes.c_longlong * len(vs))(*vs)

    def dx_separate():
        # dV first (store), then dK and dQ accumulate, as the tape walks them
        for i, mode in ((2, 0), (1, 1), (0, 1)):
            eb.call("eisen_gemm_bf16", s, 0, 0, M, d, Ns[i], P(dYs[i]), Ns[i], P(Ws[i]), Ns[i], P(dX), d, mode, 1, 1.0, P(st))

    def dx_fused():
        eb.call("eisen_gemm_bf16_concat_k", s, 0, 0, M, d, 3, pa(dYs), la(Ns), pa(Ws), la(Ns), la(Ns), P(dX), d, 0, 1, 1.0, P(st))

    def dw_separate():
        for i in range(3):
            eb.call("eisen_gemm_bf16", s, 1, 1, d, Ns[i], M, P(X), d, P(dYs[i]), Ns[i], P(dWs[i]), Ns[i], 4, 0, 1.0, P(st))

    modes = (ctypes.c_int * 3)(4, 4, 4)

    def dw_fused():
        eb.call("eisen_gemm_bf16_multi_n", s, 1, 1, d, M, P(X), d, 3, pa(dYs), la(Ns), la(Ns), pa(dWs), la(Ns), modes, 0, 1.0,
                None, 0, 0, P(st))

    fl = 2.0 * M * d * sum(Ns)
    out = {}
    for name, fn in (("dx_separate", dx_separate), ("dx_fused", dx_fused), ("dw_separate", dw_separate), ("dw_fused", dw_fused)):
        ms = timed(fn, iters)
        out[name] = dict(ms=ms, tflops=fl / ms / 1e9)
    out["status"] = int(st.item())
    out["shape"] = dict(tokens=M, d=d, nq=nq, nkv=nkv)
    return out


def case_attn(B_, S, Hq, Hkv, D, iters=3, sets=0):
    dev, s, st = _ctx()
    per_set = 2 * B_ * S * D * (4 * Hq + 4 * Hkv)
    ns = n_sets_for(per_set, sets)
    sc = 1.0 / math.sqrt(D)
    ws = torch.empty(eb.lib().eisen_attn_bwd_workspace_bytes(B_, S, Hq, Hkv, D), dtype=torch.uint8, device=dev)
    ff, fb, keep = [], [], []
    for _ in range(ns):
        q = torch.randn(B_, S, Hq, D, device=dev).to(torch.bfloat16)
        k = torch.randn(B_, S, Hkv, D, device=dev).to(torch.bfloat16)
        v = torch.randn(B_, S, Hkv, D, device=dev).to(torch.bfloat16)
        do = torch.randn(B_, S, Hq, D, device=dev).to(torch.bfloat16)
        o = torch.empty_like(q)
        lse = torch.empty(B_, Hq, S, device=dev)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        keep.append((q, k, v, do, o, lse, dq, dk, dv))
        qs, ks, os_ = q.stride()[:3], k.stride()[:3], o.stride()[:3]
        ff.append(lambda q=q, k=k, v=v, o=o, lse=lse, qs=qs, ks=ks, os_=os_: eb.call(
            "eisen_attn_fwd", s, P(q), P(k), P(v), P(o), P(lse), B_, S, Hq, Hkv, D, *qs, *ks, *os_, sc, 1, P(st)))
        fb.append(lambda q=q, k=k, v=v, o=o, lse=lse, do=do, dq=dq, dk=dk, dv=dv, qs=qs, ks=ks, os_=os_: eb.call(
            "eisen_attn_bwd", s, P(q), P(k), P(v), P(o), P(lse), P(do), P(dq), P(dk), P(dv), P(ws), B_, S, Hq, Hkv, D,
            *qs, *ks, *os_, sc, 1, P(st)))
    mf = timed(ff, iters)
    mb = timed(fb, iters)
    fl = 4.0 * B_ * Hq * S * S * D / 2
    return dict(fwd_ms=mf, fwd_tflops=fl / mf / 1e9, bwd_ms=mb, bwd_tflops=2.5 * fl / mb / 1e9, fwd_flops=fl,
                bwd_flops=2.5 * fl, shape=dict(B=B_, S=S, Hq=Hq, Hkv=Hkv, D=D, causal=True), sets=ns, status=int(st.item()))


def case_ce(rows, V, iters=3, ignore_frac=0.0):
    dev, s, st = _ctx()
    lg = torch.randn(rows, V, device=dev).to(torch.bfloat16)
    t = torch.randint(0, V, (rows,), device=dev, dtype=torch.int32)
    if ignore_frac > 0:
        t[torch.rand(rows, device=dev) < ignore_frac] = -1
    loss, rl, lse = torch.zeros(1, device=dev), torch.empty(rows, device=dev), torch.empty(rows, device=dev)
    dl = torch.empty_like(lg)
    nv = max(1, int((t >= 0).sum().item()))
    mf = timed(lambda: eb.call("eisen_ce_fwd", s, P(lg), P(t), P(loss), P(rl), P(lse), rows, V, -1, 1.0 / nv, eb.BF16, None), iters)
    mb = timed(lambda: eb.call("eisen_ce_bwd", s, P(lg), P(t), P(lse), P(dl), None, rows, V, -1, 1.0 / nv, eb.BF16, 0), iters)
    # forward and backward in one launch, in place (the logits are refilled before every launch)
    lg2 = [lg.clone() for _ in range(2)]
    mfu = timed([lambda x=x: eb.call("eisen_ce_fused", s, P(x), P(t), P(loss), P(rl), P(lse), rows, V, -1, 1.0 / nv, 1.0, eb.BF16, None)
                 for x in lg2], iters)
    fb, bb = rows * V * 2 + rows * 8, rows * V * 4 + rows * 8
    return dict(fused_ms=mfu, fused_gbs=(rows * V * 4 + rows * 8) / mfu / 1e6, fused_bytes=rows * V * 4 + rows * 8, fwd_ms=mf, fwd_gbs=fb / mf / 1e6, fwd_bytes=fb, bwd_ms=mb, bwd_gbs=bb / mb / 1e6, bwd_bytes=bb,
                shape=[rows, V], ignored_rows=rows - nv)


def case_rmsnorm(rows, dim, iters=3, sets=0):
    dev, s, st = _ctx()
    ns = n_sets_for(rows * dim * 6, sets)
    w = torch.ones(dim, device=dev)
    dw = torch.zeros(dim, device=dev)
    ws = torch.empty(eb.lib().eisen_rmsnorm_bwd_workspace_bytes(rows, dim), dtype=torch.uint8, device=dev)
    ff, fb, keep = [], [], []
    for _ in range(ns):
        x = torch.randn(rows, dim, device=dev).to(torch.bfloat16)
        dy = torch.randn(rows, dim, device=dev).to(torch.bfloat16)
        y, dx = torch.empty_like(x), torch.empty_like(x)
        keep.append((x, dy, y, dx))
        ff.append(lambda x=x, y=y: eb.call("eisen_rmsnorm_fwd", s, P(x), P(w), P(y), None, rows, dim, 1e-5, eb.BF16))
        fb.append(lambda x=x, dy=dy, dx=dx: eb.call("eisen_rmsnorm_bwd", s, P(x), P(w), P(dy), P(dx), P(dw), P(ws), rows, dim,
                                                     1e-5, eb.BF16, 0))
    mf = timed(ff, iters)
    mb = timed(fb, iters)
    bb = rows * dim * 6 + 8 * dim
    return dict(fwd_ms=mf, fwd_gbs=rows * dim * 4 / mf / 1e6, bwd_ms=mb, bwd_gbs=bb / mb / 1e6, bwd_bytes=bb,
                shape=[rows, dim], sets=ns)


def case_swiglu(rows, dim, iters=3, sets=0):
    dev, s, st = _ctx()
    n = rows * dim
    ns = n_sets_for(n * 10, sets)
    ff, fb, keep = [], [], []
    for _ in range(ns):
        g_, u_, dh = (torch.randn(n, device=dev).to(torch.bfloat16) for _ in range(3))
        h, dg, du = torch.empty_like(g_), torch.empty_like(g_), torch.empty_like(g_)
        keep.append((g_, u_, dh, h, dg, du))
        ff.append(lambda g_=g_, u_=u_, h=h: eb.call("eisen_swiglu_fwd", s, P(g_), P(u_), P(h), n, eb.BF16))
        fb.append(lambda g_=g_, u_=u_, dh=dh, dg=dg, du=du: eb.call("eisen_swiglu_bwd", s, P(g_), P(u_), P(dh), P(dg), P(du), n, eb.BF16, 0))
    mf = timed(ff, iters)
    mb = timed(fb, iters)
    return dict(fwd_ms=mf, fwd_gbs=n * 6 / mf / 1e6, bwd_ms=mb, bwd_gbs=n * 10 / mb / 1e6, bwd_bytes=n * 10, shape=[rows, dim], sets=ns)


def case_adamw(n, iters=3):
    dev, s, st = _ctx()
    w, g_, m, v = (torch.randn(n, device=dev) * 1e-3 for _ in range(4))
    v.abs_()
    wb = torch.empty(n, dtype=torch.bfloat16, device=dev)
    ms = timed(lambda: eb.call("eisen_adamw_step", s, P(w), P(wb), P(g_), P(m), P(v), n, 3e-4, 0.9, 0.95, 1e-8, 0.1,
                               10.0, 20.0, 1.0, None, 0.0), iters)
    return dict(ms=ms, gbs=n * 30 / ms / 1e6, bytes=n * 30, n=n)


def case_elementwise(rows, dim, seq, head_dim, vocab, nelem, iters=3, sets=0):
    # residual add, gradient accumulate, RoPE forward / backward, embedding gather / scatter, squared norm
    dev, s, st = _ctx()
    out = {}
    n = rows * dim
    ns = n_sets_for(n * 6, sets)
    xs = [torch.randn(n, device=dev).to(torch.bfloat16) for _ in range(ns)]
    ys = [torch.randn(n, device=dev).to(torch.bfloat16) for _ in range(ns)]
    os_ = [torch.empty_like(xs[0]) for _ in range(ns)]
    ms = timed([lambda x=x, y=y, o=o: eb.call("eisen_add", s, P(x), P(y), P(o), n, n, eb.BF16) for x, y, o in zip(xs, ys, os_)], iters)
    out["add_gbs"] = n * 6 / ms / 1e6
    ms = timed([lambda x=x, o=o: eb.call("eisen_accumulate", s, P(o), eb.BF16, P(x), eb.BF16, n, 1) for x, o in zip(xs, os_)], iters)
    out["accumulate_gbs"] = n * 6 / ms / 1e6
    tab = torch.empty(seq, head_dim // 2, 2, device=dev)
    eb.call("eisen_rope_table", s, P(tab), seq, head_dim, 10000.0)
    ms = timed([lambda x=x, o=o: eb.call("eisen_rope", s, P(x), P(o), P(tab), rows // seq, seq, dim, head_dim, eb.BF16, 0, 0) for x, o in zip(xs, os_)], iters)
    out["rope_fwd_gbs"] = n * 4 / ms / 1e6
    ms = timed([lambda x=x, o=o: eb.call("eisen_rope", s, P(x), P(o), P(tab), rows // seq, seq, dim, head_dim, eb.BF16, 1, 0) for x, o in zip(xs, os_)], iters)
    out["rope_bwd_gbs"] = n * 4 / ms / 1e6
    table = torch.randn(vocab, dim, device=dev).to(torch.bfloat16)
    ids = torch.randint(0, vocab, (rows,), device=dev, dtype=torch.int32)
    ms = timed([lambda o=o: eb.call("eisen_embedding_fwd", s, P(table), eb.BF16, P(ids), P(o), eb.BF16, rows, dim, vocab, None) for o in os_], iters)
    out["embedding_fwd_gbs"] = (n * 4 + rows * 4) / ms / 1e6
    dw = torch.zeros(vocab, dim, device=dev)
    ws = torch.empty(eb.lib().eisen_embedding_bwd_workspace_bytes(rows, vocab), dtype=torch.uint8, device=dev)
    ms = timed([lambda x=x: eb.call("eisen_embedding_bwd", s, P(x), eb.BF16, P(ids), P(dw), P(ws), rows, dim, vocab) for x in xs], iters)
    touched = len(torch.unique(ids))
    out["embedding_bwd_gbs"] = (n * 2 + touched * dim * 8 + rows * 4) / ms / 1e6
    out["embedding_bwd_ms"] = ms
    ms = timed([lambda x=x: eb.call("eisen_embedding_bwd_apply", s, P(x), eb.BF16, P(dw), P(ws), rows, dim, vocab) for x in xs], iters)
    out["embedding_bwd_apply_gbs"] = (n * 2 + touched * dim * 8 + rows * 4) / ms / 1e6
    out["embedding_bwd_apply_ms"] = ms
    g32 = torch.randn(nelem, device=dev)
    ws2 = torch.empty(eb.lib().eisen_sumsq_workspace_bytes(nelem), dtype=torch.uint8, device=dev)
    ss = torch.zeros(1, dtype=torch.float64, device=dev)
    ms = timed(lambda: eb.call("eisen_sumsq", s, P(g32), nelem, P(ws2), P(ss), 0), iters)
    out["sumsq_gbs"] = nelem * 4 / ms / 1e6
    out["sets"] = ns
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "gemm_swiglu", "gemm_rope", "qkv_bwd", "attn", "ce", "rmsnorm", "adamw", "swiglu", "elementwise"])
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--sets", type=int, default=0, help="buffer sets to rotate through (0: enough to cover 3 x L2)")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=5632)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--a-mn", type=int, default=0)
    ap.add_argument("--b-mn", type=int, default=1)
    ap.add_argument("--out-mode", type=int, default=0)
    ap.add_argument("--split-k", type=int, default=0)
    ap.add_argument("--gemm-mode", type=int, default=-1, help="eisen_gemm_set_mode value (default: leave as is)")
    ap.add_argument("--fwd-tiles", type=int, default=0, help="eisen_attn_set_fwd_tiles value (default: leave as is)")
    ap.add_argument("--bwd-mode", type=int, default=-1, help="eisen_attn_set_bwd_mode value (default: leave as is)")
    ap.add_argument("--rms-bwd-mode", type=int, default=-1, help="eisen_rmsnorm_bwd_set_mode value (default: leave as is)")
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=2)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--dim", type=int, default=2048)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--nelem", type=int, default=100_000_000)
    a = ap.parse_args()
    torch.cuda.set_device(0)
    torch.manual_seed(0)
    if a.gemm_mode >= 0:
        eb.call("eisen_gemm_set_mode", a.gemm_mode)
    if a.fwd_tiles > 0:
        eb.call("eisen_attn_set_fwd_tiles", a.fwd_tiles)
    if a.bwd_mode >= 0:
        eb.call("eisen_attn_set_bwd_mode", a.bwd_mode)
    if a.rms_bwd_mode >= 0:
        eb.call("eisen_rmsnorm_bwd_set_mode", a.rms_bwd_mode)
    if a.case == "gemm":
        out = case_gemm(a.m, a.n, a.k, a.a_mn, a.b_mn, a.out_mode, a.split_k, a.iters, a.sets)
    elif a.case == "gemm_swiglu":
        out = case_gemm_swiglu(a.m, a.n, a.k, a.out_mode == 1, a.iters)
    elif a.case == "gemm_rope":
        out = case_gemm_rope(a.m, a.n, a.k, a.seq, a.head_dim, a.iters, a.sets)
    elif a.case == "qkv_bwd":
        out = case_qkv_bwd(a.rows, a.dim, a.n, a.k, a.iters)
    elif a.case == "attn":
        out = case_attn(a.batch, a.seq, a.heads, a.kv_heads, a.head_dim, a.iters, a.sets)
    elif a.case == "ce":
        out = case_ce(a.rows, a.vocab, a.iters)
    elif a.case == "rmsnorm":
        out = case_rmsnorm(a.rows, a.dim, a.iters, a.sets)
    elif a.case == "swiglu":
        out = case_swiglu(a.rows, a.dim, a.iters, a.sets)
    elif a.case == "elementwise":
        out = case_elementwise(a.rows, a.dim, a.seq, a.head_dim, a.vocab, a.nelem, a.iters, a.sets)
    else:
        out = case_adamw(a.nelem, a.iters)
    out["case"] = a.case
    print(json.dumps(out))


if __name__ == "__main__":
    main()
