"""Single-kernel cases for timing and profiling one entry point of the C ABI at a time.

    python -m eisen_b200.cases gemm --m 8192 --n 5632 --k 2048 --a-mn 0 --b-mn 1 --out-mode 0
    python -m eisen_b200.cases gemm_swiglu --m 16384 --n 5632 --k 2048 --out-mode 1
    python -m eisen_b200.cases attn --batch 2 --seq 2048 --heads 8 --kv-heads 2 --head-dim 64
    python -m eisen_b200.cases ce --rows 4096 --vocab 32000
    python -m eisen_b200.cases rmsnorm --rows 16384 --dim 2048
    python -m eisen_b200.cases adamw --n 100000000

Each case allocates seeded inputs larger than L2 where the sizes allow, runs `--iters` launches
(default 3, so that a profiler capture stays short) and prints one JSON line with the CUDA-event
time per launch and the achieved algorithmic rate.
"""
import argparse
import json
import math

import torch

import eisen_b200 as eb


def P(t):
    return t.data_ptr() if t is not None else None


def timed(fn, iters, warmup=1):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "gemm_swiglu", "attn", "ce", "rmsnorm", "adamw", "swiglu", "elementwise"])
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=5632)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--a-mn", type=int, default=0)
    ap.add_argument("--b-mn", type=int, default=1)
    ap.add_argument("--out-mode", type=int, default=0)
    ap.add_argument("--split-k", type=int, default=0)
    ap.add_argument("--gemm-mode", type=int, default=-1, help="eisen_gemm_set_mode value (default: leave as is)")
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
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    s = torch.cuda.current_stream().cuda_stream
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    out = {"case": a.case}
    if a.gemm_mode >= 0:
        eb.call("eisen_gemm_set_mode", a.gemm_mode)
    if a.case == "gemm":
        M, N, K = a.m, a.n, a.k
        A = torch.randn((K, M) if a.a_mn else (M, K), device=dev).to(torch.bfloat16)
        B = torch.randn((K, N) if a.b_mn else (N, K), device=dev).to(torch.bfloat16)
        C = torch.zeros(M, N, device=dev, dtype=torch.bfloat16 if a.out_mode < 2 else torch.float32)
        ms = timed(lambda: eb.call("eisen_gemm_bf16", s, a.a_mn, a.b_mn, M, N, K, P(A), A.stride(0), P(B), B.stride(0),
                                   P(C), N, a.out_mode, a.split_k, 1.0, P(st)), a.iters)
        out.update(ms=ms, tflops=2.0 * M * N * K / ms / 1e9, shape=[M, N, K])
    elif a.case == "gemm_swiglu":
        # gate / up projections + SwiGLU in one launch; --out-mode 1 keeps G and U (a pass that is
        # followed by a backward pass), 0 writes H only
        M, N, K = a.m, a.n, a.k
        A = torch.randn(M, K, device=dev).to(torch.bfloat16)
        Wg, Wu = ((torch.randn(K, N, device=dev) * 0.05).to(torch.bfloat16) for _ in range(2))
        G, U, H = (torch.empty(M, N, device=dev, dtype=torch.bfloat16) for _ in range(3))
        keep = a.out_mode == 1
        ms = timed(lambda: eb.call("eisen_gemm_bf16_swiglu", s, M, N, K, P(A), K, P(Wg), P(Wu), N,
                                   P(G) if keep else None, P(U) if keep else None, P(H), N, P(st)), a.iters)
        out.update(ms=ms, tflops=4.0 * M * N * K / ms / 1e9, shape=[M, N, K], keep_gate_up=keep)
    elif a.case == "attn":
        B_, S, Hq, Hkv, D = a.batch, a.seq, a.heads, a.kv_heads, a.head_dim
        q = torch.randn(B_, S, Hq, D, device=dev).to(torch.bfloat16)
        k = torch.randn(B_, S, Hkv, D, device=dev).to(torch.bfloat16)
        v = torch.randn(B_, S, Hkv, D, device=dev).to(torch.bfloat16)
        do = torch.randn(B_, S, Hq, D, device=dev).to(torch.bfloat16)
        o = torch.empty_like(q)
        lse = torch.empty(B_, Hq, S, device=dev)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        ws = torch.empty(eb.lib().eisen_attn_bwd_workspace_bytes(B_, S, Hq, Hkv, D), dtype=torch.uint8, device=dev)
        sc = 1.0 / math.sqrt(D)
        qs, ks, os_ = q.stride()[:3], k.stride()[:3], o.stride()[:3]
        mf = timed(lambda: eb.call("eisen_attn_fwd", s, P(q), P(k), P(v), P(o), P(lse), B_, S, Hq, Hkv, D, *qs, *ks, *os_,
                                   sc, 1, P(st)), a.iters)
        mb = timed(lambda: eb.call("eisen_attn_bwd", s, P(q), P(k), P(v), P(o), P(lse), P(do), P(dq), P(dk), P(dv), P(ws),
                                   B_, S, Hq, Hkv, D, *qs, *ks, *os_, sc, 1, P(st)), a.iters)
        fl = 4.0 * B_ * Hq * S * S * D / 2
        out.update(fwd_ms=mf, fwd_tflops=fl / mf / 1e9, bwd_ms=mb, bwd_tflops=2.5 * fl / mb / 1e9)
    elif a.case == "ce":
        rows, V = a.rows, a.vocab
        lg = torch.randn(rows, V, device=dev).to(torch.bfloat16)
        t = torch.randint(0, V, (rows,), device=dev, dtype=torch.int32)
        loss, rl, lse = torch.zeros(1, device=dev), torch.empty(rows, device=dev), torch.empty(rows, device=dev)
        dl = torch.empty_like(lg)
        mf = timed(lambda: eb.call("eisen_ce_fwd", s, P(lg), P(t), P(loss), P(rl), P(lse), rows, V, -1, 1.0 / rows, eb.BF16, None), a.iters)
        mb = timed(lambda: eb.call("eisen_ce_bwd", s, P(lg), P(t), P(lse), P(dl), None, rows, V, -1, 1.0 / rows, eb.BF16, 0), a.iters)
        out.update(fwd_ms=mf, fwd_gbs=(rows * V * 2 + rows * 8) / mf / 1e6, bwd_ms=mb, bwd_gbs=(rows * V * 4 + rows * 8) / mb / 1e6)
    elif a.case == "rmsnorm":
        rows, dim = a.rows, a.dim
        x = torch.randn(rows, dim, device=dev).to(torch.bfloat16)
        dy = torch.randn(rows, dim, device=dev).to(torch.bfloat16)
        w = torch.ones(dim, device=dev)
        y, dx, dw = torch.empty_like(x), torch.empty_like(x), torch.zeros(dim, device=dev)
        ws = torch.empty(eb.lib().eisen_rmsnorm_bwd_workspace_bytes(rows, dim), dtype=torch.uint8, device=dev)
        mf = timed(lambda: eb.call("eisen_rmsnorm_fwd", s, P(x), P(w), P(y), None, rows, dim, 1e-5, eb.BF16), a.iters)
        mb = timed(lambda: eb.call("eisen_rmsnorm_bwd", s, P(x), P(w), P(dy), P(dx), P(dw), P(ws), rows, dim, 1e-5, eb.BF16, 0), a.iters)
        out.update(fwd_ms=mf, fwd_gbs=rows * dim * 4 / mf / 1e6, bwd_ms=mb, bwd_gbs=(rows * dim * 6 + 8 * dim) / mb / 1e6)
    elif a.case == "swiglu":
        n = a.rows * a.dim
        g_, u_, dh = (torch.randn(n, device=dev).to(torch.bfloat16) for _ in range(3))
        h, dg, du = torch.empty_like(g_), torch.empty_like(g_), torch.empty_like(g_)
        mf = timed(lambda: eb.call("eisen_swiglu_fwd", s, P(g_), P(u_), P(h), n, eb.BF16), a.iters)
        mb = timed(lambda: eb.call("eisen_swiglu_bwd", s, P(g_), P(u_), P(dh), P(dg), P(du), n, eb.BF16, 0), a.iters)
        out.update(fwd_ms=mf, fwd_gbs=n * 6 / mf / 1e6, bwd_ms=mb, bwd_gbs=n * 10 / mb / 1e6)
    elif a.case == "elementwise":
        # residual add, gradient accumulate, RoPE forward / backward, embedding gather / scatter, squared norm
        rows, dim = a.rows, a.dim
        n = rows * dim
        x, y = (torch.randn(n, device=dev).to(torch.bfloat16) for _ in range(2))
        o = torch.empty_like(x)
        ms = timed(lambda: eb.call("eisen_add", s, P(x), P(y), P(o), n, n, eb.BF16), a.iters)
        out["add_gbs"] = n * 6 / ms / 1e6
        ms = timed(lambda: eb.call("eisen_accumulate", s, P(o), eb.BF16, P(x), eb.BF16, n, 1), a.iters)
        out["accumulate_gbs"] = n * 6 / ms / 1e6
        S, hd = a.seq, a.head_dim
        tab = torch.empty(S, hd // 2, 2, device=dev)
        eb.call("eisen_rope_table", s, P(tab), S, hd, 10000.0)
        ms = timed(lambda: eb.call("eisen_rope", s, P(x), P(o), P(tab), rows // S, S, dim, hd, eb.BF16, 0, 0), a.iters)
        out["rope_fwd_gbs"] = n * 4 / ms / 1e6
        ms = timed(lambda: eb.call("eisen_rope", s, P(x), P(o), P(tab), rows // S, S, dim, hd, eb.BF16, 1, 0), a.iters)
        out["rope_bwd_gbs"] = n * 4 / ms / 1e6
        V = a.vocab
        table = torch.randn(V, dim, device=dev).to(torch.bfloat16)
        ids = torch.randint(0, V, (rows,), device=dev, dtype=torch.int32)
        ms = timed(lambda: eb.call("eisen_embedding_fwd", s, P(table), eb.BF16, P(ids), P(o), eb.BF16, rows, dim, V, None), a.iters)
        out["embedding_fwd_gbs"] = (n * 4 + rows * 4) / ms / 1e6
        dw = torch.zeros(V, dim, device=dev)
        ws = torch.empty(eb.lib().eisen_embedding_bwd_workspace_bytes(rows, V), dtype=torch.uint8, device=dev)
        ms = timed(lambda: eb.call("eisen_embedding_bwd", s, P(x), eb.BF16, P(ids), P(dw), P(ws), rows, dim, V), a.iters)
        touched = len(torch.unique(ids))
        out["embedding_bwd_gbs"] = (n * 2 + touched * dim * 8 + rows * 4) / ms / 1e6
        out["embedding_bwd_ms"] = ms
        ms = timed(lambda: eb.call("eisen_embedding_bwd_apply", s, P(x), eb.BF16, P(dw), P(ws), rows, dim, V), a.iters)
        out["embedding_bwd_apply_gbs"] = (n * 2 + touched * dim * 8 + rows * 4) / ms / 1e6
        out["embedding_bwd_apply_ms"] = ms
        g32 = torch.randn(a.nelem, device=dev)
        ws2 = torch.empty(eb.lib().eisen_sumsq_workspace_bytes(a.nelem), dtype=torch.uint8, device=dev)
        ss = torch.zeros(1, dtype=torch.float64, device=dev)
        ms = timed(lambda: eb.call("eisen_sumsq", s, P(g32), a.nelem, P(ws2), P(ss), 0), a.iters)
        out["sumsq_gbs"] = a.nelem * 4 / ms / 1e6
    else:
        n = a.nelem
        w, g_, m, v = (torch.randn(n, device=dev) * 1e-3 for _ in range(4))
        v.abs_()
        wb = torch.empty(n, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: eb.call("eisen_adamw_step", s, P(w), P(wb), P(g_), P(m), P(v), n, 3e-4, 0.9, 0.95, 1e-8, 0.1,
                                   10.0, 20.0, 1.0, None, 0.0), a.iters)
        out.update(ms=ms, gbs=n * 30 / ms / 1e6)
    out["status"] = int(st.item())
    print(json.dumps(out))


if __name__ == "__main__":
    main()
