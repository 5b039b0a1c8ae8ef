#!/usr/bin/env python
"""Benchmark of the training-step hot path: tokens/s of forward + backward + AdamW.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun)
    python bench.py --impl reference ...                     (CPU restatement of the reference)

One "step" = zero_grad, `accum` micro-steps (forward, masked cross-entropy, backward through the
tape), bucketed gradient all-reduce when N > 1, global-norm clip (1.0) and fused AdamW.  Rank 0
prints ONE JSON line.  `value` is measured with the token batches already resident in HBM;
`e2e` repeats the measurement through the public API with the batches in pinned host memory
(H2D copy of ids and targets and D2H read of the loss inside the timed region).
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # BASELINE.json configs[4]: ~0.85B-parameter GQA model, micro-batch 8 x 2048 per GPU
    "llama-0.85b-gqa": dict(vocab=32000, hidden=2048, layers=16, heads=32, kv=8, ffn=5632, batch=8, seq=2048,
                            accum=1, checkpoint=True, tie=False),
    # BASELINE.json configs[1]: ~14M-parameter model, batch 32 x 256, gradient accumulation 2
    "llama-14m": dict(vocab=8192, hidden=384, layers=6, heads=6, kv=6, ffn=1024, batch=32, seq=256, accum=2,
                      checkpoint=False, tie=False),
}
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# DRAM bytes per algorithmic FLOP of the tcgen05 GEMM, from the ncu capture summarised in
# profiles/gemm_bf16_tc2_M8192_N5632_K2048.md (128.2 MB for 1.890e11 FLOPs)
GEMM_DRAM_BYTES_PER_FLOP = 128.2e6 / 1.890e11


def model_flops_per_token(c):
    hd = c["hidden"] // c["heads"]
    kvd = c["kv"] * hd
    n_mm = c["layers"] * (2 * c["hidden"] * c["hidden"] + 2 * c["hidden"] * kvd + 3 * c["hidden"] * c["ffn"])
    n_mm += c["hidden"] * c["vocab"]  # LM head; the embedding gather is not a matmul
    return 6.0 * n_mm + 6.0 * c["layers"] * c["seq"] * c["hidden"]


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            d["_source"] = "measured"
            return d
        except Exception:
            pass
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ["clocks.sm", "clocks.max.sm", "power.draw", "clocks_event_reasons.hw_slowdown",
              "clocks_event_reasons.hw_thermal_slowdown", "clocks_event_reasons.sw_thermal_slowdown",
              "clocks_event_reasons.sw_power_cap"]

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--query-gpu=" + ",".join(self.FIELDS), "--format=csv,noheader,nounits", "-i",
                 str(self.index), "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < len(self.FIELDS):
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------
# CPU baseline: the oracle (a C++ restatement of the reference's Device::Cpu path) on a bounded
# sample of the workload
# ------------------------------------------------------------------------------------------
def cpu_sample(cfg, threads, tokens=2):
    """Times forward+backward of the full-width architecture with 1 and 2 blocks on `tokens`
    tokens and the AdamW update, and extrapolates linearly in the block count and the parameter
    count to one full step.  Returns (tokens_per_second, description, seconds_spent)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import numpy as np
    from oracle_binding import OracleAdamW, OracleGraph, OracleLM, lib as olib

    t_start = time.time()
    olib().orc_set_threads(int(threads))
    rng = np.random.default_rng(0)
    times = {}
    per_param_s = None
    for L in (1, 2):
        og = OracleGraph()
        lm = OracleLM(og, cfg["vocab"], cfg["hidden"], cfg["heads"], cfg["kv"], cfg["ffn"], L, cfg["tie"])
        og.mark_params()
        ps = lm.params()
        ids = rng.integers(0, cfg["vocab"], (1, tokens))
        tg = rng.integers(0, cfg["vocab"], tokens)
        t0 = time.time()
        x = og.alloc([1, tokens], ids.astype(np.float32))
        logits = lm.forward(x)
        og.reinterpret_shape(logits, [tokens, cfg["vocab"]])
        loss = og.cross_entropy(logits, tg.tolist())
        og.backward(loss)
        times[L] = time.time() - t0
        if L == 1:
            n_params = sum(int(np.prod(og.shape(p))) for p in ps)
            opt = OracleAdamW(og, ps, 3e-4)
            opt.config(3e-4, 0.9, 0.95, 1e-8, 0.1)
            t0 = time.time()
            opt.step()
            per_param_s = (time.time() - t0) / n_params
        del og, lm
    per_block = max(times[2] - times[1], 0.0)
    base = max(times[1] - per_block, 0.0)
    hd = cfg["hidden"] // cfg["heads"]
    kvd = cfg["kv"] * hd
    total_params = cfg["vocab"] * cfg["hidden"] * (1 if cfg["tie"] else 2) + cfg["hidden"] + cfg["layers"] * (
        2 * cfg["hidden"] + 2 * cfg["hidden"] ** 2 + 2 * cfg["hidden"] * kvd + 3 * cfg["hidden"] * cfg["ffn"])
    step_tokens = cfg["batch"] * cfg["seq"] * cfg["accum"]
    t_tokens = (base + cfg["layers"] * per_block) / tokens * step_tokens
    t_opt = per_param_s * total_params
    tps = step_tokens / (t_tokens + t_opt)
    desc = ("oracle (C++ restatement of the reference's Device::Cpu f32 path), full-width architecture with 1 and 2 "
            "blocks, forward+backward on 1x%d tokens plus one AdamW update; extrapolated linearly in blocks "
            "(%d) and parameters (%.3g) to a %d-token step; attention at this sequence length is negligible, "
            "so the figure is an upper bound" % (tokens, cfg["layers"], total_params, step_tokens))
    return tps, desc, time.time() - t_start


def run_reference(args, cfg, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    vals, secs = [], []
    for i in range(args.warmup + args.steps):
        v, desc, s = cpu_sample(cfg, cores, tokens=2)
        if i >= args.warmup:
            vals.append(v)
            secs.append(s)
    value = statistics.median(vals)
    out = {
        "impl": "reference", "metric": "train tokens/sec (fwd+bwd+AdamW)", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * statistics.mean(secs),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "global_batch": cfg["batch"] * cfg["accum"], "seq_len": cfg["seq"]},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def run_ours(args, cfg, name):
    import numpy as np
    import torch
    import torch.distributed as dist

    import eisen_b200 as eb
    from eisen_b200 import dp as edp
    from eisen_b200.graph import AdamW, BF16_MIXED, Graph, TransformerLM

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    B, S, accum = cfg["batch"], cfg["seq"], cfg["accum"]
    checkpoint = cfg["checkpoint"] and not args.no_checkpoint
    compute = torch.cuda.Stream(device=dev)
    g = Graph(BF16_MIXED, compute.cuda_stream)
    lm = TransformerLM(g, cfg["vocab"], cfg["hidden"], cfg["heads"], cfg["kv"], cfg["ffn"], cfg["layers"], cfg["tie"])

    # synthetic uniform token ids / targets from a per-rank seed; resident copies live below the
    # parameter watermark so clear_activations() keeps them
    rng = np.random.default_rng(1234 + rank)
    n_host_batches = 4
    host_ids = [torch.from_numpy(rng.integers(0, cfg["vocab"], (B, S)).astype(np.int32)).pin_memory() for _ in range(n_host_batches)]
    host_tgt = [torch.from_numpy(rng.integers(0, cfg["vocab"], (B * S,)).astype(np.int32)).pin_memory() for _ in range(n_host_batches)]
    res_ids = [g.alloc_ids([B, S], host_ids[i].data_ptr()) for i in range(accum)]
    res_tgt = [g.alloc_ids([B * S], host_tgt[i].data_ptr()) for i in range(accum)]
    g.mark_params()
    params = lm.params()
    opt = AdamW(g, params, 3e-4)
    opt.config(3e-4, 0.9, 0.95, 1e-8, 0.1)

    reducer = None
    if world > 1:
        _, _, gptr, n_arena = g.param_arena()
        flat = edp.device_view(gptr, n_arena, dev)
        shapes = []
        # creation order == arena order: embedding, 9 per block, final norm, head
        ids_sorted = sorted(params)
        for p in ids_sorted:
            shapes.append(g.shape(p))
        offs, total = edp.param_offsets(shapes)
        assert total == n_arena, (total, n_arena)
        buckets = edp.plan_buckets(offs, cfg["layers"], total, min_bucket_elems=args.bucket_mb * (1 << 20) // 4)
        reducer = edp.BucketedAllReduce(flat, buckets, comm_stream=torch.cuda.Stream(device=dev, priority=-1))
        # the persistent GEMMs leave a few SMs to the all-reduce kernels that run beside the backward
        eb.call("eisen_gemm_reserve_sms", args.comm_sms)

    state = {"loss": None}
    feeder = None
    if args.data:
        # e2e leg from a pre-tokenised u16 file (the reference's .bin format) instead of synthetic ids
        from eisen_b200.data import BinaryDataLoader, PinnedBatchFeeder
        feeder = PinnedBatchFeeder(BinaryDataLoader(args.data, S, B), g, compute)

    def step(e2e, it):
        opt.zero_grad()
        for a in range(accum):
            n_valid = B * S
            if e2e and feeder is not None:
                nxt = feeder.next()
                if nxt is None:  # end of file: start over
                    feeder.loader.reset()
                    feeder.ready = feeder._fill(feeder.cur)
                    nxt = feeder.next()
                x, t, _, n_valid = nxt
            elif e2e:
                j = (it * accum + a) % n_host_batches
                x = g.alloc_ids([B, S], host_ids[j].data_ptr())
                t = g.alloc_ids([B * S], host_tgt[j].data_ptr())
            else:
                x, t = res_ids[a], res_tgt[a]
            cb = None
            if reducer is not None and a == accum - 1:
                cb = lambda layer: reducer.on_block_done(layer, compute)  # noqa: E731
            loss = lm.train_micro_step_dev(x, t, n_valid, checkpoint=checkpoint, after_block=cb)
            if e2e:
                state["loss"] = float(g.data(loss)[0])  # D2H read of the step's loss
            g.clear_activations()
        if reducer is not None:
            reducer.finish(compute)
        opt.step_fused(1.0, 1.0 / world)

    def timed(e2e, steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(compute)
        for it in range(steps):
            step(e2e, it)
        e1.record(compute)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for it in range(args.warmup):
        step(False, it)
    g.synchronize()

    L = eb.lib()
    g.prof_enable(True)
    g.prof_read()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = L.eisen_launch_count()
    ms_total = timed(False, args.steps)
    launches = L.eisen_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    prof = g.prof_read()
    g.prof_enable(False)

    for it in range(min(args.warmup, 2)):
        step(True, it)
    ms_e2e = timed(True, args.steps)
    g.synchronize()

    step_tokens = B * S * accum * world
    tps = step_tokens * args.steps / (ms_total / 1e3)
    tps_e2e = step_tokens * args.steps / (ms_e2e / 1e3)
    if rank == 0:
        peaks = measured_peaks()
        fpt = model_flops_per_token(cfg)
        gemm_ms, gemm_fl, gemm_n = prof["gemm"]
        achieved = gemm_fl / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
        peak = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
        kernels = {}
        for k, (ms, fl, n) in prof.items():
            kernels[k] = {"ms_per_step": ms / args.steps, "launches_per_step": n / args.steps,
                          "tflops": (fl / (ms * 1e-3) / 1e12) if ms > 0 else None}
        tc_ms = sum(v[0] for v in prof.values()) / args.steps
        kernels["other_ms_per_step"] = ms_total / args.steps - tc_ms
        out = {
            "metric": "train tokens/sec (fwd+bwd+AdamW)", "value": tps, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": name, "params": None, "global_batch": B * accum * world, "seq_len": S,
                       "micro_batch_per_gpu": B, "grad_accum": accum, "parallelism": "dp%d" % world,
                       "gradient_checkpointing": "per-block" if checkpoint else "off", "grad_clip_norm": 1.0,
                       "l2": "inputs larger than L2 (weights, activations and logits far exceed 126 MB)",
                       "bucket_mb": args.bucket_mb if world > 1 else None},
            "mfu": {"model_flops_per_token": fpt,
                    "of_nominal_2250_tflops": tps / world * fpt / (NOMINAL_BF16_TFLOPS * 1e12),
                    "of_measured_burst": tps / world * fpt / (float(peaks.get("bf16_tflops", 1590.0)) * 1e12),
                    "peaks": peaks["_source"]},
            "e2e": {"value": tps_e2e, "unit": "tokens/s", "h2d_bytes_per_step": 2 * B * S * 4 * accum,
                    "d2h_bytes_per_step": 4 * accum, "ms_per_step": ms_e2e / args.steps, "last_loss": state["loss"]},
            "gpu_launches": int(launches),
            "roofline": {"kernel": "gemm_bf16_tc2_kernel / gemm_bf16_tc_kernel (all GEMM launches of the step)", "bound": "tensor",
                         "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak if peak else None,
                         "peak_source": "bf16_tflops_sustained of %s" % peaks["_source"],
                         "traffic": (gemm_fl / gemm_n) * GEMM_DRAM_BYTES_PER_FLOP if gemm_n else None,
                         "algorithmic_flops_per_launch": gemm_fl / gemm_n if gemm_n else None,
                         "avg_launch_ms": gemm_ms / gemm_n if gemm_n else None},
            "kernels": kernels,
            "clocks": clocks,
        }
        out["config"]["params"] = sum(int(np.prod(g.shape(p))) for p in params)
        if world == 1 and not args.no_cpu_baseline:
            v, desc, secs = cpu_sample(cfg, 1, tokens=4)  # about 15 s of single-thread CPU work
            out["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": 1, "kind": "port", "sample": desc,
                                   "seconds": secs}
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="llama-0.85b-gqa", choices=sorted(CONFIGS))
    ap.add_argument("--no-checkpoint", action="store_true")
    ap.add_argument("--data", default=None, help="u16 token file for the e2e leg (default: synthetic ids)")
    ap.add_argument("--comm-sms", type=int, default=0, help="SMs the GEMMs leave free for NCCL when N > 1 (measured at 8 GPUs: 0 is best)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--bucket-mb", type=int, default=256)
    args = ap.parse_args()
    cfg = CONFIGS[args.config]
    if args.impl == "reference":
        run_reference(args, cfg, args.config)
    else:
        run_ours(args, cfg, args.config)


if __name__ == "__main__":
    main()
