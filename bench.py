#!/usr/bin/env python
"""Benchmark of the training-step hot path: tokens/s of forward + backward + AdamW.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun)
    python bench.py --impl reference ...                     (CPU restatement of the reference)

One "step" = zero_grad, `accum` micro-steps (forward, masked cross-entropy, backward through the
tape), bucketed gradient exchange when N > 1, global-norm clip (1.0) and fused AdamW.  Rank 0
prints ONE JSON line.  `value` is measured with the token batches already resident in HBM and no
per-launch instrumentation; the per-kernel-class breakdown (`kernels`, `roofline`) comes from a
second pass with CUDA events around every tensor-core launch; `e2e` repeats the measurement
through the public API with the batches in pinned host memory (H2D copy of ids and targets and
D2H read of the loss inside the timed region).  At N = 1 the line also carries `cases`: the other
benchmark configurations (isolated attention backward, cross-entropy + LM-head dW + RMSNorm
backward + AdamW at their full sizes, the 14M model, the tiny f32 model) timed after the main
measurement, and `cpu_baseline`: the CPU restatement's full step of the tiny f32 model, measured.
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
                      checkpoint=False, tie=False, overlap_optimizer=False),  # its step is also replayed from a CUDA graph
    # BASELINE.json configs[0]: the CPU-runnable tiny f32 model, one step of batch 4 x 64
    "tiny-f32": dict(vocab=512, hidden=128, layers=2, heads=4, kv=4, ffn=384, batch=4, seq=64, accum=1,
                     checkpoint=False, tie=False, f32=True),
}
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# DRAM bytes per algorithmic FLOP of the tcgen05 GEMM: one ncu capture of the M=8192, N=5632,
# K=2048 launch read and wrote 128.2 MB for 1.890e11 FLOPs; traffic grows with the tile count
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
# CPU arm: the oracle (a C++ restatement of the reference's Device::Cpu path; the Rust reference
# itself cannot be built in this image).  Everything here is measured, nothing extrapolated.
# ------------------------------------------------------------------------------------------
def _oracle():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_binding as ob
    return ob


def cpu_step_times(cfg, threads, batch, tokens_per_row, steps, warmup, clip=None):
    """Builds the model of `cfg` in the oracle and times full steps (zero_grad, forward,
    cross-entropy, backward, AdamW) on a [batch, tokens_per_row] token batch.  Returns
    (seconds per timed step, seconds spent building the model)."""
    import numpy as np
    ob = _oracle()
    ob.lib().orc_set_threads(int(threads))
    t0 = time.time()
    og = ob.OracleGraph()
    lm = ob.OracleLM(og, cfg["vocab"], cfg["hidden"], cfg["heads"], cfg["kv"], cfg["ffn"], cfg["layers"], cfg["tie"])
    og.mark_params()
    ps = lm.params()
    rng = np.random.default_rng(0)
    if cfg.get("f32"):  # BASELINE configs[0]: N(0, 0.02) weights from seed 0, norms 1
        for p in ps:
            shp = og.shape(p)
            if len(shp) == 2:
                og.load_tensor_data(p, (rng.standard_normal(int(np.prod(shp))) * 0.02).astype(np.float32))
    opt = ob.OracleAdamW(og, ps, 3e-4)
    opt.config(3e-4, 0.9, 0.95, 1e-8, 0.1)
    build_s = time.time() - t0
    n = batch * tokens_per_row
    secs = []
    for it in range(warmup + steps):
        ids = rng.integers(0, cfg["vocab"], (batch, tokens_per_row))
        tg = rng.integers(0, cfg["vocab"], n)
        t0 = time.time()
        opt.zero_grad()
        x = og.alloc([batch, tokens_per_row], ids.astype(np.float32))
        logits = lm.forward(x)
        og.reinterpret_shape(logits, [n, cfg["vocab"]])
        loss = og.cross_entropy(logits, tg.tolist())
        og.backward(loss)
        og.clear_activations()
        if clip:
            opt.clip_grad_norm(clip)
        opt.step()
        if it >= warmup:
            secs.append(time.time() - t0)
    return secs, build_s


def cpu_tiny_step(repeats=5):
    """configs[0] (the reference's CPU-runnable case): the full f32 step of batch 4 x 64 on one
    thread (the reference's schedule), median of `repeats`."""
    cfg = CONFIGS["tiny-f32"]
    secs, _ = cpu_step_times(cfg, 1, cfg["batch"], cfg["seq"], repeats, 1)
    med = statistics.median(secs)
    n = cfg["batch"] * cfg["seq"]
    return {"workload": "tiny-f32 (BASELINE configs[0]): vocab 512, d 128, 2 blocks, 4 heads, ffn 384, batch 4 x 64, f32",
            "tokens_per_s": n / med, "ms_per_step": 1e3 * med, "tokens_per_step": n, "cores": 1, "repeats": repeats}


def run_reference(args, cfg, name):
    """CPU arm.  A step is one full training step (forward, cross-entropy, backward, AdamW over
    all parameters) of the SAME architecture on a bounded sample of the batch: 1 x `t` tokens
    instead of 8 x 2048, with every host thread the oracle can use.  The CPU path has no batching
    effects (scalar loops, no BLAS), so its per-token cost does not fall with more tokens; the
    full batch itself would take hours.  value = sample tokens / measured step time."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    total_steps = args.warmup + args.steps
    if name == "llama-0.85b-gqa":
        # about 8 s per token and step on 8 cores: keep the whole run within a few minutes
        t = 2 if total_steps <= 10 else 1
        batch, row = 1, t
    else:
        batch, row = cfg["batch"], cfg["seq"]
    secs, build_s = cpu_step_times(cfg, cores, batch, row, args.steps, args.warmup)
    n = batch * row
    total = sum(secs)
    value = n * len(secs) / total
    sample = ("oracle (C++ restatement of the reference's Device::Cpu f32 path; the Rust reference cannot be built "
              "here), %d threads; each step = zero_grad + forward + cross-entropy + backward + AdamW of the full "
              "%s architecture on a %d x %d token batch (the GPU arm runs %d x %d per step); measured, not "
              "extrapolated; model built in %.1f s outside the timed steps"
              % (cores, name, batch, row, cfg["batch"] * cfg["accum"], cfg["seq"], build_s))
    out = {
        "impl": "reference", "metric": "train tokens/sec (fwd+bwd+AdamW)", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(secs),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "global_batch": batch, "seq_len": row, "sample_tokens_per_step": n,
                   "full_tokens_per_step": cfg["batch"] * cfg["accum"] * cfg["seq"]},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "tiny_f32_step": cpu_tiny_step(5),
    }
    print(json.dumps(out), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
class Runner:
    """One model on one rank: resident and pinned-host batches, optimizer, gradient exchange."""

    def __init__(self, cfg, args, rank, world, dev, compute):
        import numpy as np
        import torch

        import eisen_b200 as eb
        from eisen_b200 import dp as edp
        from eisen_b200.graph import AdamW, BF16_MIXED, FP32, Graph, TransformerLM

        self.cfg, self.args, self.rank, self.world, self.dev, self.compute = cfg, args, rank, world, dev, compute
        B, S, accum = cfg["batch"], cfg["seq"], cfg["accum"]
        self.checkpoint = cfg["checkpoint"] and not args.no_checkpoint
        self.clip = 0.0 if cfg.get("f32") else 1.0
        g = self.g = Graph(FP32 if cfg.get("f32") else BF16_MIXED, compute.cuda_stream)
        lm = self.lm = TransformerLM(g, cfg["vocab"], cfg["hidden"], cfg["heads"], cfg["kv"], cfg["ffn"], cfg["layers"], cfg["tie"])
        # synthetic uniform token ids / targets from a per-rank seed; resident copies live below the
        # parameter watermark so clear_activations() keeps them
        rng = np.random.default_rng(1234 + rank)
        self.n_host = 4
        self.host_ids = [torch.from_numpy(rng.integers(0, cfg["vocab"], (B, S)).astype(np.int32)).pin_memory() for _ in range(self.n_host)]
        self.host_tgt = [torch.from_numpy(rng.integers(0, cfg["vocab"], (B * S,)).astype(np.int32)).pin_memory() for _ in range(self.n_host)]
        self.res_ids = [g.alloc_ids([B, S], self.host_ids[i % self.n_host].data_ptr()) for i in range(accum)]
        self.res_tgt = [g.alloc_ids([B * S], self.host_tgt[i % self.n_host].data_ptr()) for i in range(accum)]
        g.mark_params()
        self.params = lm.params()
        self.opt = AdamW(g, self.params, 3e-4)
        self.opt.config(3e-4, 0.9, 0.95, 1e-8, 0.1)
        self.n_params = sum(int(np.prod(g.shape(p))) for p in self.params)
        self.reducer = None
        self.sharded = False
        self.overlapped = False
        if world == 1 and not cfg.get("f32") and getattr(args, "optimizer_overlap", False) and cfg.get("overlap_optimizer", True):
            # the update of step t runs on a side stream beside the forward pass of step t + 1
            from eisen_b200.overlap import OverlappedAdamW
            self.opt = OverlappedAdamW(g, lm, self.params, 3e-4, cfg["layers"], compute)
            self.opt.config(3e-4, 0.9, 0.95, 1e-8, 0.1)
            self.overlapped = True
        if world > 1:
            import torch.distributed as dist
            wptr, sptr, gptr, n_arena = g.param_arena()
            flat = edp.device_view(gptr, n_arena, dev)
            shapes = [g.shape(p) for p in sorted(self.params)]  # creation order == arena order
            offs, total = edp.param_offsets(shapes)
            assert total == n_arena, (total, n_arena)
            buckets = edp.plan_buckets(offs, cfg["layers"], total, min_bucket_elems=args.bucket_mb * (1 << 20) // 4)
            comm = torch.cuda.Stream(device=dev, priority=-1)
            if args.backend == "abi":
                # the library's own NCCL layer (eisen_dp_*); the 128-byte id travels over the process group
                def exchange_id(raw):
                    t = torch.zeros(128, dtype=torch.uint8, device=dev)
                    if raw is not None:
                        t.copy_(torch.frombuffer(bytearray(raw), dtype=torch.uint8))
                    dist.broadcast(t, src=0)
                    return bytes(t.cpu().numpy().tobytes())
                backend = edp.NcclAbiBackend(rank, world, comm, exchange_id)
            else:
                backend = edp.TorchBackend(None, comm)
            hs = None
            if not args.no_handshake:
                hs = edp.StepHandshake(dist.distributed_c10d._get_default_store(), rank, world, timeout_s=120.0)
            if args.exchange == "zero1":
                exact = [(o, o + s[0]) for o, s in zip(offs, shapes) if len(s) == 1]  # norm weights are read in f32
                self.reducer = edp.ShardedExchange(flat, buckets, gather=edp.device_view(sptr, n_arena, dev, torch.bfloat16),
                                                   flat_w=edp.device_view(wptr, n_arena, dev), exact_ranges=exact,
                                                   backend=backend, handshake=hs)
                from eisen_b200.graph import ShardedAdamW
                self.opt = ShardedAdamW(g, self.params, 3e-4, self.reducer.pieces())
                self.opt.config(3e-4, 0.9, 0.95, 1e-8, 0.1)
                self.sharded = True
                if not args.no_gather_overlap:
                    # the forward pass waits per block for the all-gather of the weights it is about to read
                    lm.set_forward_hook(lambda l: self.reducer.wait_for_block(l, self.compute))
            else:
                self.reducer = edp.BucketedAllReduce(flat, buckets, backend=backend, handshake=hs)
            eb.call("eisen_gemm_reserve_sms", args.comm_sms)
        self.last_loss = None
        self.feeder = None
        if args.data:
            # e2e leg from a pre-tokenised u16 file (the reference's .bin format) instead of synthetic ids
            from eisen_b200.data import BinaryDataLoader, PinnedBatchFeeder
            self.feeder = PinnedBatchFeeder(BinaryDataLoader(args.data, S, B), g, compute)

    def step(self, e2e, it):
        cfg, g = self.cfg, self.g
        B, S, accum = cfg["batch"], cfg["seq"], cfg["accum"]
        self.opt.zero_grad()
        for a in range(accum):
            n_valid = B * S
            if e2e and self.feeder is not None:
                nxt = self.feeder.next()
                if nxt is None:  # end of file: start over
                    self.feeder.loader.reset()
                    self.feeder.ready = self.feeder._fill(self.feeder.cur)
                    nxt = self.feeder.next()
                x, t, _, n_valid = nxt
            elif e2e:
                j = (it * accum + a) % self.n_host
                x = g.alloc_ids([B, S], self.host_ids[j].data_ptr())
                t = g.alloc_ids([B * S], self.host_tgt[j].data_ptr())
            else:
                x, t = self.res_ids[a], self.res_tgt[a]
            cb = None
            if self.reducer is not None and a == accum - 1:
                if self.sharded:
                    cb = lambda layer: self.reducer.on_block_done(layer, self.compute, optimizer=self.opt)  # noqa: E731
                else:
                    cb = lambda layer: self.reducer.on_block_done(layer, self.compute)  # noqa: E731
            loss = self.lm.train_micro_step_dev(x, t, n_valid, checkpoint=self.checkpoint, after_block=cb)
            if e2e:
                self.last_loss = float(g.data(loss)[0])  # D2H read of the step's loss
            g.clear_activations()
        if self.sharded:
            self.reducer.finish_and_step(self.opt, self.clip, self.compute, overlap=not self.args.no_gather_overlap)
            return
        if self.reducer is not None:
            self.reducer.finish(self.compute)
        self.opt.step_fused(self.clip, 1.0 / self.world)

    def timed(self, e2e, steps):
        import torch
        import torch.distributed as dist
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(self.compute)
        for it in range(steps):
            self.step(e2e, it)
        if self.overlapped:
            self.opt.finish()  # the last step's update runs on the side stream: it belongs to the timed region
        e1.record(self.compute)
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=self.dev)
        if self.world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def close(self):
        if self.overlapped:
            self.opt.close()
        if self.sharded:
            self.reducer.wait_all(self.compute)
            self.lm.set_forward_hook(None)
        self.g.synchronize()
        self.feeder = None
        self.reducer = None
        self.opt = None
        self.lm = None
        self.g.close()


def side_cases(args, peaks, dev, compute):
    """The other benchmark configurations, timed with CUDA events after the main measurement (rank 0,
    one GPU): every entry carries its algorithmic bytes or FLOPs, its time and its fraction of the
    measured peak (HBM copy bandwidth, or the bf16 GEMM burst rate for a kernel timed alone)."""
    import torch

    import bench_cases as bc
    hbm = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    burst = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    out = {"peaks": {"hbm_gbs": hbm, "bf16_tflops_burst": burst, "source": peaks["_source"]},
           "l2": "inputs larger than L2, or rotated through enough buffer sets to cover 3 x L2"}
    with torch.cuda.stream(compute):
        # configs[2]: isolated flash-attention backward with GQA, B 8, 32 / 8 heads, D 128, S 2048, causal
        a = bc.case_attn(8, 2048, 32, 8, 128, iters=6)
        out["cfg3_attn_B8_Hq32_Hkv8_D128_S2048"] = {
            "bwd_tflops": a["bwd_tflops"], "bwd_ms": a["bwd_ms"], "bwd_flops": a["bwd_flops"],
            "bwd_frac_of_burst": a["bwd_tflops"] / burst, "fwd_tflops": a["fwd_tflops"], "fwd_ms": a["fwd_ms"],
            "fwd_frac_of_burst": a["fwd_tflops"] / burst, "status": a["status"]}
        # the attention shape of the headline model (configs[4]): B 8, 32 / 8 heads, D 64, S 2048
        a = bc.case_attn(8, 2048, 32, 8, 64, iters=6)
        out["cfg5_attn_B8_Hq32_Hkv8_D64_S2048"] = {
            "bwd_tflops": a["bwd_tflops"], "bwd_ms": a["bwd_ms"], "bwd_flops": a["bwd_flops"],
            "bwd_frac_of_burst": a["bwd_tflops"] / burst, "fwd_tflops": a["fwd_tflops"], "fwd_ms": a["fwd_ms"],
            "fwd_frac_of_burst": a["fwd_tflops"] / burst, "status": a["status"]}
        # configs[3]: cross-entropy forward + backward over [16384, 32000] (5 % ignored), LM-head dW GEMM,
        # RMSNorm backward on [16384, 2048], AdamW over 1.1e9 f32 parameters
        c = bc.case_ce(16384, 32000, iters=5, ignore_frac=0.05)
        c4 = {"ce_fwd": {"gbs": c["fwd_gbs"], "ms": c["fwd_ms"], "bytes": c["fwd_bytes"], "frac_of_hbm": c["fwd_gbs"] / hbm},
              "ce_bwd": {"gbs": c["bwd_gbs"], "ms": c["bwd_ms"], "bytes": c["bwd_bytes"], "frac_of_hbm": c["bwd_gbs"] / hbm},
              "ce_fused_fwd_bwd": {"gbs": c["fused_gbs"], "ms": c["fused_ms"], "bytes": c["fused_bytes"],
                                   "frac_of_hbm": c["fused_gbs"] / hbm}}
        del c
        torch.cuda.empty_cache()
        d = bc.case_gemm(2048, 32000, 16384, a_mn=1, b_mn=1, out_mode=4, split_k=0, iters=5)
        c4["lm_head_dw_gemm"] = {"tflops": d["tflops"], "ms": d["ms"], "flops": d["flops"], "frac_of_burst": d["tflops"] / burst,
                                 "shape_mnk": d["shape"]}
        torch.cuda.empty_cache()
        r = bc.case_rmsnorm(16384, 2048, iters=12)
        c4["rmsnorm_bwd"] = {"gbs": r["bwd_gbs"], "ms": r["bwd_ms"], "bytes": r["bwd_bytes"], "frac_of_hbm": r["bwd_gbs"] / hbm,
                             "buffer_sets": r["sets"]}
        c4["rmsnorm_fwd"] = {"gbs": r["fwd_gbs"], "ms": r["fwd_ms"], "frac_of_hbm": r["fwd_gbs"] / hbm}
        sw = bc.case_swiglu(16384, 5632, iters=6)
        c4["swiglu_bwd"] = {"gbs": sw["bwd_gbs"], "ms": sw["bwd_ms"], "bytes": sw["bwd_bytes"], "frac_of_hbm": sw["bwd_gbs"] / hbm}
        del r, sw
        torch.cuda.empty_cache()
        e = bc.case_elementwise(16384, 2048, 2048, 64, 32000, 100_000_000, iters=12)
        c4["rope_bwd"] = {"gbs": e["rope_bwd_gbs"], "frac_of_hbm": e["rope_bwd_gbs"] / hbm}
        c4["embedding_bwd"] = {"gbs": e["embedding_bwd_gbs"], "ms": e["embedding_bwd_ms"], "frac_of_hbm": e["embedding_bwd_gbs"] / hbm,
                               "what": "whole call: grouping of the positions by id (five small launches on the ids alone) + row sums"}
        c4["embedding_bwd_row_sums"] = {"gbs": e["embedding_bwd_apply_gbs"], "ms": e["embedding_bwd_apply_ms"],
                                        "frac_of_hbm": e["embedding_bwd_apply_gbs"] / hbm,
                                        "what": "eisen_embedding_bwd_apply, the part on the backward path: the model runs the grouping on a side stream during the forward pass"}
        c4["sumsq"] = {"gbs": e["sumsq_gbs"], "frac_of_hbm": e["sumsq_gbs"] / hbm}
        del e
        torch.cuda.empty_cache()
        w = bc.case_adamw(1_100_000_000, iters=3)
        c4["adamw_1.1e9"] = {"gbs": w["gbs"], "ms": w["ms"], "bytes": w["bytes"], "frac_of_hbm": w["gbs"] / hbm}
        del w
        torch.cuda.empty_cache()
        out["cfg4_ce_head_rmsnorm_adamw"] = c4
    return out


def side_models(args, dev, compute):
    """configs[1] (14M bf16 model, accumulation 2) and configs[0] (tiny f32 model) through the same
    step as the headline model."""
    out = {}
    for key, name, steps in (("cfg2_llama-14m", "llama-14m", 10), ("cfg1_tiny-f32", "tiny-f32", 20)):
        cfg = CONFIGS[name]
        r = Runner(cfg, args, 0, 1, dev, compute)
        for it in range(3):
            r.step(False, it)
        ms = r.timed(False, steps) / steps
        n = cfg["batch"] * cfg["seq"] * cfg["accum"]
        out[key] = {"ms_per_step": ms, "tokens_per_s": n / (ms * 1e-3), "tokens_per_step": n, "params": r.n_params,
                    "dtype": "f32" if cfg.get("f32") else "bf16"}
        if not cfg.get("f32"):
            # the same step recorded once into a CUDA graph and replayed (the eager step of this small
            # model is bound by its ~1500 launches); the Fp32 graph's reference attention chain uploads
            # its mask from the host and cannot be captured
            import torch
            r.opt.advance()
            captured = r.g.capture(lambda: r.step(False, 0))
            for _ in range(3):
                r.opt.advance()
                captured.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(compute)
            for _ in range(steps):
                r.opt.advance()
                captured.replay()
            e1.record(compute)
            torch.cuda.synchronize()
            gms = e0.elapsed_time(e1) / steps
            out[key]["cuda_graph"] = {"ms_per_step": gms, "tokens_per_s": n / (gms * 1e-3)}
            captured.close()
        r.close()
    return out


def run_ours(args, cfg, name):
    import torch
    import torch.distributed as dist

    import eisen_b200 as eb

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
    compute = torch.cuda.Stream(device=dev)
    r = Runner(cfg, args, rank, world, dev, compute)
    g = r.g
    for it in range(args.warmup):
        r.step(False, it)
    g.synchronize()

    # ---- value: device-resident batches, no per-launch instrumentation
    L = eb.lib()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = L.eisen_launch_count()
    ms_total = r.timed(False, args.steps)
    launches = L.eisen_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None

    # ---- e2e: pinned host batches, H2D of ids / targets and D2H of the loss in the timed region
    for it in range(min(args.warmup, 2)):
        r.step(True, it)
    ms_e2e = r.timed(True, args.steps)

    # ---- second pass: CUDA events around every tensor-core launch for the per-class breakdown
    prof_steps = min(args.steps, 5)
    g.prof_enable(True)
    g.prof_read()
    ms_prof = r.timed(False, prof_steps)
    prof = g.prof_read()
    g.prof_enable(False)
    g.synchronize()

    # ---- variant: per-block checkpointing that keeps each block's attention output and log-sum-exp
    # (66 MB per block here) instead of running the attention forward again in the backward pass
    ms_keep = None
    if r.checkpoint and not args.no_variants:
        r.lm.set_keep_attention(True)
        for it in range(2):
            r.step(False, it)
        ms_keep = r.timed(False, args.steps)
        r.lm.set_keep_attention(False)
        g.synchronize()
    # ---- variant: no recomputation at all (every block's activations are kept: about 1 GB per block here)
    ms_plain = None
    if r.checkpoint and world == 1 and not args.no_variants:
        r.checkpoint = False
        try:
            for it in range(2):
                r.step(False, it)
            ms_plain = r.timed(False, min(args.steps, 3)) / min(args.steps, 3)
        finally:
            r.checkpoint = True
        g.synchronize()
    # ---- variant: fixed-order arithmetic (one slice per weight-gradient tile, dQ summed in key order):
    # gradients are bit-identical from run to run
    ms_det = None
    if world == 1 and not args.no_variants:
        eb.call("eisen_set_deterministic", 1)
        try:
            for it in range(2):
                r.step(False, it)
            ms_det = r.timed(False, min(args.steps, 3)) / min(args.steps, 3)
        finally:
            eb.call("eisen_set_deterministic", 0)
        g.synchronize()

    step_tokens = B * S * accum * world
    tps = step_tokens * args.steps / (ms_total / 1e3)
    tps_e2e = step_tokens * args.steps / (ms_e2e / 1e3)
    out = None
    if rank == 0:
        peaks = measured_peaks()
        fpt = model_flops_per_token(cfg)
        gemm_ms, gemm_fl, gemm_n = prof["gemm"]
        achieved = gemm_fl / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
        peak = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
        kernels = {"pass": "second pass of %d steps with two CUDA events around each tensor-core launch" % prof_steps,
                   "ms_per_step_in_this_pass": ms_prof / prof_steps}
        for k, (ms, fl, n) in prof.items():
            kernels[k] = {"ms_per_step": ms / prof_steps, "launches_per_step": n / prof_steps,
                          "tflops": (fl / (ms * 1e-3) / 1e12) if ms > 0 else None}
        tc_ms = sum(v[0] for v in prof.values()) / prof_steps
        kernels["other_ms_per_step"] = ms_prof / prof_steps - tc_ms
        out = {
            "metric": "train tokens/sec (fwd+bwd+AdamW)", "value": tps, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": name, "params": r.n_params, "global_batch": B * accum * world, "seq_len": S,
                       "micro_batch_per_gpu": B, "grad_accum": accum, "parallelism": "dp%d" % world,
                       "gradient_checkpointing": "per-block" if r.checkpoint else "off", "grad_clip_norm": r.clip,
                       "l2": "inputs larger than L2 (weights, activations and logits far exceed 126 MB)",
                       "bucket_mb": args.bucket_mb if world > 1 else None,
                       "exchange": (args.exchange + " via " + ("eisen_dp_* (NCCL)" if args.backend == "abi" else "torch.distributed")) if world > 1 else None,
                       "optimizer": ("AdamW pieces on a side stream beside the next step's forward pass; every timed step "
                                     "contains one full update" if r.overlapped else "AdamW on the compute stream")},
            "mfu": {"model_flops_per_token": fpt,
                    "of_nominal_2250_tflops": tps / world * fpt / (NOMINAL_BF16_TFLOPS * 1e12),
                    "of_measured_burst": tps / world * fpt / (float(peaks.get("bf16_tflops", 1590.0)) * 1e12),
                    "peaks": peaks["_source"]},
            "e2e": {"value": tps_e2e, "unit": "tokens/s", "h2d_bytes_per_step": 2 * B * S * 4 * accum,
                    "d2h_bytes_per_step": 4 * accum, "ms_per_step": ms_e2e / args.steps, "last_loss": r.last_loss},
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
        if ms_keep is not None:
            out["variants"] = {"keep_attention_output": {
                "what": "per-block checkpointing that keeps every block's attention output and log-sum-exp from the first "
                        "forward pass and recomputes the rest of the block (`value` recomputes the whole block)",
                "ms_per_step": ms_keep / args.steps, "tokens_per_s": step_tokens * args.steps / (ms_keep / 1e3),
                "mfu_of_nominal_2250_tflops": step_tokens * args.steps / (ms_keep / 1e3) / world * fpt / (NOMINAL_BF16_TFLOPS * 1e12)}}
        if ms_plain is not None:
            out.setdefault("variants", {})["no_checkpointing"] = {
                "what": "the same step without recomputation (activations of all blocks kept, about 16 GB at this batch): what the "
                        "step costs when memory, not the benchmark's configuration, decides; `value` recomputes every block",
                "ms_per_step": ms_plain, "tokens_per_s": step_tokens / (ms_plain / 1e3),
                "mfu_of_nominal_2250_tflops": step_tokens / (ms_plain / 1e3) / world * fpt / (NOMINAL_BF16_TFLOPS * 1e12)}
        if ms_det is not None:
            out.setdefault("variants", {})["fixed_order_arithmetic"] = {
                "what": "eisen_set_deterministic(1): weight-gradient GEMMs with one slice per tile, attention dQ written per key "
                        "tile and summed in key order; gradients are bit-identical from run to run (`value` uses split-K and "
                        "atomic adds)",
                "ms_per_step": ms_det, "tokens_per_s": step_tokens / (ms_det / 1e3)}
    r.close()
    del r, g
    if rank == 0 and world == 1 and not args.no_cases:
        peaks = measured_peaks()
        cases = side_cases(args, peaks, dev, compute)
        cases.update(side_models(args, dev, compute))
        out["cases"] = cases
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tiny = cpu_tiny_step(5)
        gpu_tiny = (out.get("cases") or {}).get("cfg1_tiny-f32")
        out["cpu_baseline"] = {
            "value": tiny["tokens_per_s"], "unit": "tokens/s", "cores": 1, "kind": "port",
            "sample": "oracle (C++ restatement of the reference's Device::Cpu f32 path), one thread: the FULL step "
                      "(zero_grad, forward, cross-entropy, backward, AdamW) of BASELINE configs[0], the reference's "
                      "CPU-runnable model (vocab 512, d 128, 2 blocks, batch 4 x 64), median of 5 measured steps; the "
                      "headline workload and configs[2..4] are infeasible on this CPU path at full size (hours per step) "
                      "and are not extrapolated; `bench.py --impl reference` times a bounded sample of the headline model",
            "workload": "tiny-f32", "ms_per_step": tiny["ms_per_step"], "tokens_per_step": tiny["tokens_per_step"],
            "gpu_same_workload": gpu_tiny,
        }
    if rank == 0:
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
    ap.add_argument("--no-variants", action="store_true", help="skip the kept-attention-output variant")
    ap.add_argument("--no-cases", action="store_true", help="skip the other benchmark configurations (N = 1 only)")
    ap.add_argument("--bucket-mb", type=int, default=256)
    ap.add_argument("--optimizer-overlap", action="store_true",
                    help="1 GPU: run AdamW block by block on a side stream beside the next step's forward pass "
                         "(eisen_b200.overlap.OverlappedAdamW; measured no faster: the step is power-limited)")
    ap.add_argument("--no-gather-overlap", action="store_true",
                    help="zero1: wait for the whole weight all-gather after the optimizer instead of per block in the next forward")
    ap.add_argument("--exchange", default="zero1", choices=["allreduce", "zero1"],
                    help="N > 1: all-reduce of gradient buckets with replicated AdamW, or reduce-scatter + sharded AdamW + all-gather")
    ap.add_argument("--backend", default="abi", choices=["abi", "torch"],
                    help="N > 1: collectives through the library's eisen_dp_* C ABI over NCCL, or through torch.distributed")
    ap.add_argument("--no-handshake", action="store_true", help="N > 1: skip the per-step host-side step handshake")
    args = ap.parse_args()
    cfg = CONFIGS[args.config]
    if args.impl == "reference":
        run_reference(args, cfg, args.config)
    else:
        run_ours(args, cfg, args.config)


if __name__ == "__main__":
    main()
