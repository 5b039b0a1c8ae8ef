"""Python mirror of the reference's `Graph`, `TransformerLM` and `AdamW` over the C ABI.

Method names and argument meaning follow `impl Graph` (src/graph/ops/*.rs, src/graph/mod.rs),
`TransformerLM` (src/nn/transformer.rs) and `AdamW` (src/nn/optim.rs).  Everything computes on the
GPU through libeisen_b200.so; a failed call raises EisenError.
"""
import ctypes as C

import numpy as np

from ._lib import EisenError, call, lib

FP32 = 0
BF16_MIXED = 1
IGNORE_INDEX = -1  # stands for the reference's usize::MAX (src/data/fim.rs:173)

BLOCK_CB = C.CFUNCTYPE(None, C.c_longlong, C.c_void_p)


def _ll(seq):
    return (C.c_longlong * max(1, len(seq)))(*[int(x) for x in seq])


class CapturedStep:
    """An executable CUDA graph of a captured step (Graph.capture)."""

    def __init__(self, handle, stream):
        self._h, self.stream = handle, stream

    def replay(self):
        call("eisen_graph_replay", self._h, self.stream)

    def close(self):
        if self._h:
            lib().eisen_graph_exec_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Graph:
    def __init__(self, precision=FP32, stream=0):
        """stream: a cudaStream_t as an integer (e.g. torch.cuda.current_stream().cuda_stream)."""
        self._h = C.c_void_p()
        call("eisen_graph_create", int(precision), stream, C.byref(self._h))
        self.precision = precision
        self.stream = stream

    def close(self):
        if self._h:
            lib().eisen_graph_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def capture(self, fn):
        """Records everything fn() enqueues on the graph's stream into a CUDA graph and returns a
        CapturedStep.  Run fn() once eagerly beforehand so that the capture allocates nothing."""
        call("eisen_graph_capture_begin", self._h)
        try:
            fn()
        except Exception:
            lib().eisen_graph_capture_abort(self._h)
            raise
        h = C.c_void_p()
        call("eisen_graph_capture_end", self._h, C.byref(h))
        return CapturedStep(h, self.stream)

    def set_vram_budget(self, budget_bytes, activation_reserve_bytes=64 << 20):
        """Budget for everything the graph allocates on the device; set it before building the model."""
        call("eisen_graph_set_vram_budget", self._h, int(budget_bytes), int(activation_reserve_bytes))

    def vram_usage(self):
        u, b = C.c_longlong(), C.c_longlong()
        call("eisen_graph_vram_usage", self._h, C.byref(u), C.byref(b))
        return u.value, b.value

    def plan_streaming(self, budget_bytes, activation_reserve_bytes, pinned_ids, apply=True):
        """Graph::plan_streaming (src/graph/memory.rs:64-187); returns the report as a dict."""
        n = self.counts()[2]
        res, stm = (C.c_longlong * max(1, n))(), (C.c_longlong * max(1, n))()
        nr, ns = C.c_int(), C.c_int()
        b4 = (C.c_longlong * 4)()
        call("eisen_graph_plan_streaming", self._h, int(budget_bytes), int(activation_reserve_bytes), _ll(pinned_ids),
             len(pinned_ids), 1 if apply else 0, res, C.byref(nr), stm, C.byref(ns), b4)
        return {"resident_param_ids": [res[i] for i in range(nr.value)], "streamed_param_ids": [stm[i] for i in range(ns.value)],
                "resident_bytes": b4[0], "resident_headroom_bytes": b4[1], "streamed_bytes": b4[2],
                "streaming_headroom_bytes": b4[3]}

    def _op(self, name, *args):
        out = C.c_longlong(-1)
        call("eisen_graph_" + name, self._h, *args, C.byref(out))
        return out.value

    # ---- storage
    def alloc(self, shape, data):
        a = np.ascontiguousarray(np.asarray(data, dtype=np.float32).reshape(-1))
        return self._op("alloc", _ll(shape), len(shape), a.ctypes.data)

    def alloc_ids(self, shape, ids):
        """ids: int32 numpy array or an integer host address of int32 values (pinned memory)."""
        if isinstance(ids, int):
            return self._op("alloc_ids", _ll(shape), len(shape), ids)
        a = np.ascontiguousarray(np.asarray(ids, dtype=np.int32).reshape(-1))
        return self._op("alloc_ids", _ll(shape), len(shape), a.ctypes.data)

    def alloc_pooled(self, shape):
        return self._op("alloc_pooled", _ll(shape), len(shape))

    def load_tensor_data(self, i, data):
        a = np.ascontiguousarray(np.asarray(data, dtype=np.float32).reshape(-1))
        call("eisen_graph_load_tensor_data", self._h, i, a.ctypes.data, a.size)

    def shape(self, i):
        buf = (C.c_longlong * 8)()
        n = C.c_int(0)
        call("eisen_graph_shape", self._h, i, buf, C.byref(n))
        return [buf[k] for k in range(n.value)]

    def numel(self, i):
        n = 1
        for d in self.shape(i):
            n *= d
        return n

    def sync_to_cpu(self, i):
        out = np.empty(self.numel(i), dtype=np.float32)
        call("eisen_graph_sync_to_cpu", self._h, i, out.ctypes.data)
        return out

    data = sync_to_cpu

    def sync_grad_to_cpu(self, i):
        out = np.empty(self.numel(i), dtype=np.float32)
        call("eisen_graph_sync_grad_to_cpu", self._h, i, out.ctypes.data)
        return out

    grad = sync_grad_to_cpu

    def tensor_ptrs(self, i):
        d, g = C.c_void_p(), C.c_void_p()
        dt, gdt = C.c_int(), C.c_int()
        call("eisen_graph_tensor_ptrs", self._h, i, C.byref(d), C.byref(g), C.byref(dt), C.byref(gdt))
        return d.value, g.value, dt.value, gdt.value

    def param_arena(self):
        w, s, g = C.c_void_p(), C.c_void_p(), C.c_void_p()
        n = C.c_longlong()
        call("eisen_graph_param_arena", self._h, C.byref(w), C.byref(s), C.byref(g), C.byref(n))
        return w.value, s.value, g.value, n.value

    # ---- graph state
    def save_weights(self, path):
        """All parameter tensors in id order, f32 (examples/train_llm.rs save_weights)."""
        call("eisen_graph_save_weights", self._h, str(path).encode())

    def load_weights(self, path):
        call("eisen_graph_load_weights", self._h, str(path).encode())

    def set_no_grad(self, flag):
        call("eisen_graph_set_no_grad", self._h, 1 if flag else 0)

    def flags(self):
        """(no_grad, skip_forward) as the graph holds them now."""
        a, b = C.c_int(), C.c_int()
        call("eisen_graph_get_flags", self._h, C.byref(a), C.byref(b))
        return bool(a.value), bool(b.value)

    def mark_params(self):
        call("eisen_graph_mark_params", self._h)

    def mark_save_point(self):
        out = C.c_longlong()
        call("eisen_graph_mark_save_point", self._h, C.byref(out))
        return out.value

    def restore_save_point(self, sp):
        call("eisen_graph_restore_save_point", self._h, sp)

    def clear_activations(self):
        call("eisen_graph_clear_activations", self._h)

    def tape_clear(self):
        call("eisen_graph_tape_clear", self._h)

    def reinterpret_shape(self, i, shape):
        call("eisen_graph_reinterpret_shape", self._h, i, _ll(shape), len(shape))

    def zero_grad_tensor(self, i):
        call("eisen_graph_zero_grad", self._h, i)

    def backward(self, loss):
        call("eisen_graph_backward", self._h, loss)

    def synchronize(self):
        call("eisen_graph_synchronize", self._h)

    def counts(self):
        a, b, c = C.c_longlong(), C.c_longlong(), C.c_longlong()
        call("eisen_graph_counts", self._h, C.byref(a), C.byref(b), C.byref(c))
        return a.value, b.value, c.value

    def num_tensors(self):
        return self.counts()[0]

    def tape_len(self):
        return self.counts()[1]

    def pool_stats(self):
        buf = (C.c_longlong * 5)()
        call("eisen_graph_pool_stats", self._h, buf)
        return dict(zip(("live_bytes", "cached_bytes", "device_bytes", "hits", "misses"), list(buf)))

    def prof_enable(self, on=True):
        call("eisen_graph_prof_enable", self._h, 1 if on else 0)

    def prof_read(self):
        """{class: (ms, flops, launches)} of the tensor-core kernels timed since the last read."""
        buf = (C.c_double * 9)()
        call("eisen_graph_prof_read", self._h, buf)
        return {n: (buf[3 * i], buf[3 * i + 1], int(buf[3 * i + 2])) for i, n in enumerate(("gemm", "attn_fwd", "attn_bwd"))}

    # ---- ops
    def add(self, a, b):
        return self._op("add", a, b)

    def mul(self, a, b):
        return self._op("mul", a, b)

    def silu(self, a):
        return self._op("silu", a)

    def swiglu(self, gate, up):
        return self._op("swiglu", gate, up)

    def matmul(self, a, b):
        return self._op("matmul", a, b)

    def matmul_add(self, a, b, r):
        """r + a @ b with the residual add fused into the GEMM epilogue (Bf16Mixed)."""
        return self._op("matmul_add", a, b, r)

    def matmul_trans_b(self, a, b):
        return self._op("matmul_trans_b", a, b)

    def bmm(self, a, b, trans_b):
        return self._op("bmm", a, b, 1 if trans_b else 0)

    def softmax(self, a):
        return self._op("softmax", a)

    def cross_entropy(self, logits, targets):
        return self._op("cross_entropy", logits, _ll(targets), len(targets))

    def cross_entropy_masked(self, logits, targets):
        return self._op("cross_entropy_masked", logits, _ll(targets), len(targets))

    def rms_norm(self, x, w, eps):
        return self._op("rms_norm", x, w, eps)

    def rope(self, a, head_dim):
        return self._op("rope", a, head_dim)

    def gather(self, w, idx):
        return self._op("gather", w, idx)

    def reshape(self, a, shape):
        return self._op("reshape", a, _ll(shape), len(shape))

    def transpose_0213(self, a):
        return self._op("transpose_0213", a)

    def repeat_kv(self, a, r):
        return self._op("repeat_kv", a, r)

    def flash_attention(self, q, k, v, scale, causal):
        return self._op("flash_attention", q, k, v, scale, 1 if causal else 0)

    def lm_head_cross_entropy(self, h, w, target_ids, n_valid, trans_b=False, chunk_rows=0):
        return self._op("lm_head_cross_entropy", h, w, target_ids, n_valid, 1 if trans_b else 0, chunk_rows)

    def attention(self, q, k, v, num_heads, num_kv_heads, causal=True):
        return self._op("attention", q, k, v, num_heads, num_kv_heads, 1 if causal else 0)


class TransformerLM:
    def __init__(self, g, vocab, hidden, heads, kv_heads, ffn, layers, tie=False):
        self.g = g
        self._h = C.c_void_p()
        call("eisen_lm_create", g._h, vocab, hidden, heads, kv_heads, ffn, layers, 1 if tie else 0, C.byref(self._h))
        self.vocab, self.hidden, self.heads, self.kv_heads, self.ffn, self.layers, self.tie = (
            vocab, hidden, heads, kv_heads, ffn, layers, tie)

    def __del__(self):
        try:
            if self._h:
                lib().eisen_lm_destroy(self._h)
        except Exception:
            pass

    def set_fused(self, flag):
        call("eisen_lm_set_fused", self._h, 1 if flag else 0)

    def set_forward_hook(self, before_block):
        """before_block(l) runs before the forward pass first reads block l's parameters (-1: embedding,
        layers: final norm and head)."""
        self._fwd_cb = BLOCK_CB(lambda layer, user: before_block(layer)) if before_block else None
        call("eisen_lm_set_forward_hook", self._h, C.cast(self._fwd_cb, C.c_void_p) if self._fwd_cb else None, None)

    def set_keep_attention(self, keep=True):
        """Checkpointed steps keep each block's attention output + log-sum-exp instead of recomputing them."""
        call("eisen_lm_set_keep_attention", self._h, 1 if keep else 0)

    def set_head_fusion(self, fused=True, chunk_rows=0):
        """Head projection + cross-entropy as one chunked op in train_micro_step (default on)."""
        call("eisen_lm_set_head_fusion", self._h, 1 if fused else 0, chunk_rows)

    def forward(self, x_id):
        out = C.c_longlong()
        call("eisen_lm_forward", self._h, self.g._h, x_id, C.byref(out))
        return out.value

    def params(self):
        buf = (C.c_longlong * (16 + 10 * self.layers))()
        n = C.c_int()
        call("eisen_lm_params", self._h, buf, C.byref(n))
        return [buf[i] for i in range(n.value)]

    def generate(self, prompt, max_new_tokens, max_context, kv_cache=True, return_logits=False):
        """Greedy generation (examples/train_llm.rs:560-584); kv_cache=False is the reference's loop."""
        p = np.ascontiguousarray(np.asarray(prompt, dtype=np.int32).reshape(-1))
        out = np.empty(max_new_tokens, dtype=np.int32)
        logits = np.empty(self.vocab, dtype=np.float32) if return_logits else None
        call("eisen_lm_generate", self._h, self.g._h, p.ctypes.data, p.size, max_new_tokens, max_context,
             1 if kv_cache else 0, out.ctypes.data, logits.ctypes.data if return_logits else None)
        return (out, logits) if return_logits else out

    def export_hf(self, safetensors_path, config_path=None, max_position_embeddings=2048):
        """model.safetensors (+ config.json) loadable as transformers.LlamaForCausalLM."""
        call("eisen_lm_export_hf", self._h, self.g._h, str(safetensors_path).encode(),
             str(config_path).encode() if config_path else None, max_position_embeddings)

    def train_micro_step(self, x_id, targets, checkpoint=False, after_block=None):
        """targets: sequence of ints or a ctypes long long array.  Returns the loss tensor id."""
        t = targets if isinstance(targets, C.Array) else _ll(targets)
        cb = BLOCK_CB(lambda layer, user: after_block(layer)) if after_block else None
        out = C.c_longlong()
        call("eisen_lm_train_micro_step", self._h, self.g._h, x_id, t, len(t), 1 if checkpoint else 0,
             C.cast(cb, C.c_void_p) if cb else None, None, C.byref(out))
        return out.value


    def train_micro_step_dev(self, x_id, target_ids_id, n_valid, checkpoint=False, after_block=None):
        """As train_micro_step with the targets already on the device (alloc_ids, -1 = ignored)."""
        cb = BLOCK_CB(lambda layer, user: after_block(layer)) if after_block else None
        out = C.c_longlong()
        call("eisen_lm_train_micro_step_dev", self._h, self.g._h, x_id, target_ids_id, n_valid, 1 if checkpoint else 0,
             C.cast(cb, C.c_void_p) if cb else None, None, C.byref(out))
        return out.value


class AdamW:
    def __init__(self, g, params, lr):
        self.g = g
        self._h = C.c_void_p()
        call("eisen_optim_create", g._h, _ll(params), len(params), lr, C.byref(self._h))

    def __del__(self):
        try:
            if self._h:
                lib().eisen_optim_destroy(self._h)
        except Exception:
            pass

    def config(self, lr, beta1, beta2, eps, weight_decay):
        call("eisen_optim_config", self._h, lr, beta1, beta2, eps, weight_decay)

    def zero_grad(self):
        call("eisen_optim_zero_grad", self._h)

    def clip_grad_norm(self, max_norm):
        n, c = C.c_float(), C.c_float()
        call("eisen_optim_clip_grad_norm", self._h, max_norm, C.byref(n), C.byref(c))
        return n.value, c.value

    def step(self):
        call("eisen_optim_step", self._h)

    def step_fused(self, max_norm=0.0, grad_scale=1.0):
        call("eisen_optim_step_fused", self._h, max_norm, grad_scale)

    def advance(self):
        """For steps replayed from a CUDA graph: t += 1 and this step's lr / bias corrections into
        the record the captured optimizer launch reads; call before the capture and before every replay."""
        call("eisen_optim_advance", self._h)

    def save_state(self, path):
        """Step count, hyper-parameters and moments: with the weights file this resumes a run bit for bit."""
        call("eisen_optim_save_state", self._h, str(path).encode())

    def load_state(self, path):
        call("eisen_optim_load_state", self._h, str(path).encode())

    def is_flat(self):
        f = C.c_int()
        call("eisen_optim_is_flat", self._h, C.byref(f))
        return bool(f.value)


class ShardedAdamW(AdamW):
    """AdamW that keeps moments for, and updates, only `pieces` (element ranges of the flat
    parameter arena): the optimizer of a ZeRO-1 data-parallel step (eisen_b200.dp.ShardedExchange)."""

    def __init__(self, g, params, lr, pieces):
        self.g = g
        self._h = C.c_void_p()
        lo, hi = _ll([a for a, _ in pieces]), _ll([b for _, b in pieces])
        call("eisen_optim_create_sharded", g._h, _ll(params), len(params), lr, lo, hi, len(pieces), C.byref(self._h))
        self.pieces = list(pieces)
        self._sumsq = None

    @property
    def sumsq(self):
        """One-element float64 device tensor: the squared gradient norm the clip uses."""
        if self._sumsq is None:
            import torch

            p = C.c_void_p()
            call("eisen_optim_sumsq_ptr", self._h, C.byref(p))

            class _V:
                __cuda_array_interface__ = {"shape": (1,), "typestr": "<f8", "data": (p.value, False), "version": 2}

            self._sumsq = torch.as_tensor(_V(), device=torch.device("cuda", torch.cuda.current_device()))
        return self._sumsq

    def begin_step(self):
        call("eisen_optim_begin_step", self._h)

    def sumsq_piece(self, i, accumulate, stream=None):
        call("eisen_optim_sumsq_piece", self._h, i, 1 if accumulate else 0, stream.cuda_stream if stream is not None else None)

    def step_piece(self, i, max_norm=0.0, grad_scale=1.0):
        call("eisen_optim_step_piece", self._h, i, max_norm, grad_scale)

    def step_piece_on(self, i, max_norm=0.0, grad_scale=1.0, stream=None, zero_grads=False):
        """step_piece on `stream` (a torch stream; None: the graph's), optionally clearing the piece's gradients."""
        call("eisen_optim_step_piece_on", self._h, i, max_norm, grad_scale, stream.cuda_stream if stream is not None else None,
             1 if zero_grads else 0)
