"""ctypes binding of the CPU oracle (oracle/liboracle.so).  Test infrastructure only.

The class mirrors the method names of the reference's `impl Graph` (src/graph/ops/*.rs) so the
parity tests read like the reference's own tests.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_SO = os.path.join(_ROOT, "oracle", "liboracle.so")
IGNORE_INDEX = -1  # stands for the reference's usize::MAX (src/data/fim.rs:173)

_lib = None


def build_oracle():
    src = os.path.join(_ROOT, "oracle", "oracle.cpp")
    if (not os.path.exists(_SO)) or (
        os.path.exists(src) and os.path.getmtime(src) > os.path.getmtime(_SO)
    ):
        subprocess.check_call(["make", "-C", os.path.join(_ROOT, "oracle"), "liboracle.so"])


def lib():
    global _lib
    if _lib is None:
        build_oracle()
        L = C.CDLL(_SO)
        LL, P, F, I = C.c_longlong, C.c_void_p, C.c_float, C.c_int
        PLL, PF = C.POINTER(C.c_longlong), C.POINTER(C.c_float)
        sig = {
            "orc_set_threads": (None, [I]),
            "orc_max_threads": (I, []),
            "orc_graph_new": (P, []),
            "orc_graph_free": (None, [P]),
            "orc_alloc": (LL, [P, PLL, I, PF]),
            "orc_numel": (LL, [P, LL]),
            "orc_shape": (I, [P, LL, PLL]),
            "orc_get_data": (None, [P, LL, PF]),
            "orc_get_grad": (None, [P, LL, PF]),
            "orc_set_data": (None, [P, LL, PF]),
            "orc_set_no_grad": (None, [P, I]),
            "orc_num_tensors": (LL, [P]),
            "orc_tape_len": (LL, [P]),
            "orc_tape_clear": (None, [P]),
            "orc_mark_params": (None, [P]),
            "orc_mark_save_point": (LL, [P]),
            "orc_restore_save_point": (None, [P, LL]),
            "orc_clear_activations": (None, [P]),
            "orc_reinterpret_shape": (None, [P, LL, PLL, I]),
            "orc_zero_grad_tensor": (None, [P, LL]),
            "orc_add": (LL, [P, LL, LL]),
            "orc_mul": (LL, [P, LL, LL]),
            "orc_silu": (LL, [P, LL]),
            "orc_matmul": (LL, [P, LL, LL]),
            "orc_matmul_trans_b": (LL, [P, LL, LL]),
            "orc_bmm": (LL, [P, LL, LL, I]),
            "orc_softmax": (LL, [P, LL]),
            "orc_cross_entropy": (LL, [P, LL, PLL, LL]),
            "orc_cross_entropy_masked": (LL, [P, LL, PLL, LL]),
            "orc_rms_norm": (LL, [P, LL, LL, F]),
            "orc_rope": (LL, [P, LL, LL]),
            "orc_gather": (LL, [P, LL, LL]),
            "orc_reshape": (LL, [P, LL, PLL, I]),
            "orc_transpose_0213": (LL, [P, LL]),
            "orc_repeat_kv": (LL, [P, LL, LL]),
            "orc_flash_attention": (LL, [P, LL, LL, LL, F, I]),
            "orc_backward": (None, [P, LL]),
            "orc_lm_new": (P, [P, LL, LL, LL, LL, LL, LL, I]),
            "orc_lm_free": (None, [P]),
            "orc_lm_forward": (LL, [P, P, LL]),
            "orc_lm_params": (I, [P, PLL]),
            "orc_adamw_new": (P, [PLL, I, F]),
            "orc_adamw_free": (None, [P]),
            "orc_adamw_config": (None, [P, F, F, F, F, F]),
            "orc_adamw_zero_grad": (None, [P, P]),
            "orc_adamw_clip_grad_norm": (F, [P, P, F, PF]),
            "orc_adamw_step": (None, [P, P]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def _ll(seq):
    arr = (C.c_longlong * max(1, len(seq)))(*[int(x) for x in seq])
    return arr


def _pf(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


class OracleGraph:
    def __init__(self):
        self.L = lib()
        self.h = self.L.orc_graph_new()

    def __del__(self):
        try:
            self.L.orc_graph_free(self.h)
        except Exception:
            pass

    # ---- storage
    def alloc(self, shape, data):
        a = np.ascontiguousarray(np.asarray(data, dtype=np.float32).reshape(-1))
        return self.L.orc_alloc(self.h, _ll(shape), len(shape), _pf(a))

    def shape(self, i):
        buf = (C.c_longlong * 8)()
        n = self.L.orc_shape(self.h, i, buf)
        return [buf[k] for k in range(n)]

    def data(self, i):
        out = np.empty(self.L.orc_numel(self.h, i), dtype=np.float32)
        self.L.orc_get_data(self.h, i, _pf(out))
        return out

    def grad(self, i):
        out = np.empty(self.L.orc_numel(self.h, i), dtype=np.float32)
        self.L.orc_get_grad(self.h, i, _pf(out))
        return out

    def load_tensor_data(self, i, data):
        a = np.ascontiguousarray(np.asarray(data, dtype=np.float32).reshape(-1))
        assert a.size == self.L.orc_numel(self.h, i)
        self.L.orc_set_data(self.h, i, _pf(a))

    def zero_grad_tensor(self, i):
        self.L.orc_zero_grad_tensor(self.h, i)

    # ---- graph state
    def set_no_grad(self, f):
        self.L.orc_set_no_grad(self.h, 1 if f else 0)

    def num_tensors(self):
        return self.L.orc_num_tensors(self.h)

    def tape_len(self):
        return self.L.orc_tape_len(self.h)

    def tape_clear(self):
        self.L.orc_tape_clear(self.h)

    def mark_params(self):
        self.L.orc_mark_params(self.h)

    def mark_save_point(self):
        return self.L.orc_mark_save_point(self.h)

    def restore_save_point(self, sp):
        self.L.orc_restore_save_point(self.h, sp)

    def clear_activations(self):
        self.L.orc_clear_activations(self.h)

    def reinterpret_shape(self, i, shape):
        self.L.orc_reinterpret_shape(self.h, i, _ll(shape), len(shape))

    # ---- ops
    def add(self, a, b):
        return self.L.orc_add(self.h, a, b)

    def mul(self, a, b):
        return self.L.orc_mul(self.h, a, b)

    def silu(self, a):
        return self.L.orc_silu(self.h, a)

    def matmul(self, a, b):
        return self.L.orc_matmul(self.h, a, b)

    def matmul_trans_b(self, a, b):
        return self.L.orc_matmul_trans_b(self.h, a, b)

    def bmm(self, a, b, trans_b):
        return self.L.orc_bmm(self.h, a, b, 1 if trans_b else 0)

    def softmax(self, a):
        return self.L.orc_softmax(self.h, a)

    def cross_entropy(self, logits, targets):
        return self.L.orc_cross_entropy(self.h, logits, _ll(targets), len(targets))

    def cross_entropy_masked(self, logits, targets):
        return self.L.orc_cross_entropy_masked(self.h, logits, _ll(targets), len(targets))

    def rms_norm(self, x, w, eps):
        return self.L.orc_rms_norm(self.h, x, w, eps)

    def rope(self, a, head_dim):
        return self.L.orc_rope(self.h, a, head_dim)

    def gather(self, w, idx):
        return self.L.orc_gather(self.h, w, idx)

    def reshape(self, a, shape):
        return self.L.orc_reshape(self.h, a, _ll(shape), len(shape))

    def transpose_0213(self, a):
        return self.L.orc_transpose_0213(self.h, a)

    def repeat_kv(self, a, r):
        return self.L.orc_repeat_kv(self.h, a, r)

    def flash_attention(self, q, k, v, scale, causal):
        return self.L.orc_flash_attention(self.h, q, k, v, scale, 1 if causal else 0)

    def backward(self, loss):
        self.L.orc_backward(self.h, loss)


class OracleLM:
    """TransformerLM of src/nn/transformer.rs:69-211 on the oracle graph."""

    def __init__(self, g, vocab, hidden, heads, kv_heads, ffn, layers, tie=False):
        self.g = g
        self.h = g.L.orc_lm_new(g.h, vocab, hidden, heads, kv_heads, ffn, layers, 1 if tie else 0)

    def forward(self, x_id):
        return self.g.L.orc_lm_forward(self.h, self.g.h, x_id)

    def params(self):
        buf = (C.c_longlong * 4096)()
        n = self.g.L.orc_lm_params(self.h, buf)
        return [buf[i] for i in range(n)]


class OracleAdamW:
    def __init__(self, g, params, lr):
        self.g = g
        self.h = g.L.orc_adamw_new(_ll(params), len(params), lr)

    def config(self, lr, beta1, beta2, eps, wd):
        self.g.L.orc_adamw_config(self.h, lr, beta1, beta2, eps, wd)

    def zero_grad(self):
        self.g.L.orc_adamw_zero_grad(self.h, self.g.h)

    def clip_grad_norm(self, max_norm):
        coef = C.c_float(1.0)
        n = self.g.L.orc_adamw_clip_grad_norm(self.h, self.g.h, max_norm, C.byref(coef))
        return n, coef.value

    def step(self):
        self.g.L.orc_adamw_step(self.h, self.g.h)
