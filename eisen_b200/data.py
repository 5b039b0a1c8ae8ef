"""Input side of the training step: the reference's BinaryDataLoader (src/data/dataloader.rs:89-214)
over the library's eisen_loader_* entry points, plus a double-buffered pinned staging area that feeds
the graph's id tensors without a host synchronisation in the loop."""
import ctypes

import numpy as np

from ._lib import call, lib


class BinaryDataLoader:
    """u16 token file -> (ids, targets) int32 batches; targets use -1 as the ignore index.

    `fim` = (base_vocab, rate, spm_rate) turns the fill-in-the-middle transform on
    (`BinaryDataLoader::with_fim`, control tokens base_vocab .. base_vocab + 3)."""

    def __init__(self, path, seq_len, batch, fim=None, seed=None):
        self._h = ctypes.c_void_p()
        call("eisen_loader_open", str(path).encode(), seq_len, batch, ctypes.byref(self._h))
        self.seq_len, self.batch = seq_len, batch
        if fim is not None:
            call("eisen_loader_set_fim", self._h, int(fim[0]), float(fim[1]), float(fim[2]))
        if seed is not None:
            call("eisen_loader_seed", self._h, int(seed))

    def close(self):
        if self._h:
            call("eisen_loader_close", self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def total_batches(self):
        return int(lib().eisen_loader_total_batches(self._h))

    def reset(self):
        call("eisen_loader_reset", self._h)

    def next_into(self, x_ptr, t_ptr):
        """Writes the next batch to two host buffers of batch * seq_len int32; returns has_masked
        (bool), or None at the end of the file."""
        flag = ctypes.c_int(0)
        rc = lib().eisen_loader_next(self._h, ctypes.c_void_p(x_ptr), ctypes.c_void_p(t_ptr), ctypes.byref(flag))
        if rc == 1:
            return None
        if rc != 0:
            call("eisen_loader_next", self._h, ctypes.c_void_p(x_ptr), ctypes.c_void_p(t_ptr), ctypes.byref(flag))
        return bool(flag.value)

    def next_batch(self):
        """numpy convenience form: (x, targets, has_masked) or None."""
        n = self.batch * self.seq_len
        x = np.empty(n, dtype=np.int32)
        t = np.empty(n, dtype=np.int32)
        m = self.next_into(x.ctypes.data, t.ctypes.data)
        return None if m is None else (x, t, m)


class PinnedBatchFeeder:
    """Two pinned host buffers per stream of batches: while the device copies batch i from one
    buffer (Graph.alloc_ids issues the asynchronous copy on the graph's stream), the loader fills
    the other with batch i + 1.  A CUDA event per buffer says when its copy has been consumed."""

    def __init__(self, loader, graph, torch_stream):
        import torch

        self.loader, self.g, self.stream = loader, graph, torch_stream
        n = loader.batch * loader.seq_len
        self.x = [torch.empty(n, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.t = [torch.empty(n, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.free = [torch.cuda.Event() for _ in range(2)]
        self.cur = 0
        self.ready = self._fill(0)

    def _fill(self, i):
        self.free[i].synchronize()  # the copy that last read this buffer is done (no-op if never recorded)
        return self.loader.next_into(self.x[i].data_ptr(), self.t[i].data_ptr())

    def next(self):
        """-> (ids tensor id, targets tensor id, has_masked, n_valid) on the graph, or None at end
        of file; n_valid counts the targets that are not the ignore index (the loss normaliser)."""
        if self.ready is None:
            return None
        i = self.cur
        B, S = self.loader.batch, self.loader.seq_len
        n_valid = int((self.t[i].numpy() != -1).sum()) if self.ready else B * S
        ids = self.g.alloc_ids([B, S], self.x[i].data_ptr())
        tgt = self.g.alloc_ids([B * S], self.t[i].data_ptr())
        self.free[i].record(self.stream)
        masked = self.ready
        self.cur = 1 - i
        self.ready = self._fill(self.cur)
        return ids, tgt, masked, n_valid
