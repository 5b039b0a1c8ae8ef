"""Data-parallel plumbing: one process per GPU, bucketed gradient exchange overlapped with backward.

The reference has no distributed code; this is the exchange step the data-parallel training step
adds.  Every rank runs the whole forward/backward on its own micro-batch; the flat f32 gradient
buffer is cut into buckets in backward order (head and final norm first, then the blocks from
last to first, then the embedding) and a bucket is exchanged on a side stream as soon as the
backward pass has finished writing it.  Two exchanges:

* `BucketedAllReduce`: every rank holds full replicas; buckets are all-reduced (sum), every rank
  runs the whole optimizer, which folds 1/world into its gradient scale.
* `ShardedExchange` (ZeRO-1): a bucket is reduce-scattered, each rank keeps AdamW moments for and
  updates only its 1/world piece of every bucket, and the updated bf16 weights are all-gathered:
  1.5 instead of 2 gradient-sized transfers per step and 1/world of the optimizer's memory traffic.

Both run on one of two backends with the same interface: `NcclAbiBackend` (the library's own
eisen_dp_* C ABI over NCCL, raw device pointers, what a non-Python host would call) and
`TorchBackend` (torch.distributed; with gloo on CPU tensors this is how the host logic and the
failure handling are tested without GPUs).  No kernel of this package touches a peer's memory.

Failure handling is host-side and bounded: `StepHandshake` has every rank publish its step number
and the collectives it enqueued in a key-value store and read its peers' records with a deadline,
so a rank that left, or that skipped a bucket, is reported as an `EisenError` before anyone waits
on a collective that cannot complete; `finish(deadline_s=...)` bounds the wait itself and aborts
the communicator when it runs out.
"""
import ctypes as C
import datetime
import time

import torch
import torch.distributed as dist

from ._lib import EisenError, call, lib

F32, BF16, F64, I64 = 0, 1, 3, 4
_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float64: F64, torch.int64: I64}


class _CudaView:
    """Zero-copy torch view of device memory owned by the C++ graph."""

    def __init__(self, ptr, n, typestr="<f4"):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 2}


def device_view(ptr, n, device, dtype=torch.float32):
    if dtype == torch.bfloat16:  # no typestr for bf16: view 16-bit integers, reinterpret
        return torch.as_tensor(_CudaView(ptr, n, "<i2"), device=device).view(torch.bfloat16)
    return torch.as_tensor(_CudaView(ptr, n), device=device)


def plan_buckets(param_offsets, layers, total, min_bucket_elems=0):
    """Bucket boundaries over the flat gradient buffer in the order the backward pass completes them.

    param_offsets: element offset of every parameter in creation order (embedding, then 9 per
    block, then final norm and, if untied, the head), as laid out by TransformerLM.
    Returns [(event_key, start, end)], event_key being the after_block() index that completes
    the range: `layers` for final norm + head, l for block l, -1 for the embedding.
    Adjacent block ranges are merged until a bucket holds at least min_bucket_elems elements.
    """
    emb_end = param_offsets[1]
    block_starts = [param_offsets[1 + 9 * l] for l in range(layers)]
    tail_start = param_offsets[1 + 9 * layers]
    buckets = [(layers, tail_start, total)]
    hi = tail_start
    pending_hi = hi
    for l in range(layers - 1, -1, -1):
        lo = block_starts[l]
        if pending_hi - lo >= min_bucket_elems or l == 0:
            buckets.append((l, lo, pending_hi))
            pending_hi = lo
    buckets.append((-1, 0, emb_end))
    return buckets


def param_offsets(shapes):
    """Element offsets of parameters laid out back to back with 64-element alignment."""
    offs, pos = [], 0
    for s in shapes:
        n = 1
        for d in s:
            n *= d
        offs.append(pos)
        pos += (n + 63) // 64 * 64
    return offs, pos


# ---------------------------------------------------------------------------------------------
# backends
# ---------------------------------------------------------------------------------------------
class TorchBackend:
    """torch.distributed process group (gloo on CPU tensors, nccl on CUDA tensors)."""

    def __init__(self, group=None, comm_stream=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.comm_stream = comm_stream
        self.pending = []
        self.launched = 0
        self._gloo = dist.is_initialized() and dist.get_backend(group) == "gloo"

    def _run(self, fn):
        if self.comm_stream is not None:
            with torch.cuda.stream(self.comm_stream):
                w = fn()
        else:
            w = fn()
        self.launched += 1
        if w is not None:
            self.pending.append(w)

    def all_reduce(self, view):
        self._run(lambda: dist.all_reduce(view, op=dist.ReduceOp.SUM, group=self.group, async_op=True))

    def reduce_scatter(self, view, piece):
        """view: the whole bucket; piece: this rank's slice of it (receives the sum)."""
        if self._gloo:  # gloo has no reduce-scatter: an all-reduce leaves the same values in the piece
            self.all_reduce(view)
        else:
            self._run(lambda: dist.reduce_scatter_tensor(piece, view, op=dist.ReduceOp.SUM, group=self.group, async_op=True))

    def all_gather(self, view, piece):
        """view: the whole bucket, piece: this rank's slice of it (already up to date)."""
        if self._gloo:
            parts = list(view.chunk(self.world))
            self._run(lambda: dist.all_gather(parts, piece.clone(), group=self.group, async_op=True))
        else:
            self._run(lambda: dist.all_gather_into_tensor(view, piece, group=self.group, async_op=True))

    def broadcast(self, view, root):
        self._run(lambda: dist.broadcast(view, src=dist.get_global_rank(self.group, root) if self.group else root,
                                         group=self.group, async_op=True))

    def group_begin(self):
        pass

    def group_end(self):
        pass

    def wait(self, compute_stream=None, deadline_s=None):
        """Without a deadline: stream-ordered wait on CUDA (no host block), blocking wait on CPU.
        With one: polls on the host and raises EisenError when it passes."""
        works, self.pending = self.pending, []
        if deadline_s is None:
            if compute_stream is not None:
                with torch.cuda.stream(compute_stream):
                    for w in works:
                        w.wait()
            else:
                for w in works:
                    w.wait()
            return
        t0 = time.monotonic()
        for w in works:
            while not w.is_completed():
                if time.monotonic() - t0 > deadline_s:
                    self.abort()
                    raise EisenError("gradient exchange did not finish within %.1f s; communicator aborted" % deadline_s)
                time.sleep(0.001)
            w.wait()

    def poll_error(self):
        pass

    def abort(self):
        self.pending = []


class NcclAbiBackend:
    """The library's eisen_dp_* entry points (NCCL bound at run time) on raw device pointers.
    The 128-byte unique id travels through `exchange_id`, a callable that takes rank 0's bytes (or
    None on the other ranks) and returns rank 0's bytes on every rank."""

    stream_ordered = True  # every collective runs on comm_stream itself: an event recorded there covers it

    def __init__(self, rank, world, comm_stream, exchange_id):
        self.rank, self.world, self.comm_stream = rank, world, comm_stream
        buf = (C.c_char * 128)()
        if rank == 0:
            call("eisen_dp_unique_id", buf)
        raw = exchange_id(bytes(buf.raw) if rank == 0 else None)
        self._h = C.c_void_p()
        call("eisen_dp_init", rank, world, C.create_string_buffer(raw, 128), C.byref(self._h))
        self._s = comm_stream.cuda_stream

    @property
    def launched(self):
        n = C.c_longlong()
        call("eisen_dp_rank_world", self._h, None, None, C.byref(n))
        return n.value

    def all_reduce(self, view):
        call("eisen_dp_allreduce_bucket", self._h, view.data_ptr(), view.numel(), _DT[view.dtype], self._s)

    def reduce_scatter(self, view, piece):
        call("eisen_dp_reduce_scatter", self._h, view.data_ptr(), piece.data_ptr(), piece.numel(), _DT[view.dtype], self._s)

    def all_gather(self, view, piece):
        call("eisen_dp_all_gather", self._h, piece.data_ptr(), view.data_ptr(), piece.numel(), _DT[view.dtype], self._s)

    def broadcast(self, view, root):
        call("eisen_dp_broadcast", self._h, view.data_ptr(), view.numel(), _DT[view.dtype], root, self._s)

    def group_begin(self):
        call("eisen_dp_group_begin")

    def group_end(self):
        call("eisen_dp_group_end")

    def wait(self, compute_stream=None, deadline_s=None):
        if deadline_s is None:
            ev = torch.cuda.Event()
            ev.record(self.comm_stream)
            compute_stream.wait_event(ev)
            return
        call("eisen_dp_wait", self._h, self._s, int(deadline_s * 1000))
        ev = torch.cuda.Event()
        ev.record(self.comm_stream)
        compute_stream.wait_event(ev)

    def poll_error(self):
        call("eisen_dp_poll_error", self._h)

    def abort(self):
        lib().eisen_dp_abort(self._h)

    def close(self):
        if self._h:
            lib().eisen_dp_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class StepHandshake:
    """Host-side check, once per step, that every rank is at the same step and has enqueued the
    same collectives: each rank writes `step:launched:elements` under its own key of a key-value
    store (torch.distributed's c10d Store) and reads its peers' keys with a deadline.  A peer that
    left shows as a timeout, a peer that skipped (or added) a bucket as a mismatch; both raise
    EisenError before this rank blocks on a collective that cannot complete."""

    def __init__(self, store, rank, world, timeout_s=30.0, prefix="eisen/hs"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix

    def _key(self, step, rank):
        return "%s/%d/%d" % (self.prefix, step, rank)

    def check(self, step, launched, elements):
        mine = "%d:%d:%d" % (step, launched, elements)
        self.store.set(self._key(step, self.rank), mine)
        for r in range(self.world):
            if r == self.rank:
                continue
            k = self._key(step, r)
            try:
                self.store.wait([k], datetime.timedelta(seconds=self.timeout_s))
                theirs = self.store.get(k).decode()
            except Exception as e:  # c10d raises its own timeout types
                raise EisenError("rank %d did not reach step %d within %.1f s (%s)" % (r, step, self.timeout_s, type(e).__name__))
            if theirs != mine:
                raise EisenError("rank %d is out of step: it recorded step:collectives:elements = %s, this rank %s"
                                 % (r, theirs, mine))
        if step >= 2:  # forget the records of two steps ago
            try:
                self.store.delete_key(self._key(step - 2, self.rank))
            except Exception:
                pass


# ---------------------------------------------------------------------------------------------
# exchanges
# ---------------------------------------------------------------------------------------------
class _Exchange:
    def __init__(self, flat_grads, buckets, backend=None, group=None, comm_stream=None, handshake=None):
        self.flat = flat_grads
        self.order = [k for k, _, _ in buckets]
        self.buckets = {k: (a, b) for k, a, b in buckets}
        self.cuda = flat_grads.is_cuda
        if backend is None:
            if comm_stream is None and self.cuda:
                comm_stream = torch.cuda.Stream()
            backend = TorchBackend(group, comm_stream if self.cuda else None)
        self.backend = backend
        self.comm_stream = getattr(backend, "comm_stream", None)
        self.world, self.rank = backend.world, backend.rank
        self.handshake = handshake
        self.enabled = True
        self.step_no = 0
        self.skip_keys = set()  # fault injection for the host-side tests: buckets this rank "forgets"
        self._launched0 = backend.launched
        self._elements = 0

    def _comm_waits_for_compute(self, compute_stream):
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(compute_stream)
            self.comm_stream.wait_event(ev)

    def _handshake(self):
        if self.handshake is not None:
            try:
                self.handshake.check(self.step_no, self.backend.launched - self._launched0, self._elements)
            except EisenError:
                self.backend.abort()
                raise
        self.step_no += 1
        self._launched0 = self.backend.launched
        self._elements = 0

    def grad_scale(self):
        return 1.0 / float(self.world)


class BucketedAllReduce(_Exchange):
    def on_block_done(self, key, compute_stream=None):
        """Call when the gradients of `key` are final; starts the bucket's all-reduce if one ends here."""
        if not self.enabled or self.world == 1 or key not in self.buckets or key in self.skip_keys:
            return
        a, b = self.buckets[key]
        self._comm_waits_for_compute(compute_stream)
        self.backend.all_reduce(self.flat[a:b])
        self._elements += b - a

    def finish(self, compute_stream=None, deadline_s=None):
        """Handshake, then make the compute stream wait for every bucket (no host synchronisation
        on CUDA unless a deadline is given)."""
        if self.world == 1:
            return
        self._handshake()
        self.backend.wait(compute_stream, deadline_s)


class ShardedExchange(_Exchange):
    """ZeRO-1 over the flat buffers.  `optimizer` has begin_step(), sumsq_piece(i, accumulate,
    stream), step_piece(i, max_norm, grad_scale) over the pieces returned by `pieces()` (in bucket
    order) and a one-element float64 `sumsq` tensor; on the GPU that is eisen_b200.graph.ShardedAdamW.
    `gather`: the flat buffer all-gathered after the update (the bf16 weights the kernels read; the
    f32 weights in the CPU tests).  `exact_ranges`: element ranges (the norm weights) that the
    kernels read from `flat_w` in f32 and that are therefore broadcast from their owners as well."""

    def __init__(self, flat_grads, buckets, gather, flat_w=None, exact_ranges=(), **kw):
        super().__init__(flat_grads, buckets, **kw)
        self.gather, self.flat_w = gather, flat_w
        for k, (a, b) in self.buckets.items():
            if (b - a) % (self.world * 8):
                raise EisenError("bucket %d of %d elements does not split into %d 16-byte aligned pieces" % (k, b - a, self.world))
        # broadcast list: (lo, hi, owner) for every intersection of an exact range with a piece
        self.exact = []
        for lo, hi in exact_ranges:
            for k in self.order:
                a, b = self.buckets[k]
                per = (b - a) // self.world
                for r in range(self.world):
                    x, y = max(lo, a + r * per), min(hi, a + (r + 1) * per)
                    if x < y:
                        self.exact.append((x, y, r))
        self._first = True

    def piece(self, key, rank=None):
        a, b = self.buckets[key]
        per = (b - a) // self.world
        r = self.rank if rank is None else rank
        return a + r * per, a + (r + 1) * per

    def pieces(self):
        return [self.piece(k) for k in self.order]

    def on_block_done(self, key, compute_stream=None, optimizer=None):
        if not self.enabled or key not in self.buckets or key in self.skip_keys:
            return
        a, b = self.buckets[key]
        lo, hi = self.piece(key)
        self._comm_waits_for_compute(compute_stream)
        if self.world > 1:
            self.backend.reduce_scatter(self.flat[a:b], self.flat[lo:hi])
            self._elements += b - a
        if optimizer is not None:  # this piece's share of the squared norm, right behind its reduction
            if not self.cuda and self.world > 1:
                self.backend.wait()  # CPU tensors have no stream order: the sum must have landed
            optimizer.sumsq_piece(self.order.index(key), not self._first, self.comm_stream)
            self._first = False

    def finish_and_step(self, optimizer, max_norm, compute_stream=None, deadline_s=None, overlap=False):
        """Squared-norm all-reduce, the optimizer on this rank's pieces, broadcast of the exact (f32)
        ranges, then the all-gather of the updated weights bucket by bucket in forward order.
        overlap=False: the compute stream waits for all of it.  overlap=True (stream-ordered
        backends): it waits for nothing here; wait_for_block(l), called from the model's forward
        hook, makes it wait for exactly the bucket block l reads, so the gathers of later blocks run
        beside the next step's forward pass."""
        self._first = True
        if self.world > 1:
            if max_norm > 0.0:
                self.backend.all_reduce(optimizer.sumsq)
                self._elements += 1
            self._handshake()
        self.backend.wait(compute_stream, deadline_s)
        optimizer.begin_step()
        for i in range(len(self.order)):
            optimizer.step_piece(i, max_norm, self.grad_scale())
        if self.world == 1:
            return
        overlap = overlap and self.cuda and getattr(self.backend, "stream_ordered", False)
        self._comm_waits_for_compute(compute_stream)
        self._gather_events = {}
        if self.exact and self.flat_w is not None:
            self.backend.group_begin()
            for x, y, r in self.exact:
                self.backend.broadcast(self.flat_w[x:y], r)
            self.backend.group_end()
        for key in reversed(self.order):  # forward order: embedding, blocks from first to last, final norm + head
            a, b = self.buckets[key]
            lo, hi = self.piece(key)
            self.backend.all_gather(self.gather[a:b], self.gather[lo:hi])
            if overlap:
                ev = torch.cuda.Event()
                ev.record(self.comm_stream)
                self._gather_events[key] = ev
        if not overlap:
            self.backend.wait(compute_stream, deadline_s)
        self._launched0 = self.backend.launched

    def wait_for_block(self, l, compute_stream):
        """Forward hook of an overlapped step: block l (-1 embedding, `layers` final norm + head) is
        about to read its weights; wait for the gather of the bucket that holds them."""
        evs = getattr(self, "_gather_events", None)
        if not evs:
            return
        block_keys = sorted(k for k in self.order if 0 <= k < max(self.order))
        if l < 0:
            key = -1
        elif l >= max(self.order):
            key = max(self.order)
        else:
            key = max([k for k in block_keys if k <= l], default=block_keys[0])
        # buckets were gathered in forward order on one stream: waiting for this one covers the earlier ones
        ev = evs.pop(key, None)
        if ev is not None:
            compute_stream.wait_event(ev)
            for k in [k for k in evs if k < key]:
                evs.pop(k)

    def wait_all(self, compute_stream):
        """Makes the compute stream wait for every outstanding gather (end of training, checkpoints)."""
        evs = getattr(self, "_gather_events", None)
        if evs:
            for ev in evs.values():
                compute_stream.wait_event(ev)
            evs.clear()

    def gather_master(self, compute_stream=None):
        """All-gathers the f32 master weights (for a checkpoint: under ZeRO-1 a rank's master copy
        is current only inside its own pieces)."""
        if self.world == 1 or self.flat_w is None:
            return
        if compute_stream is not None:
            self.wait_all(compute_stream)
        self._comm_waits_for_compute(compute_stream)
        for key in self.order:
            a, b = self.buckets[key]
            lo, hi = self.piece(key)
            self.backend.all_gather(self.flat_w[a:b], self.flat_w[lo:hi])
        self.backend.wait(compute_stream, None)
        self._launched0 = self.backend.launched
