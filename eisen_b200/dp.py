"""Data-parallel plumbing: one process per GPU, bucketed gradient all-reduce over torch.distributed.

The reference has no distributed code; this is the exchange step the data-parallel training step
adds.  Every rank holds full replicas and runs the whole forward/backward on its own micro-batch;
the flat f32 gradient buffer is cut into buckets in backward order (head and final norm first,
then the blocks from last to first, then the embedding).  A bucket is all-reduced (sum) on a side
stream as soon as the backward pass has finished writing it, so the exchange overlaps the rest of
the backward; the optimizer folds 1/world into its gradient scale.  NCCL picks its own algorithm;
no kernel of this package touches a peer's memory.

The same class runs on CPU tensors with the gloo backend, which is how the host logic is tested
without GPUs.
"""
import torch
import torch.distributed as dist


class _CudaView:
    """Zero-copy torch view of device memory owned by the C++ graph."""

    def __init__(self, ptr, n, typestr="<f4"):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 2}


def device_view(ptr, n, device):
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


class BucketedAllReduce:
    def __init__(self, flat_grads, buckets, group=None, comm_stream=None):
        self.flat = flat_grads
        self.buckets = {k: (a, b) for k, a, b in buckets}
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.cuda = flat_grads.is_cuda
        self.comm_stream = comm_stream if comm_stream is not None else (torch.cuda.Stream() if self.cuda else None)
        self.pending = []
        self.enabled = True

    def on_block_done(self, key, compute_stream=None):
        """Call when the gradients of `key` are final; starts the bucket's all-reduce if one ends here."""
        if not self.enabled or self.world == 1 or key not in self.buckets:
            return
        a, b = self.buckets[key]
        view = self.flat[a:b]
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(compute_stream)
            self.comm_stream.wait_event(ev)
            with torch.cuda.stream(self.comm_stream):
                self.pending.append(dist.all_reduce(view, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
        else:
            self.pending.append(dist.all_reduce(view, op=dist.ReduceOp.SUM, group=self.group, async_op=True))

    def finish(self, compute_stream=None):
        """Makes the compute stream wait for every bucket (no host synchronisation on CUDA)."""
        if self.cuda:
            with torch.cuda.stream(compute_stream):
                for w in self.pending:
                    w.wait()
        else:
            for w in self.pending:
                w.wait()
        self.pending = []

    def grad_scale(self):
        return 1.0 / float(self.world)


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
