"""Data-parallel plumbing for the row-sharded path: which sequences a rank owns, and the one exchange step
(sum of weight gradients across ranks) as bucketed all-reduces through torch.distributed.

The reference is single-GPU (src/pctx/mod.rs:303-311 takes device 0); rows (sequences) are independent in
every thunk of the path, so ranks need no data-path collective.  Gradient dtype = parameter dtype, as in the
reference (examples/open_llama_3b_train.rs:161-169).
"""
from __future__ import annotations

import datetime

import torch
import torch.distributed as dist


def shard_sequences(n_seq: int, world: int, rank: int):
    """Contiguous block of sequences for `rank`: (first, count).  Earlier ranks take the remainder."""
    base, rem = divmod(n_seq, world)
    first = rank * base + min(rank, rem)
    return first, base + (1 if rank < rem else 0)


def alloc_bucketed_grads(params):
    """Gradient tensors shaped like `params`; each layer's gradients are views of one flat buffer (a bucket).
    The output head (`lm_head`, `head_norm`), whose gradients are the first to be complete in the backward pass,
    gets bucket len(layers); the remaining parameters (the embedding, complete last) bucket len(layers) + 1.
    Returns (grads, buckets)."""
    def carve(named):
        total = sum((t.numel() + 127) // 128 * 128 for _, t in named)
        first = named[0][1]
        flat = torch.zeros(total, dtype=first.dtype, device=first.device)
        out, off = {}, 0
        for k, t in named:
            out[k] = flat[off:off + t.numel()].view(t.shape)
            off += (t.numel() + 127) // 128 * 128
        return out, flat

    grads, buckets = {"layers": []}, []
    for L in params["layers"]:
        g, flat = carve(list(L.items()))
        grads["layers"].append(g)
        buckets.append(flat)
    head_keys = [k for k in ("lm_head", "head_norm") if k in params]
    rest_keys = [k for k in params if k != "layers" and k not in head_keys]
    for keys in (head_keys, rest_keys):
        if keys:
            g, flat = carve([(k, params[k]) for k in keys])
            grads.update(g)
            buckets.append(flat)
    return grads, buckets


class GradReducer:
    """Launches one asynchronous all-reduce per bucket as soon as the bucket is complete, so the exchange
    overlaps the rest of the backward pass; `finish()` waits for all of them.

    What a caller sees when a rank is lost (it exited, or never reached the exchange): nothing hangs for good.  A
    collective that cannot complete ends with an exception, from `reduce_bucket` or from `finish`, no later than
    `timeout_s` seconds after `finish` is called, or after the process group's own timeout where the backend waits
    on the device rather than on the host (NCCL: the timeout given to init_process_group; its watchdog then ends the
    communicator).  The reference has no counterpart (single GPU; any error is a panic, src/spine.rs:1856-1865)."""

    def __init__(self, buckets, group=None, timeout_s: float | None = None):
        self.buckets, self.group, self.pending, self.timeout_s = buckets, group, [], timeout_s
        self.enabled = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1

    def reduce_bucket(self, i: int):
        if self.enabled:
            self.pending.append(dist.all_reduce(self.buckets[i], op=dist.ReduceOp.SUM, group=self.group, async_op=True))

    def finish(self):
        pending, self.pending = self.pending, []
        for w in pending:
            if self.timeout_s is None:
                w.wait()
            elif not w.wait(timeout=datetime.timedelta(seconds=self.timeout_s)):
                raise RuntimeError("gradient exchange did not complete")
