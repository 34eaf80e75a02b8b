"""Batch-sharded data parallelism for the checkpointed training step.

Sequences are independent and the loss is a mean over tokens, so a global batch of B
sequences splits into B/g contiguous slices, one per rank; every rank scales its loss by
1/g and the ranks exchange exactly one thing: the SUM of their fp32 parameter gradients.
The gradients of one transformer block are one contiguous range of the flat gradient
buffer (a "bucket"); a block's bucket is all-reduced as soon as that block's backward has
been enqueued, which overlaps the transfer with the recompute + backward of the next
block. Embeddings, final norm and head form the last bucket.

The reference has no multi-GPU path; its closest relative is gradient accumulation over
micro-batches with the loss pre-scaled by 1/accum (tools/mtstudio.cpp:456-474), which is
the same identity.

The collectives go through torch.distributed (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np


def shard_range(global_batch: int, rank: int, world: int) -> Tuple[int, int]:
    """Sequences [lo, hi) of the global batch that `rank` owns."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} / world {world}")
    if global_batch % world:
        raise ValueError(f"global batch {global_batch} does not divide over {world} ranks")
    per = global_batch // world
    return rank * per, (rank + 1) * per


def shard_tokens(stream: np.ndarray, global_batch: int, seq_len: int, rank: int, world: int):
    """Local (ids, targets) of a token stream of global_batch*seq_len + 1 ids: inputs are
    stream[:-1], targets stream[1:], cut into sequences of seq_len (the reference's pattern,
    tests/test_checkpointing.cpp:63-64)."""
    n = global_batch * seq_len
    if len(stream) != n + 1:
        raise ValueError("token stream must hold global_batch*seq_len + 1 ids")
    lo, hi = shard_range(global_batch, rank, world)
    return stream[lo * seq_len:hi * seq_len], stream[lo * seq_len + 1:hi * seq_len + 1]


class BucketAllReducer:
    """Starts the all-reduce of block bucket i when told that block i finished its backward.

    buckets: torch tensors viewing the gradient ranges, block 0 .. block L-1, then "rest".
    Checkpointed segments finish in reverse forward order: the k-th finished segment is
    block L-1-k.
    """

    def __init__(self, buckets: Sequence, dist_module=None):
        import torch.distributed as dist
        self.dist = dist_module or dist
        self.buckets = list(buckets)
        self.n_blocks = len(self.buckets) - 1
        self.pending: List = []
        self.order: List[int] = []  # bucket indices in launch order (for tests)
        # Under gradient accumulation the buckets are complete only after the last
        # micro-step: the launcher clears this for the earlier ones.
        self.enabled = True

    def on_segment(self, k: int):
        if not self.enabled:
            return
        i = self.n_blocks - 1 - k
        if 0 <= i < self.n_blocks:
            self._launch(i)

    def _launch(self, i: int):
        self.order.append(i)
        self.pending.append(self.dist.all_reduce(self.buckets[i], op=self.dist.ReduceOp.SUM, async_op=True))

    def finish(self):
        """All-reduce what has not been sent yet (the last bucket and, for models run without
        checkpointing, every block), then wait for everything."""
        sent = set(self.order)
        for i in range(len(self.buckets)):
            if i not in sent:
                self._launch(i)
        for h in self.pending:
            h.wait()
        self.pending.clear()
        self.order.clear()
