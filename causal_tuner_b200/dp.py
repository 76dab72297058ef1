"""Batch data parallelism for the adapter gradients: one process per GPU, one exchange step.

Every rank holds a full replica (frozen NF4 base + fp32 adapters) and runs the projection /
MLP operators on its own packed rows. The only collective is a SUM all-reduce of the fp32
LoRA gradients (plus, for a trainer, the scalar loss weight and loss) - the insertion point
is between the last micro-batch backward and the gradient division of the reference's
Trainer.update (training/engine.py:90-97), which then yields exactly the single-device
weighted mean. The reference itself is single-device; this module is the added exchange.

Gradients are packed into flat fp32 buckets so that a collective moves tens of megabytes,
and each bucket's all-reduce is issued asynchronously as soon as it is full, so that the
collectives of early buckets overlap whatever the caller computes next (NCCL over
NVLink/NVSwitch on GPUs, gloo on CPU ranks in the tests).
"""

import torch
import torch.distributed as dist


class GradientExchange:
    """SUM all-reduce of a list of gradient tensors through flat buckets.

    >>> exchange = GradientExchange(bucket_bytes=64 << 20)
    >>> exchange.add(da); exchange.add(db)      # may launch a bucket's collective
    >>> exchange.finish()                       # launches the rest, waits, writes results back in place
    """

    def __init__(self, group=None, bucket_bytes=64 << 20):
        if bucket_bytes <= 0:
            raise ValueError("bucket_bytes must be positive")
        self.group, self.bucket_bytes = group, bucket_bytes
        self._pending, self._pending_bytes, self._inflight = [], 0, []
        self.collectives = 0

    @property
    def world_size(self):
        return dist.get_world_size(self.group) if dist.is_available() and dist.is_initialized() else 1

    def add(self, gradient):
        if gradient.dtype != torch.float32:
            raise TypeError("adapter gradients are exchanged in fp32")
        if self.world_size == 1:
            return
        self._pending.append(gradient)
        self._pending_bytes += gradient.numel() * 4
        if self._pending_bytes >= self.bucket_bytes:
            self._launch()

    def _launch(self):
        if not self._pending:
            return
        tensors, self._pending, self._pending_bytes = self._pending, [], 0
        if len(tensors) == 1 and tensors[0].is_contiguous():
            flat = tensors[0].view(-1)
        else:
            flat = torch.cat([t.reshape(-1) for t in tensors])
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        self.collectives += 1
        self._inflight.append((work, flat, tensors))

    def finish(self):
        """Flush the last bucket, wait for every collective and copy the sums back into the gradients."""
        self._launch()
        for work, flat, tensors in self._inflight:
            work.wait()
            if len(tensors) == 1 and flat.data_ptr() == tensors[0].data_ptr():
                continue
            offset = 0
            for tensor in tensors:
                count = tensor.numel()
                tensor.copy_(flat[offset:offset + count].view_as(tensor))
                offset += count
        self._inflight = []


class BucketPlan:
    """Fixed assignment of a trainer's gradient tensors to flat fp32 buckets.

    Tensors are taken in REVERSE parameter order - the order in which a backward pass finishes
    them - and packed into buckets of at least `bucket_bytes`. The plan depends on the shapes
    only, so every rank builds the same one, and because `PlannedExchange` launches buckets
    strictly in plan order the sequence of collectives is the same on every rank whatever
    happens to one of them. The flat buffers are allocated once and reused by every update."""

    def __init__(self, shapes, device, bucket_bytes=64 << 20):
        if bucket_bytes <= 0:
            raise ValueError("bucket_bytes must be positive")
        self.shapes = [tuple(shape) for shape in shapes]
        self.slot = [None] * len(self.shapes)          # tensor index -> (bucket, offset, count)
        self.members, sizes = [[]], [0]
        for index in reversed(range(len(self.shapes))):
            count = 1
            for extent in self.shapes[index]:
                count *= extent
            if sizes[-1] * 4 >= bucket_bytes:
                self.members.append([])
                sizes.append(0)
            self.slot[index] = (len(self.members) - 1, sizes[-1], count)
            self.members[-1].append(index)
            sizes[-1] += count
        self.buffers = [torch.empty(size, device=device, dtype=torch.float32) for size in sizes]

    def view(self, index):
        bucket, offset, count = self.slot[index]
        return self.buffers[bucket][offset:offset + count].view(self.shapes[index])


class PlannedExchange:
    """One update's SUM all-reduce over a `BucketPlan`.

    `add(index, gradient)` copies a finished gradient into its slot; a bucket is all-reduced
    (asynchronously) as soon as it is complete AND every earlier bucket has been launched.
    `finish(extra)` launches what is left, all-reduces the small `extra` tensor last (loss,
    weight and a failure flag travel there), waits, and returns the views that now hold the sums.
    `flush()` is for a rank whose update failed: it launches every bucket not yet launched,
    whatever it contains, so that the peers' collectives complete and they can read the flag."""

    def __init__(self, plan, group=None):
        self.plan, self.group = plan, group
        self._missing = [len(members) for members in plan.members]
        self._next, self._inflight = 0, []
        self.collectives = 0

    def add(self, index, gradient):
        bucket = self.plan.slot[index][0]
        self.plan.view(index).copy_(gradient)
        self._missing[bucket] -= 1
        self._advance()

    def _advance(self, force=False):
        while self._next < len(self._missing) and (force or self._missing[self._next] <= 0):
            work = dist.all_reduce(self.plan.buffers[self._next], op=dist.ReduceOp.SUM, group=self.group, async_op=True)
            self._inflight.append(work)
            self.collectives += 1
            self._next += 1

    def flush(self):
        self._advance(force=True)

    def finish(self, extra=None):
        if any(self._missing[self._next:]):
            raise RuntimeError("gradient exchange finished before every gradient was added")
        self._advance()
        if extra is not None:
            self._inflight.append(dist.all_reduce(extra, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            self.collectives += 1
        for work in self._inflight:
            work.wait()
        self._inflight = []
        return [self.plan.view(index) for index in range(len(self.plan.shapes))]


def exchange_gradients(gradients, group=None, bucket_bytes=64 << 20):
    """In-place SUM all-reduce of `gradients` across the ranks of `group`; returns the number of collectives."""
    exchange = GradientExchange(group, bucket_bytes)
    for gradient in gradients:
        exchange.add(gradient)
    exchange.finish()
    return exchange.collectives


def shard_rows(total_rows, rank, world_size):
    """Contiguous [start, stop) slice of packed rows owned by `rank`; remainders go to the first ranks."""
    if not 0 <= rank < world_size:
        raise ValueError("rank outside the world")
    base, extra = divmod(total_rows, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def row_costs(attention_mask, segment_ids=None, *, linear=1.0, quadratic=None, width=4096):
    """Relative cost of each packed row: `linear` per valid token (projections, MLP, loss) plus
    `quadratic` per pair of tokens that attend to each other, i.e. the sum over the row's
    documents of length^2 / 2 (causal attention inside a document, none across documents).
    The default `quadratic` = 1 / (6 * width) weighs a full-width single document about 8 %
    above a row of short documents, the ratio of attention to projection FLOP in a decoder
    whose MLP is 3.5 times its hidden width."""
    from .segments import canonical_segments, runs
    if quadratic is None:
        quadratic = 1.0 / (6.0 * width)
    segments = canonical_segments(attention_mask, segment_ids)
    costs = [0.0] * segments.shape[0]
    for row, start, end in runs(segments):
        length = end - start
        costs[row] += linear * length + quadratic * length * length / 2
    return costs


def balance_rows(costs, world_size):
    """Assign packed rows to ranks so that the largest per-rank cost is small: rows in order of
    decreasing cost, each to the least-loaded rank that still has room, every rank getting
    ceil(len(costs) / world_size) rows at most (the per-rank batch shape stays fixed, which keeps
    the exchange step aligned). Returns one ascending list of row indices per rank; ties break
    towards the lower rank and the lower row index, so every rank computes the same assignment."""
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    capacity = -(-len(costs) // world_size)
    loads, members = [0.0] * world_size, [[] for _ in range(world_size)]
    for row in sorted(range(len(costs)), key=lambda r: (-costs[r], r)):
        open_ranks = [r for r in range(world_size) if len(members[r]) < capacity]
        rank = min(open_ranks, key=lambda r: (loads[r], r))
        members[rank].append(row)
        loads[rank] += costs[row]
    return [sorted(rows) for rows in members]
