"""lm_head logits tile -> weighted CE -> gradient tile -> hidden / head gradients, tile by tile.

Drop-in for the reference's kernels/loss_cuda.py (`weighted_ce`, `FusedProjectionLoss`, :58-162).
Per tile of at most `tile` supervised rows:

    logits  = x @ head.T                      tcgen05 GEMM (ct_matmul), compute dtype
    losses, logits <- d(losses)/d(logits)     ct_weighted_ce, one pass per row, in place
    d_head (+)= logits.T @ x                  token contraction with fp32 accumulation (ct_matmul),
                                              only when the head trains (kernels/loss_cuda.py:120-121)
    d_hidden[rows] = logits @ head            tcgen05 GEMM, written straight into its destination

Both gradients are finished in the forward pass and cached; backward only scales them.
"""

import torch

from .. import _lib
from .linear import accumulate, cast, matmul
from .loss import row_count


def weighted_ce(logits, targets, weights, *, gradient, loss=None, partials=None):
    """Per-row weighted losses; with `gradient` the logits are overwritten by their derivatives
    (kernels/loss_cuda.py:58-72). The reference's kernel splits a row into 4096-column parts and
    keeps per-part statistics in `partials`; this kernel reduces a row in one block, so the
    argument is accepted and left untouched."""
    _lib.require_cuda(logits, targets, weights)
    rows, vocab = logits.shape
    if not logits.is_contiguous():
        raise ValueError("logits must be contiguous")
    if loss is None:
        loss = torch.empty(rows, device=logits.device, dtype=torch.float32)
    targets = targets.contiguous().long()
    weights = weights.contiguous().float()
    with _lib.on_device(logits):
        _lib.check(_lib.load().ct_weighted_ce(logits.data_ptr(), targets.data_ptr(), weights.data_ptr(), loss.data_ptr(),
                                             rows, vocab, int(bool(gradient)), _lib.code_of(logits.dtype),
                                             _lib.stream_of(logits)))
    return loss


def _clear_unsupervised(gradient, weights):
    """Zero the rows of `gradient` whose weight is not positive (they still hold hidden states)."""
    gradient.mul_((weights > 0).to(gradient.dtype).unsqueeze(-1))


class FusedProjectionLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, head, targets, weights, tile, dtype, reuse_hidden, active):
        _lib.require_cuda(hidden, head)
        flat = hidden.reshape(-1, hidden.shape[-1])
        labels, factors = targets.reshape(-1), weights.reshape(-1)
        total, width = flat.shape
        supervised = row_count(active)
        run = isinstance(active, slice)              # supervised rows form one run: work on views
        want_hidden, want_head = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        in_place = bool(reuse_hidden and want_hidden)
        d_hidden = d_head = None
        if want_hidden:
            d_hidden = flat if in_place else (torch.empty_like(flat) if run else torch.zeros_like(flat))
        if want_head:
            d_head = torch.empty_like(head) if supervised else torch.zeros_like(head)
        losses = torch.empty(supervised, device=hidden.device, dtype=torch.float32)
        held = min(tile, supervised)
        straight = run and d_hidden is not None and d_hidden.dtype == dtype   # GEMM writes its destination rows
        if held:
            matrix = cast(head, dtype)
            logits_buffer = torch.empty((held, matrix.shape[0]), device=hidden.device, dtype=dtype)
            statistics = torch.empty((held, 1), device=hidden.device, dtype=torch.float32)
            staged = None
            if d_hidden is not None and not straight:
                staged = torch.empty((held, width), device=hidden.device, dtype=dtype)
            if not run:
                label_buffer, factor_buffer = labels.new_empty(held), factors.new_empty(held)
        for first in range(0, supervised, tile):
            size = min(tile, supervised - first)
            if run:
                where = slice(active.start + first, active.start + first + size)
                x, label, factor = cast(flat[where], dtype), labels[where], factors[where]
            else:
                where = active[first:first + size]
                x = cast(torch.index_select(flat, 0, where), dtype)
                label = torch.index_select(labels, 0, where, out=label_buffer[:size])
                factor = torch.index_select(factors, 0, where, out=factor_buffer[:size])
            logits = logits_buffer[:size]
            matmul(x, matrix.T, out=logits)
            weighted_ce(logits, label, factor, gradient=want_hidden or want_head, loss=losses[first:first + size],
                        partials=statistics[:size])
            if d_head is not None:
                # before d_hidden: with in-place reuse the next product may overwrite the rows x views
                accumulate(d_head, logits.T, x, add=first > 0)
            if d_hidden is None:
                continue
            if straight:
                matmul(logits, matrix, out=d_hidden[where])
            else:
                matmul(logits, matrix, out=staged[:size])
                if run:
                    d_hidden[where].copy_(staged[:size])
                else:
                    d_hidden.index_copy_(0, where, staged[:size].to(d_hidden.dtype))
        if d_hidden is not None:
            if run:
                d_hidden[:active.start].zero_()
                d_hidden[active.stop:].zero_()
            elif in_place and supervised != total:
                _clear_unsupervised(d_hidden, factors)
        if in_place:
            ctx.mark_dirty(hidden)
            d_hidden = hidden
        elif d_hidden is not None:
            d_hidden = d_hidden.reshape(hidden.shape)
        if d_hidden is not None:
            ctx.mark_non_differentiable(d_hidden)
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(d_hidden, d_head)
        return losses.sum(), d_hidden

    @staticmethod
    def backward(ctx, upstream, unused):
        d_hidden, d_head = ctx.saved_tensors
        if float(upstream) != 1:        # the training call has unit upstream; the cache itself is never modified
            d_hidden = None if d_hidden is None else d_hidden * upstream
            d_head = None if d_head is None else d_head * upstream
        return d_hidden, d_head, None, None, None, None, None, None
