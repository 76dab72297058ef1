"""lm_head logits tile -> weighted CE -> gradient tile -> hidden gradient, tile by tile.

Drop-in for the reference's kernels/loss_cuda.py (`weighted_ce`, `FusedProjectionLoss`) with a
frozen head: logits = x @ head.T and dHidden = dLogits @ head run on the tcgen05 GEMM
(ct_matmul), the statistics / gradient pass is ct_weighted_ce. The hidden gradient is computed
in the forward pass and cached, as in the reference (kernels/loss_cuda.py:81-162).
"""

import torch

from .. import _lib
from .linear import cast, matmul
from .loss import row_count


def weighted_ce(logits, targets, weights, *, gradient, loss=None, partials=None):
    """Per-row weighted losses; with `gradient` the logits are overwritten by their derivatives
    (kernels/loss_cuda.py:58-72). `partials` is accepted for signature compatibility and unused."""
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


class FusedProjectionLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, head, targets, weights, tile, dtype, reuse_hidden, active):
        if ctx.needs_input_grad[1]:
            raise NotImplementedError("causal_tuner_b200 covers a frozen lm_head (adapter training) only")
        h = hidden.reshape(-1, hidden.shape[-1])
        t, w = targets.flatten(), weights.flatten()
        count = row_count(active)
        contiguous = isinstance(active, slice)
        want_dh = ctx.needs_input_grad[0]
        reuse_hidden = reuse_hidden and want_dh
        dh = None
        if want_dh:
            dh = h if reuse_hidden else (torch.empty_like(h) if contiguous else torch.zeros_like(h))
        losses = torch.empty(count, device=hidden.device, dtype=torch.float32)
        rows = min(tile, count)
        direct = contiguous and dh is not None and dh.dtype == dtype
        if rows:
            matrix = cast(head, dtype)
            workspace = torch.empty((rows, matrix.shape[0]), device=hidden.device, dtype=dtype)
            signals = None if dh is None or direct else torch.empty((rows, h.shape[-1]), device=hidden.device, dtype=dtype)
        for start in range(0, count, tile):
            size = min(tile, count - start)
            if contiguous:
                indices = slice(active.start + start, active.start + start + size)
                x, target, weight = cast(h[indices], dtype), t[indices], w[indices]
            else:
                indices = active[start:start + size]
                x = cast(torch.index_select(h, 0, indices), dtype)
                target, weight = torch.index_select(t, 0, indices), torch.index_select(w, 0, indices)
            logits = workspace[:size]
            matmul(x, matrix.T, out=logits)
            weighted_ce(logits, target, weight, gradient=dh is not None, loss=losses[start:start + size])
            if dh is not None:
                if direct:
                    matmul(logits, matrix, out=dh[indices])
                else:
                    matmul(logits, matrix, out=signals[:size])
                    if contiguous:
                        dh[indices].copy_(signals[:size])
                    else:
                        dh.index_copy_(0, indices, signals[:size].to(dh.dtype))
        if dh is not None and contiguous:
            if active.start:
                dh[:active.start].zero_()
            if active.stop < len(h):
                dh[active.stop:].zero_()
        if reuse_hidden:
            if not contiguous and count != len(h):
                dh.mul_((w > 0).to(dh.dtype)[:, None])   # inactive rows still hold hidden values, not gradients
            ctx.mark_dirty(hidden)
            dh = hidden
        elif dh is not None:
            dh = dh.reshape(hidden.shape)
        if dh is not None:
            ctx.mark_non_differentiable(dh)
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(dh)
        return losses.sum(), dh

    @staticmethod
    def backward(ctx, upstream, unused):
        dh, = ctx.saved_tensors
        scale = float(upstream)
        if dh is not None and scale != 1:
            dh = dh * upstream
        return dh, None, None, None, None, None, None, None
