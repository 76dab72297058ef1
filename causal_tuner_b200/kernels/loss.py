"""Tiled lm_head projection + weighted cross-entropy; the full-sequence logits never exist.

Drop-in for the fused branch of the reference's kernels/loss.py (`active_rows`, `row_count`,
`projection_loss`). Only the "fused" implementation with a frozen head is covered.
"""

import torch


def active_rows(weights, device=None):
    """Rows with positive weight: a slice when they are contiguous (or all / none), else indices
    (kernels/loss.py:6-16). Selection happens on the host before the transfer."""
    indices = torch.nonzero(weights.flatten() > 0, as_tuple=False).flatten()
    count = len(indices)
    if not count or count == weights.numel():
        return slice(0, count)
    if weights.device.type == "cpu":
        first, last = int(indices[0]), int(indices[-1])
        if last - first + 1 == count:
            return slice(first, last + 1)
    return indices.to(device) if device is not None else indices


def row_count(rows):
    return rows.stop - rows.start if isinstance(rows, slice) else len(rows)


def projection_loss(hidden, head, targets, weights, *, token_budget=128, compute_dtype=torch.bfloat16,
                    implementation="fused", cut_chunk_size=0, reuse_hidden=False, rows=None):
    """Sum over rows of weights * CE(hidden @ head.T, targets), `token_budget` rows of logits at a time
    (kernels/loss.py:23-66). reuse_hidden lets the cached hidden gradient overwrite `hidden`."""
    if token_budget <= 0:
        raise ValueError("loss_token_budget must be positive")
    if implementation != "fused":
        raise ValueError("Unsupported projection-loss backend")
    if cut_chunk_size:
        raise ValueError("cut_chunk_size applies only to the cut backend")
    if not hidden.is_cuda:
        raise RuntimeError("causal_tuner_b200.projection_loss runs on CUDA tensors only; there is no CPU path")
    rows = active_rows(weights, hidden.device) if rows is None else rows
    from .loss_cuda import FusedProjectionLoss
    if not torch.is_grad_enabled():
        hidden, head = hidden.detach(), head.detach()
    if reuse_hidden and hidden.requires_grad and (hidden.is_leaf or hidden._base is not None or not hidden.is_contiguous()):
        raise ValueError("Hidden reuse requires an exclusive contiguous non-leaf tensor")
    return FusedProjectionLoss.apply(hidden, head, targets, weights, token_budget, compute_dtype, reuse_hidden, rows)[0]
