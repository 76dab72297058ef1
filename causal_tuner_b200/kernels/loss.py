"""Tiled lm_head projection + weighted cross-entropy; the full-sequence logits never exist.

Drop-in for the reference's kernels/loss.py (`active_rows`, `row_count`, `projection_loss`,
:6-66): same arguments, same exceptions. Only the "fused" backend exists here, and only on
CUDA tensors.
"""

import torch


def active_rows(weights, device=None):
    """Which flattened rows carry supervision (weight > 0).

    Returns a slice when the supervised rows form one run - including "all of them" and "none" -
    so that callers can work on views; otherwise an index tensor (moved to `device` when given).
    The run test needs the first and last index on the host, so it is only made for host weights;
    device weights with gaps or a partial run always give indices (kernels/loss.py:6-16)."""
    flat = weights.reshape(-1)
    positive = (flat > 0).nonzero().reshape(-1)
    supervised, total = positive.numel(), flat.numel()
    if supervised in (0, total):
        return slice(0, supervised)
    if not flat.is_cuda:
        low, high = positive[0].item(), positive[-1].item()
        if high - low == supervised - 1:
            return slice(low, high + 1)
    return positive if device is None else positive.to(device)


def row_count(rows):
    """Number of rows a selection made by `active_rows` covers."""
    if isinstance(rows, slice):
        return rows.stop - rows.start
    return len(rows)


def projection_loss(hidden, head, targets, weights, *, token_budget=128, compute_dtype=torch.bfloat16,
                    implementation="fused", cut_chunk_size=0, reuse_hidden=False, rows=None):
    """sum_rows weights * CE(hidden @ head.T, targets), at most `token_budget` rows of logits alive at
    a time (kernels/loss.py:23-66). The hidden gradient (and the head gradient when the head trains) is
    produced during the forward pass and cached; `reuse_hidden` lets that cache overwrite `hidden`,
    which must then be a tensor nobody else reads: contiguous, not a leaf, not a view."""
    if token_budget <= 0:
        raise ValueError("loss_token_budget must be positive")
    if implementation != "fused":
        if implementation == "cut":
            raise RuntimeError("The cut backend requires cut-cross-entropy, which this package does not call")
        raise ValueError("Unsupported projection-loss backend")
    if cut_chunk_size:
        raise ValueError("cut_chunk_size applies only to the cut backend")
    if not hidden.is_cuda:
        raise RuntimeError("causal_tuner_b200.projection_loss runs on CUDA tensors only; there is no CPU path")
    if rows is None:
        rows = active_rows(weights, hidden.device)
    if not torch.is_grad_enabled():
        hidden, head = hidden.detach(), head.detach()
    exclusive = not hidden.is_leaf and hidden._base is None and hidden.is_contiguous()
    if reuse_hidden and hidden.requires_grad and not exclusive:
        raise ValueError("Hidden reuse requires an exclusive contiguous non-leaf tensor")
    from .loss_cuda import FusedProjectionLoss
    return FusedProjectionLoss.apply(hidden, head, targets, weights, token_budget, compute_dtype, reuse_hidden, rows)[0]
