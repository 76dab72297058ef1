"""Packed-row bookkeeping shared by the model and the trainer: contiguous valid runs, positions
that restart at every document, next-token targets that never cross a document boundary.
Same functions as the reference's data/segments.py:6-58."""

import torch
from torch.nn import functional as F


def canonical_segments(mask, labels=None):
    valid = mask.bool()
    if valid.ndim != 2:
        raise ValueError("attention_mask must have shape [batch, sequence]")
    labels = torch.zeros_like(mask) if labels is None else labels
    if labels.shape != mask.shape:
        raise ValueError("segment_ids must match attention_mask")
    previous = F.pad(valid[:, :-1], (1, 0), value=False)
    changed = F.pad(labels[:, 1:] != labels[:, :-1], (1, 0), value=True)
    starts = valid & (~previous | changed)
    return starts.to(torch.int32).cumsum(1).to(torch.int32) * valid


def position_ids(segments):
    index = torch.arange(segments.shape[1], device=segments.device).expand_as(segments)
    previous = F.pad(segments[:, :-1], (1, 0))
    starts = torch.where((segments != previous) & (segments > 0), index, 0)
    return torch.where(segments > 0, index - starts.cummax(1).values, 0)


def runs(segments):
    """((row, start, end), ...) of every valid run; host metadata made once per batch."""
    result = []
    for row, labels in enumerate(segments.cpu().tolist()):
        start = 0
        while start < len(labels):
            end = start + 1
            while end < len(labels) and labels[end] == labels[start]:
                end += 1
            if labels[start] > 0:
                result.append((row, start, end))
            start = end
    return tuple(result)


def prediction_targets(batch):
    ids = batch["input_ids"]
    valid = batch["attention_mask"].bool()
    segments = canonical_segments(valid, batch.get("segment_ids"))
    labels = batch.get("labels", ids)
    weights = batch.get("loss_weights")
    weights = torch.ones_like(ids, dtype=torch.float32) if weights is None else weights.float()
    edges = valid[:, :-1] & valid[:, 1:] & (segments[:, :-1] == segments[:, 1:])
    targets = F.pad(labels[:, 1:], (0, 1))
    weights = F.pad(weights[:, 1:] * edges, (0, 1))
    weights = weights * (targets != -100)
    return torch.where(weights > 0, targets, 0).long(), weights
