"""Packed-row bookkeeping shared by the model and the trainer.

A packed row holds several documents end to end. Everything downstream (positions, attention
spans, next-token targets) works from one canonical labelling: maximal runs of valid tokens that
share a raw label are numbered 1, 2, ... per row, padding is 0. The functions keep the names and
results of the reference's data/segments.py (:6-58), which the reference's trainer and model
import; tests/test_host_logic.py holds them against the oracle's restatement.
"""

import torch


def _shifted_right(values, fill):
    """values[:, i-1] at column i, `fill` in column 0."""
    first = torch.full_like(values[:, :1], fill)
    return torch.cat((first, values[:, :-1]), dim=1)


def canonical_segments(mask, labels=None):
    """int32 [batch, sequence]: run number of every valid token (from 1, per row), 0 where mask is 0.
    A run ends where validity ends or the raw label changes; raw label 0 is an ordinary label."""
    if mask.ndim != 2:
        raise ValueError("attention_mask must have shape [batch, sequence]")
    if labels is None:
        labels = torch.zeros_like(mask)
    elif labels.shape != mask.shape:
        raise ValueError("segment_ids must match attention_mask")
    valid = mask.bool()
    after_gap = ~_shifted_right(valid, False)
    new_label = labels != _shifted_right(labels, 0)
    new_label[:, 0] = True
    opens_run = valid & (after_gap | new_label)
    return (opens_run.int().cumsum(dim=1) * valid).to(torch.int32)


def position_ids(segments):
    """Offset of every token inside its run (0 for padding): positions restart at each document."""
    columns = torch.arange(segments.shape[1], device=segments.device).expand_as(segments)
    opens_run = (segments > 0) & (segments != _shifted_right(segments, 0))
    run_start = torch.where(opens_run, columns, torch.zeros_like(columns)).cummax(dim=1).values
    return torch.where(segments > 0, columns - run_start, torch.zeros_like(columns))


def runs(segments):
    """((row, start, end), ...) for every run of equal non-zero labels, in row-major order. Host
    metadata: computed once per batch and shared by all layers."""
    table = segments.detach().to("cpu", torch.int64)
    rows, width = table.shape
    if rows == 0 or width == 0:
        return ()
    zero = table.new_zeros(rows, 1)
    padded = torch.cat((zero, table, zero), dim=1)
    edge_row, edge_column = (padded[:, 1:] != padded[:, :-1]).nonzero(as_tuple=True)
    if edge_row.numel() < 2:
        return ()
    # consecutive edges of one row bound a stretch of equal labels; keep the labelled stretches
    same_row = edge_row[1:] == edge_row[:-1]
    row, start, end = edge_row[:-1][same_row], edge_column[:-1][same_row], edge_column[1:][same_row]
    keep = table[row, start] > 0
    return tuple(zip(row[keep].tolist(), start[keep].tolist(), end[keep].tolist()))


def prediction_targets(batch):
    """(targets int64, weights fp32), both [batch, sequence]: the token to predict at every position and
    how much it counts. Explicit `prediction_targets` / `prediction_weights` win; otherwise position i
    predicts `labels[i + 1]` (default: the input ids) when i and i + 1 are valid tokens of the same
    run, weighted by `loss_weights[i + 1]` (or `assistant_masks`, or 1). Targets equal to -100 and
    unweighted positions get target 0 and weight 0."""
    ids = batch["input_ids"]
    valid = batch["attention_mask"].bool()
    if "prediction_targets" in batch:
        targets = batch["prediction_targets"]
        weights = batch["prediction_weights"].float() * valid
    else:
        segments = canonical_segments(valid, batch.get("segment_ids"))
        labels = batch.get("labels", ids)
        if "loss_weights" in batch and batch["loss_weights"] is not None:
            per_token = batch["loss_weights"].float()
        else:
            per_token = torch.ones_like(ids, dtype=torch.float32)
            if "assistant_masks" in batch:
                per_token = per_token * batch["assistant_masks"]
        same_run = valid[:, 1:] & valid[:, :-1] & (segments[:, 1:] == segments[:, :-1])
        last = torch.zeros_like(labels[:, :1])
        targets = torch.cat((labels[:, 1:], last), dim=1)
        weights = torch.cat((per_token[:, 1:] * same_run, torch.zeros_like(per_token[:, :1])), dim=1)
    weights = weights * (targets != -100)
    targets = torch.where(weights > 0, targets, torch.zeros_like(targets))
    return targets.long(), weights
