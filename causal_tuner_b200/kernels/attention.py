"""Causal attention over packed documents.

Attention itself is a library call here, as it is in the reference: FlashAttention-2's dense and
variable-length kernels (kernels/attention.py:58-93 of the reference). This module only decides
which of the two to call from the document spans of the batch - once per step, shared by every
layer and by checkpoint replays - and provides the small dense fp32 form behind the "vanilla"
setting (kernels/reference.py:11-27), which the whole-step fixtures use.

Layout modes, by increasing amount of data movement:
  "empty"   no valid token;
  "full"    every row is one document covering the whole row  -> flash_attn_func on the batch;
  "packed"  documents tile the flattened rows without gaps    -> flash_attn_varlen_func on views;
  "gaps"    padding between documents                         -> gather, varlen call, scatter.
Bidirectional groups (`attention_end`) are not part of this package.
"""

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class DenseLayout:
    spans: tuple
    mode: str
    offsets: torch.Tensor | None = None      # int32 cumulative document lengths, on the device
    maximum: int = 0                         # longest document
    groups: tuple = ()                       # kept for field compatibility; always empty here


def prepare_dense_layout(shape, spans, device, attention_end=None):
    """Classify `spans` ((row, start, end), ...) of a [rows, width] batch and build the offsets the
    variable-length kernel needs."""
    if attention_end is not None:
        raise NotImplementedError("bidirectional attention groups are not part of this package")
    spans = tuple(spans)
    rows, width = shape
    if len(spans) == 0:
        return DenseLayout(spans, "empty")
    if len(spans) == rows and all(span == (row, 0, width) for row, span in enumerate(spans)):
        return DenseLayout(spans, "full")
    lengths = [end - start for _, start, end in spans]
    cumulative, total = [0], 0
    for length in lengths:
        total += length
        cumulative.append(total)
    # "packed": in flattened token order each document starts where the previous one ended, and
    # together they cover every token
    expected, tiled = 0, True
    for row, start, end in spans:
        if row * width + start != expected:
            tiled = False
            break
        expected = row * width + end
    tiled = tiled and expected == rows * width
    offsets = torch.tensor(cumulative, dtype=torch.int32, device=device)
    return DenseLayout(spans, "packed" if tiled else "gaps", offsets, max(lengths))


def flash_dense(q, k, v, spans, attention_end=None, *, layout=None):
    """q [rows, width, heads, d], k / v [rows, width, 1, d] -> attention output shaped like q."""
    if not q.is_cuda or q.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError("flash_attention_2 requires CUDA and BF16/FP16 inputs")
    try:
        import flash_attn
    except ImportError as error:
        raise RuntimeError("flash_attention_2 is unavailable; install flash-attn (no automatic fallback)") from error
    if layout is None:
        layout = prepare_dense_layout(q.shape[:2], spans, q.device, attention_end)
    options = dict(dropout_p=0.0, causal=True)
    if layout.mode == "empty":
        return q * 0 + (k.sum() + v.sum()) * 0           # zeros that still reach k and v in the graph
    if layout.mode == "full":
        return flash_attn.flash_attn_func(q, k, v, **options)
    bounds = (layout.offsets, layout.offsets, layout.maximum, layout.maximum)
    if layout.mode == "packed":
        flat = [tensor.flatten(0, 1) for tensor in (q, k, v)]           # views: nothing is copied
        return flash_attn.flash_attn_varlen_func(*flat, *bounds, **options).reshape(q.shape)
    gathered = [torch.cat([tensor[row, start:end] for row, start, end in layout.spans]) for tensor in (q, k, v)]
    compact = flash_attn.flash_attn_varlen_func(*gathered, *bounds, **options)
    output, cursor = torch.zeros_like(q), 0
    for row, start, end in layout.spans:
        output[row, start:end] = compact[cursor:cursor + end - start]
        cursor += end - start
    return output


def dense_attention(q, k, v, segments):
    """Masked fp32 attention for small shapes: a token attends to the earlier tokens of its own
    document. Limited to batch * heads * width^2 <= 2^23 score elements."""
    rows, width, heads, dim = q.shape
    if rows * heads * width * width > 8_388_608:
        raise ValueError("vanilla attention exceeds the small-shape limit")
    order = torch.arange(width, device=q.device)
    same_document = (segments.unsqueeze(2) == segments.unsqueeze(1)) & (segments.unsqueeze(2) > 0)
    allowed = (same_document & (order.view(1, 1, -1) <= order.view(1, -1, 1))).unsqueeze(1)   # [rows, 1, query, key]
    scores = torch.einsum("bqhd,bkd->bhqk", q.float(), k[:, :, 0].float()) * dim ** -0.5
    scores = scores.masked_fill(~allowed, float("-inf"))
    scores = torch.where(allowed.any(-1, keepdim=True), scores, torch.zeros_like(scores))    # padding rows: no NaN
    weights = torch.softmax(scores, dim=-1) * allowed
    return torch.einsum("bhqk,bkd->bqhd", weights, v[:, :, 0].float()).to(q.dtype)
