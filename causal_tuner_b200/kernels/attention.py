"""Causal attention over packed documents: the call into FlashAttention-2 is kept as the reference
has it (kernels/attention.py:16-93; attention itself is outside this package's kernels), plus the
small dense fp32 form the reference uses for its "vanilla" setting (kernels/reference.py:11-27)."""

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class DenseLayout:
    spans: tuple
    mode: str
    offsets: torch.Tensor | None = None
    maximum: int = 0


def prepare_dense_layout(shape, spans, device, attention_end=None):
    """Batch metadata built once per step: 'full' rows, 'packed' documents that tile the rows in
    order, or 'gaps' (padding between documents)."""
    if attention_end is not None:
        raise NotImplementedError("bidirectional attention groups are not part of this package")
    spans = tuple(spans)
    if not spans:
        return DenseLayout(spans, "empty")
    if spans == tuple((row, 0, shape[1]) for row in range(shape[0])):
        return DenseLayout(spans, "full")
    sizes = [end - start for _, start, end in spans]
    boundaries = [0]
    for size in sizes:
        boundaries.append(boundaries[-1] + size)
    offsets = torch.tensor(boundaries, dtype=torch.int32, device=device)
    cursor, contiguous = 0, True
    for row, start, end in spans:
        contiguous = contiguous and row * shape[1] + start == cursor
        cursor = row * shape[1] + end
    mode = "packed" if contiguous and cursor == shape[0] * shape[1] else "gaps"
    return DenseLayout(spans, mode, offsets, max(sizes))


def flash_dense(q, k, v, spans, attention_end=None, *, layout=None):
    if q.device.type != "cuda" or q.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("flash_attention_2 requires CUDA and BF16/FP16 inputs")
    try:
        from flash_attn import flash_attn_varlen_func, flash_attn_func
    except ImportError as exc:
        raise RuntimeError("flash_attention_2 is unavailable; install flash-attn (no automatic fallback)") from exc
    layout = layout or prepare_dense_layout(q.shape[:2], spans, q.device, attention_end)
    if layout.mode == "empty":
        return q * 0 + (k.sum() + v.sum()) * 0
    if layout.mode == "full":
        return flash_attn_func(q, k, v, dropout_p=0.0, causal=True)
    if layout.mode == "packed":
        return flash_attn_varlen_func(q.flatten(0, 1), k.flatten(0, 1), v.flatten(0, 1), layout.offsets, layout.offsets,
                                      layout.maximum, layout.maximum, dropout_p=0.0, causal=True).reshape_as(q)
    compact = lambda x: torch.cat([x[row, start:end] for row, start, end in layout.spans], 0)
    packed = flash_attn_varlen_func(compact(q), compact(k), compact(v), layout.offsets, layout.offsets,
                                    layout.maximum, layout.maximum, dropout_p=0.0, causal=True)
    output = torch.zeros_like(q)
    offset = 0
    for row, start, end in layout.spans:
        output[row, start:end] = packed[offset:offset + end - start]
        offset += end - start
    return output


def dense_attention(q, k, v, segments):
    """Masked fp32 attention for small shapes: same document, causal (the 'vanilla' setting)."""
    b, s, h, _ = q.shape
    if b * h * s * s > 8_388_608:
        raise ValueError("vanilla attention exceeds the small-shape limit")
    index = torch.arange(s, device=q.device)
    mask = ((segments[:, :, None] == segments[:, None, :]) & (segments[:, :, None] > 0)
            & (index[None, None, :] <= index[None, :, None]))[:, None]
    score = torch.einsum("bqhd,bkd->bhqk", q.float(), k[:, :, 0].float()) / q.shape[-1] ** 0.5
    score = score.masked_fill(~mask, -torch.inf)
    score = torch.where(mask.any(-1, keepdim=True), score, 0)
    probs = torch.softmax(score, -1) * mask
    return torch.einsum("bhqk,bkd->bqhd", probs, v[:, :, 0].float()).to(q.dtype)
