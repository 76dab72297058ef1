"""Adjacent-pair partial RoPE used inside the projection operator.

Drop-in for the rotary entry points of the reference's kernels/core_cuda.py that the
projection op calls: ``rotate_owned_qk`` (:192), ``inverse_rope_tile`` (:203) and the
``PartialRoPE`` autograd function (:211). Rounding contract (kernels/core_cuda.py:134-142):
every product is rounded to the activation dtype before the add, so the fused and the
stand-alone rotation agree bit for bit.
"""

import torch

from .. import _lib


def _rope(x, cosine, sine, y, heads, head_dim, inverse):
    rows = x.numel() // (heads * head_dim)
    half = cosine.shape[-1]
    if cosine.dtype != x.dtype:
        cosine, sine = cosine.to(x.dtype), sine.to(x.dtype)
    cosine, sine = cosine.contiguous(), sine.contiguous()
    with _lib.on_device(x):
        _lib.check(_lib.load().ct_rope(x.data_ptr(), cosine.data_ptr(), sine.data_ptr(), y.data_ptr(), rows, heads,
                                      head_dim, half, int(inverse), _lib.code_of(x.dtype), _lib.stream_of(x)))
    return y


def rotate_owned_qk(query, key, cosine, sine, head_dim):
    """Rotate freshly produced projection outputs in place (they are not yet visible to autograd)."""
    _lib.require_cuda(query, key)
    for tensor in (query, key):
        if not tensor.is_contiguous():
            raise ValueError("owned projection outputs are contiguous")
        _rope(tensor, cosine, sine, tensor, tensor.shape[-1] // head_dim, head_dim, False)


def inverse_rope_tile(grad, cosine, sine, head_dim, output):
    """Write the inverse rotation of `grad` into the private tile `output`; `grad` is left untouched."""
    _lib.require_cuda(grad, output)
    return _rope(grad.contiguous(), cosine, sine, output, grad.shape[-1] // head_dim, head_dim, True)


class PartialRoPE(torch.autograd.Function):
    """x[..., heads, head_dim] -> rotated copy; the backward pass is the inverse rotation."""

    @staticmethod
    def forward(ctx, x, cosine, sine):
        _lib.require_cuda(x)
        x = x.contiguous()
        ctx.shape = x.shape
        ctx.save_for_backward(cosine, sine)
        return _rope(x, cosine, sine, torch.empty_like(x), x.shape[-2], x.shape[-1], False)

    @staticmethod
    def backward(ctx, grad):
        cosine, sine = ctx.saved_tensors
        grad = grad.contiguous()
        return _rope(grad, cosine, sine, torch.empty_like(grad), ctx.shape[-2], ctx.shape[-1], True), None, None
