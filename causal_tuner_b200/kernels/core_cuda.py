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


# ---- RMSNorm and the rotary position table ------------------------------------------------

def position_values(positions, inverse, dtype):
    """cos/sin of positions[..., None] * inverse, fp32 product and full-range evaluation, then rounded
    to `dtype` (kernels/core_cuda.py:11-27). One launch per batch on [tokens, rotary_dim / 2] values."""
    _lib.require_cuda(positions, inverse)
    half = len(inverse)
    cosine = torch.empty((*positions.shape, half), device=positions.device, dtype=dtype)
    sine = torch.empty_like(cosine)
    positions = positions.to(torch.int64).contiguous()
    inverse = inverse.to(torch.float32).contiguous()
    with _lib.on_device(positions):
        _lib.check(_lib.load().ct_position_values(
            positions.data_ptr(), inverse.data_ptr(), cosine.data_ptr(), sine.data_ptr(), positions.numel(), half,
            _lib.code_of(dtype), _lib.stream_of(positions)))
    return cosine, sine


def _sm_count(device):
    return torch.cuda.get_device_properties(device).multi_processor_count


class RMS(torch.autograd.Function):
    """y = round(x * rstd) * round(w) (kernels/core_cuda.py:94-131).

    `reuse_grad=True` writes the input gradient over the upstream gradient, which the caller
    guarantees to be a private tensor (the projection operators return fresh input gradients).
    `reconstruct=True` saves the OUTPUT instead of the input - the projection that follows keeps it
    anyway - and the backward pass rebuilds the normalised row as y / w. Both belong to frozen
    pre-norms and are ignored for a trainable weight, whose fp32 gradient is summed over at most
    4 x SM-count row groups in a fixed order.
    """

    @staticmethod
    def forward(ctx, x, weight, eps, reuse_grad=False, reconstruct=False):
        _lib.require_cuda(x, weight)
        ctx.reuse_grad = reuse_grad and not weight.requires_grad
        ctx.reconstruct = reconstruct and not weight.requires_grad
        x = x.contiguous()
        output = torch.empty_like(x)
        width = x.shape[-1]
        rows = x.numel() // width
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        weight_values = weight.contiguous()
        with _lib.on_device(x):
            _lib.check(_lib.load().ct_rmsnorm_forward(
                x.data_ptr(), weight_values.data_ptr(), output.data_ptr(), rstd.data_ptr(), rows, width, float(eps),
                _lib.code_of(x.dtype), _lib.code_of(weight.dtype), _lib.stream_of(x)))
        ctx.save_for_backward(output if ctx.reconstruct else x, weight, rstd)
        return output

    @staticmethod
    def backward(ctx, grad):
        x, weight, rstd = ctx.saved_tensors
        grad = grad.contiguous()
        if grad.dtype != x.dtype:
            grad = grad.to(x.dtype)
        want_dx, want_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        result = (grad if ctx.reuse_grad else torch.empty_like(x)) if want_dx else None
        width, rows = x.shape[-1], rstd.numel()
        library = _lib.load()
        codes = (_lib.code_of(x.dtype), _lib.code_of(weight.dtype))
        weight_values = weight.contiguous()
        dw = None
        with _lib.on_device(x):
            stream = _lib.stream_of(x)
            if want_dw:
                dw = torch.empty_like(weight_values)
                groups = min(rows, 4 * _sm_count(x.device))
                per_group = -(-rows // groups) if groups else 1
                groups = -(-rows // per_group)
                partials = torch.empty((groups, width), device=x.device, dtype=torch.float32)
                if rows:
                    _lib.check(library.ct_rmsnorm_weight_gradient(
                        x.data_ptr(), weight_values.data_ptr(), rstd.data_ptr(), grad.data_ptr(), _lib.pointer(result),
                        partials.data_ptr(), rows, width, per_group, *codes, stream))
                _lib.check(library.ct_rmsnorm_weight_reduce(partials.data_ptr(), groups, width, dw.data_ptr(), codes[1],
                                                            stream))
            elif want_dx and rows:
                entry = library.ct_rmsnorm_backward_from_output if ctx.reconstruct else library.ct_rmsnorm_backward_add
                _lib.check(entry(x.data_ptr(), weight_values.data_ptr(), rstd.data_ptr(), grad.data_ptr(), None,
                                 result.data_ptr(), rows, width, *codes, stream))
        return result, dw, None, None, None


class RMSWithShortcut(torch.autograd.Function):
    """(RMS(x), x) for a pre-norm residual block `x + block(RMS(x))`: the normalised activations and
    the same x as the block's residual input (modeling/model.py:153-155 of the reference, where x
    feeds both and autograd adds the two gradients with a separate kernel). Here the backward pass
    receives both gradients and forms round(round(RMS gradient) + shortcut gradient) inside the
    RMSNorm kernel, over the upstream gradient of the normalised branch, which the projection
    operators hand over as a private tensor. Frozen weight only; `reconstruct` saves the output
    instead of x, as in `RMS`."""

    @staticmethod
    def forward(ctx, x, weight, eps, reconstruct=False):
        _lib.require_cuda(x, weight)
        if weight.requires_grad:
            raise ValueError("RMSWithShortcut is for frozen norm weights; use RMS for a trainable one")
        source = x.contiguous()
        output = torch.empty_like(source)
        width = source.shape[-1]
        rows = source.numel() // width
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        weight = weight.contiguous()
        with _lib.on_device(source):
            _lib.check(_lib.load().ct_rmsnorm_forward(
                source.data_ptr(), weight.data_ptr(), output.data_ptr(), rstd.data_ptr(), rows, width, float(eps),
                _lib.code_of(source.dtype), _lib.code_of(weight.dtype), _lib.stream_of(source)))
        ctx.reconstruct = bool(reconstruct)
        ctx.save_for_backward(output if ctx.reconstruct else source, weight, rstd)
        return output, x

    @staticmethod
    def backward(ctx, grad, shortcut_grad):
        x, weight, rstd = ctx.saved_tensors
        if not ctx.needs_input_grad[0]:
            return None, None, None, None
        if grad is None:
            return shortcut_grad, None, None, None
        grad = grad.contiguous()
        if grad.dtype != x.dtype:
            grad = grad.to(x.dtype)
        fused = shortcut_grad is not None and shortcut_grad.dtype == x.dtype and shortcut_grad.shape == x.shape
        extra = shortcut_grad.contiguous() if fused else None
        width = x.shape[-1]
        library = _lib.load()
        entry = library.ct_rmsnorm_backward_from_output if ctx.reconstruct else library.ct_rmsnorm_backward_add
        with _lib.on_device(x):
            _lib.check(entry(x.data_ptr(), weight.data_ptr(), rstd.data_ptr(), grad.data_ptr(), _lib.pointer(extra),
                             grad.data_ptr(), x.numel() // width, width, _lib.code_of(x.dtype),
                             _lib.code_of(weight.dtype), _lib.stream_of(x)))
        if shortcut_grad is not None and not fused:
            grad = grad + shortcut_grad
        return grad, None, None, None
