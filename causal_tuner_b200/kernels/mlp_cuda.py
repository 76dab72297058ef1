"""SwiGLU LoRA MLP: tiled forward outside autograd and an analytic backward that recomputes
the gate/up projections instead of storing them.

Drop-in for the reference's kernels/mlp_cuda.py (same names, arguments and ownership rules).
The three projections run through ``forward_linear`` / ``input_gradient`` /
``parameter_gradients`` of ``.linear`` (tcgen05 GEMMs in libct_b200.so); the SiLU product
and its in-place backward are ct_swiglu.
"""

import torch

from .. import _lib
from .linear import (cast, materialize, forward_linear, input_gradient, input_gradient_group, parameter_gradients,
                     projection_parameters, matmul)


def _swiglu(gate, up, grad, out, dg, du, reconstruct):
    with _lib.on_device(gate):
        _lib.check(_lib.load().ct_swiglu(gate.data_ptr(), up.data_ptr(), _lib.pointer(grad), _lib.pointer(out),
                                        _lib.pointer(dg), _lib.pointer(du), gate.numel(), _lib.code_of(gate.dtype),
                                        int(reconstruct), _lib.stream_of(gate)))


def _dense(*tensors):
    for tensor in tensors:
        if tensor is not None and not tensor.is_contiguous():
            raise ValueError("SwiGLU buffers must be contiguous")


def activation(gate, up, gradient=None, *, out=None):
    """Forward: out = round(silu(gate)) * up. With `gradient`: rewrites (gate, up, gradient) in place
    to (d_gate, d_up, hidden) and returns the hidden buffer (kernels/mlp_cuda.py:28-35)."""
    _lib.require_cuda(gate, up, gradient, out)
    if gradient is not None:
        out = gradient
    elif out is None:
        out = torch.empty_like(gate)
    _dense(gate, up, out)
    if gradient is None:
        _swiglu(gate, up, None, out, None, None, True)
    else:
        _swiglu(gate, up, gradient, out, gate, up, True)
    return out


class _SiLUMultiply(torch.autograd.Function):
    """silu(gate) * up as an autograd node with separate gradient buffers (kernels/mlp_cuda.py:38-51)."""

    @staticmethod
    def forward(ctx, gate, up):
        gate, up = gate.contiguous(), up.contiguous()
        ctx.save_for_backward(gate, up)
        return activation(gate, up)

    @staticmethod
    def backward(ctx, grad):
        gate, up = ctx.saved_tensors
        dg, du = torch.empty_like(gate), torch.empty_like(up)
        _swiglu(gate, up, grad.contiguous(), None, dg, du, False)
        return dg, du


def silu_multiply(gate, up):
    return _SiLUMultiply.apply(gate, up)


def _prepare(parameters, states, dtype):
    matrices = [materialize(parameters[4 * i], state, dtype) for i, state in enumerate(states)]
    adapters = [(cast(parameters[4 * i + 1], dtype), cast(parameters[4 * i + 2], dtype)) for i in range(3)]
    return matrices, adapters


@torch.no_grad()
def _forward_into(output, x, dtype, tile, states, parameters, residual, *, save=False):
    """Fill `output` with down(silu(gate(x)) * up(x)) [+ residual], `tile` rows at a time.

    With save=True also returns (gate, up, xa_gate, xa_up) for all rows (kernels/mlp_cuda.py:58-81).
    The residual is added in the epilogue of the down projection.
    """
    flat = cast(x.reshape(-1, x.shape[-1]), dtype)
    rows = flat.shape[0]
    matrices, adapters = _prepare(parameters, states, dtype)
    width = matrices[0].shape[0]
    step = max(1, min(tile, rows))
    held = min(step, rows)
    workspace = torch.empty((1 if save else 2, held, width), device=x.device, dtype=dtype)
    low = torch.empty((held, max(a.shape[0] for a, _ in adapters)), device=x.device, dtype=dtype)
    saved = ()
    if save:
        saved = (*(torch.empty((rows, width), device=x.device, dtype=dtype) for _ in range(2)),
                 *(torch.empty((rows, a.shape[0]), device=x.device, dtype=dtype) for a, _ in adapters[:2]))
    destination = output.view(rows, output.shape[-1])
    shortcut = None if residual is None else residual.reshape(rows, residual.shape[-1])
    for start in range(0, rows, step):
        stop = min(start + step, rows)
        part, count = flat[start:stop], stop - start
        if save:
            gate, up = saved[0][start:stop], saved[1][start:stop]
            xa = [saved[2][start:stop], saved[3][start:stop], low[:count, :adapters[2][0].shape[0]]]
        else:
            gate, up = workspace[0, :count], workspace[1, :count]
            xa = [low[:count, :a.shape[0]] for a, _ in adapters]
        forward_linear(part, matrices[0], *adapters[0], out=gate, xa=xa[0])
        forward_linear(part, matrices[1], *adapters[1], out=up, xa=xa[1])
        hidden = activation(gate, up, out=workspace[0, :count] if save else gate)
        forward_linear(hidden, matrices[2], *adapters[2], out=destination[start:stop], xa=xa[2],
                       residual=None if shortcut is None else shortcut[start:stop])
    return saved


class _TiledLoRAMLP(torch.autograd.Function):
    """Autograd node of the MLP. Without caching it saves x and the parameters only and returns an
    EMPTY output that the wrapper fills afterwards, so that a checkpoint replay that stops at the
    last saved tensor never repeats the forward GEMMs (kernels/mlp_cuda.py:84-97)."""

    @staticmethod
    def forward(ctx, x, dtype, tile, states, residual, cache, *parameters):
        _lib.require_cuda(x)
        ctx.dtype, ctx.tile, ctx.states, ctx.cache = dtype, tile, states, cache
        if cache:
            output = torch.empty(x.shape, device=x.device, dtype=dtype)
            saved = _forward_into(output, x, dtype, tile, states, parameters, residual, save=True)
            ctx.save_for_backward(x, *saved, *parameters)
            return output
        ctx.save_for_backward(x, *parameters)
        return torch.empty(x.shape, device=x.device, dtype=dtype)

    @staticmethod
    def backward(ctx, grad):
        x, *parameters = ctx.saved_tensors
        saved = parameters[:4] if ctx.cache else ()
        if ctx.cache:
            parameters = parameters[4:]
        dtype = ctx.dtype
        residual_grad = grad if ctx.needs_input_grad[4] else None
        flat = cast(x.reshape(-1, x.shape[-1]), dtype)
        rows = flat.shape[0]
        upstream = cast(grad.reshape(rows, grad.shape[-1]), dtype).contiguous()
        want_dx = ctx.needs_input_grad[0]
        dx = torch.empty_like(flat) if want_dx else None
        matrices, adapters = _prepare(parameters, ctx.states, dtype)
        make = torch.empty_like if rows else torch.zeros_like
        gradients = [(make(parameters[4 * i + 1]), make(parameters[4 * i + 2])) for i in range(3)]
        step = max(1, min(ctx.tile, rows))
        held = min(step, rows)
        width = matrices[0].shape[0]
        workspace = torch.empty((3, held, width), device=x.device, dtype=dtype)
        low_inputs = [torch.empty((held, a.shape[0]), device=x.device, dtype=dtype) for a, _ in adapters]
        low_grad = torch.empty((3, held, max(a.shape[0] for a, _ in adapters)), device=x.device, dtype=dtype)
        for start in range(0, rows, step):
            stop = min(start + step, rows)
            count = stop - start
            part, dy = flat[start:stop], upstream[start:stop]
            gate, up, dh = workspace[0, :count], workspace[1, :count], workspace[2, :count]
            xa = [buffer[:count] for buffer in low_inputs]
            low = [low_grad[i, :count, :a.shape[0]] for i, (a, _) in enumerate(adapters)]
            if ctx.cache:
                xa[0], xa[1] = saved[2][start:stop], saved[3][start:stop]
            else:
                forward_linear(part, matrices[0], *adapters[0], out=gate, xa=xa[0])
                forward_linear(part, matrices[1], *adapters[1], out=up, xa=xa[1])
            input_gradient(dy, matrices[2], *adapters[2], dh, low[2])
            if ctx.cache:
                # Read the saved gate/up, write (d_gate, d_up, hidden) into the tile buffers: the saved
                # tensors stay untouched and survive a repeated backward pass, without a copy.
                _swiglu(saved[0][start:stop], saved[1][start:stop], dh, dh, gate, up, True)
                hidden = dh
            else:
                hidden = activation(gate, up, dh)  # (gate, up, dh) now hold (d_gate, d_up, hidden)
            matmul(hidden, adapters[2][0].T, out=xa[2])
            parameter_gradients(hidden, dy, *gradients[2], low[2], xa[2], add=start > 0)
            if want_dx:
                # gate and up share the input: one GEMM over [d_gate | low_g | d_up | low_u].
                input_gradient_group((gate, up), matrices[:2], [adapters[0][0], adapters[1][0]],
                                     [adapters[0][1], adapters[1][1]], dx[start:stop], low[:2])
            for index, signal in enumerate((gate, up)):
                if not want_dx:
                    matmul(signal, adapters[index][1], out=low[index])
                parameter_gradients(part, signal, *gradients[index], low[index], xa[index], add=start > 0)
        result = [value for da, db in gradients for value in (None, da, db, None)]
        dx_out = None if dx is None else cast(dx.reshape(x.shape), x.dtype)
        return (dx_out, None, None, None, residual_grad, None, *result)


def tiled_lora_mlp(module, x, residual=None, *, tile=None, cache=None):
    """SwiGLU MLP of `module` (gate_proj, up_proj, down_proj) on `x`, optionally plus `residual`
    (kernels/mlp_cuda.py:146-161). cache=True keeps gate, up and their low-rank inputs for the
    backward pass; otherwise they are recomputed there."""
    modules = (module.gate_proj, module.up_proj, module.down_proj)
    dtype = modules[0].compute_dtype
    if residual is not None and (residual.shape != x.shape or residual.dtype != dtype):
        return tiled_lora_mlp(module, x, tile=tile, cache=cache) + residual
    parameters, states = [], []
    for projection in modules:
        values, state = projection_parameters(projection)
        parameters.extend(values)
        states.append(state)
    tile = (module.tile if tile is None else tile) or max(1, x.numel() // x.shape[-1])
    cache = (module.cache_intermediates if cache is None else cache) and torch.is_grad_enabled()
    output = _TiledLoRAMLP.apply(x, dtype, tile, tuple(states), residual, cache, *parameters)
    if not cache:
        _forward_into(output, x, dtype, tile, states, parameters, residual)
    return output
