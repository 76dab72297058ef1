"""SwiGLU LoRA MLP: tiled forward outside autograd and an analytic backward that recomputes
the gate/up projections instead of storing them.

Drop-in for the reference's kernels/mlp_cuda.py (same names, arguments and ownership rules).
The three projections run through ``forward_linear`` / ``input_gradient`` /
``parameter_gradients`` of ``.linear`` (tcgen05 GEMMs in libct_b200.so); the SiLU product
and its in-place backward are ct_swiglu.
"""

import os

import torch

from .. import _lib
from .linear import (_policy, apply_projection, cast, decodes_transposed, gated_input_gradient, gated_projections,
                     gated_supported, input_gradient_swiglu, materialize, materialize_ahead, forward_linear,
                     input_gradient, input_gradient_with, input_gradient_group, parameter_gradients,
                     projection_parameters, matmul, stack_adapters, token_gradient, token_gradients)


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


def _gated(x, parameters, states, dtype, keeps):
    """Whether gate(x), up(x) and the SwiGLU run as ONE tcgen05 launch (`gated_projections`): the two base
    weights are then decoded into one buffer of interleaved 128-row blocks, a GEMM tile accumulates the same 128
    columns of both projections, and the activation (forward, or its in-place backward on recomputed tiles) is
    the tile's epilogue - gate and up never travel through memory unless the caller keeps them.

    An operator that recomputes takes this path in both passes whenever the shapes allow it (neither activation
    is written or read, and a kernel goes: 16 ms of a 690 ms 7B step that recomputes in every layer). A forward
    pass that `keeps` gate and up for the backward pass writes them anyway; there two launches of the
    512 x 256-tile GEMM plus the stand-alone activation are faster than the gated launch, whose tile is
    256 x 256 (3 ms of a 583 ms step), and are used unless CT_B200_MLP_FUSED_FORWARD=1."""
    if keeps and os.environ.get("CT_B200_MLP_FUSED_FORWARD", "0") != "1":
        return False
    if (states[0] is None) != (states[1] is None) or parameters[0].device.type != "cuda":
        return False
    shapes = [parameters[4 * i].shape if states[i] is None else tuple(states[i].shape) for i in range(2)]
    if len(shapes[0]) != 2 or shapes[0] != shapes[1]:
        return False
    return gated_supported(x, shapes[0][0], [parameters[1].shape[0], parameters[5].shape[0]], dtype)


def _prepare(parameters, states, dtype, order=(0, 1, 2), casts=None, gated=False, for_gradient=False):
    """Base weights decoding on the side stream in `order` (wait on the returned handle before a
    matrix is read), cast adapters, and the gate/up `a` matrices stacked row-wise (their low-rank
    inputs come from one product over x). `casts` = (stacked, b_gate, b_up, a_down, b_down) already in
    `dtype` (kept by the forward pass) skips the conversion. gated=True: matrices[0] and matrices[1] are one
    buffer holding both weights in interleaved 128-row blocks (complete after pending.wait(0) and wait(1)).
    `for_gradient`: the matrices (True: all; else their indices) that only input-gradient products will read."""
    matrices, pending = materialize_ahead([(parameters[4 * i], state) for i, state in enumerate(states)], dtype, order,
                                          interleave=gated, for_gradient=for_gradient)
    ranks = [parameters[1].shape[0], parameters[5].shape[0]]
    if casts is not None:
        stacked, others, offsets = casts[0], list(casts[1:]), [0, ranks[0]]
    else:
        stacked, offsets, others = stack_adapters([parameters[1], parameters[5]], dtype,
                                                  [parameters[2], parameters[6], parameters[9], parameters[10]])
    adapters = [(stacked[offsets[i]:offsets[i] + ranks[i]], others[i]) for i in range(2)]
    adapters.append((others[2], others[3]))
    return matrices, adapters, stacked, pending


@torch.no_grad()
def _forward_into(output, x, dtype, tile, states, parameters, residual, *, save=False):
    """Fill `output` with down(silu(gate(x)) * up(x)) [+ residual], `tile` rows at a time.

    With save=True also returns (gate, up, xa_gate, xa_up) for all rows (kernels/mlp_cuda.py:58-81).
    The residual is added in the epilogue of the down projection.
    """
    flat = cast(x.reshape(-1, x.shape[-1]), dtype)
    rows = flat.shape[0]
    gated = rows > 0 and _gated(flat, parameters, states, dtype, save)
    matrices, adapters, stacked, pending = _prepare(parameters, states, dtype, gated=gated)
    width = matrices[2].shape[1]
    ranks = [a.shape[0] for a, _ in adapters]
    step = max(1, min(tile, rows))
    held = min(step, rows)
    workspace = torch.empty((1 if save or gated else 2, held, width), device=x.device, dtype=dtype)
    low = torch.empty((held, stacked.shape[0]), device=x.device, dtype=dtype)
    low_down = torch.empty((held, ranks[2]), device=x.device, dtype=dtype)
    saved = ()
    if save:
        kept = torch.empty((rows, stacked.shape[0]), device=x.device, dtype=dtype)   # [xa_gate | xa_up]
        saved = (*(torch.empty((rows, width), device=x.device, dtype=dtype) for _ in range(2)),
                 kept[:, :ranks[0]], kept[:, ranks[0]:])
        if getattr(_policy, "keep_low_rank", False):
            # this library's option: the down projection's low-rank input joins the cache as a fifth tensor,
            # followed by the adapters in the compute dtype (so that backward does not convert them again)
            saved = (*saved, torch.empty((rows, ranks[2]), device=x.device, dtype=dtype),
                     stacked, adapters[0][1], adapters[1][1], adapters[2][0], adapters[2][1])
    destination = output.view(rows, output.shape[-1])
    shortcut = None if residual is None else residual.reshape(rows, residual.shape[-1])
    for start in range(0, rows, step):
        stop = min(start + step, rows)
        part, count = flat[start:stop], stop - start
        if save:
            gate, up = saved[0][start:stop], saved[1][start:stop]
            both = kept[start:stop]
        else:
            gate, up = (None, None) if gated else (workspace[0, :count], workspace[1, :count])
            both = low[:count]
        matmul(part, stacked.T, out=both)           # low-rank inputs of gate and up, reading x once
        pending.wait(0)
        if gated:
            pending.wait(1)
            hidden = gated_projections(part, matrices[0], both[:, :ranks[0]], both[:, ranks[0]:], adapters[0][1],
                                       adapters[1][1], hidden=workspace[0, :count], gate=gate if save else None,
                                       up=up if save else None)
        else:
            apply_projection(part, matrices[0], adapters[0][1], both[:, :ranks[0]], out=gate)
            pending.wait(1)
            apply_projection(part, matrices[1], adapters[1][1], both[:, ranks[0]:], out=up)
            hidden = activation(gate, up, out=workspace[0, :count] if save else gate)
        pending.wait(2)
        forward_linear(hidden, matrices[2], *adapters[2], out=destination[start:stop],
                       xa=saved[4][start:stop] if len(saved) > 4 else low_down[:count],
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
            ctx.kept = len(saved)
            ctx.save_for_backward(x, *saved, *parameters)
            return output
        ctx.save_for_backward(x, *parameters)
        return torch.empty(x.shape, device=x.device, dtype=dtype)

    @staticmethod
    def backward(ctx, grad):
        x, *parameters = ctx.saved_tensors
        saved = parameters[:ctx.kept] if ctx.cache else ()
        if ctx.cache:
            parameters = parameters[ctx.kept:]
        dtype = ctx.dtype
        residual_grad = grad if ctx.needs_input_grad[4] else None
        flat = cast(x.reshape(-1, x.shape[-1]), dtype)
        rows = flat.shape[0]
        upstream = cast(grad.reshape(rows, grad.shape[-1]), dtype).contiguous()
        want_dx = ctx.needs_input_grad[0]
        dx = torch.empty_like(flat) if want_dx else None
        # Cached: the down projection's weight is needed first, gate/up only for the input gradient.
        gated = rows > 0 and not ctx.cache and _gated(flat, parameters, ctx.states, dtype, False)
        matrices, adapters, stacked, pending = _prepare(parameters, ctx.states, dtype,
                                                        (2, 0, 1) if ctx.cache or gated else (0, 1, 2),
                                                        casts=saved[5:10] if len(saved) >= 10 else None, gated=gated,
                                                        for_gradient=(2,) if not ctx.cache else
                                                        (0, 1) if os.environ.get("CT_B200_MLP_FUSED_BACKWARD", "0") == "1"
                                                        else True)
        # The gated recompute reads gate and up from the interleaved buffer; their input gradient is faster from
        # transposed copies (K-major operands) where those can be decoded - two more decodes on the side stream.
        gradient_pair = gradient_pending = None
        if gated and want_dx and all(decodes_transposed(parameters[4 * i], ctx.states[i], dtype) for i in range(2)):
            gradient_pair, gradient_pending = materialize_ahead(
                [(parameters[4 * i], ctx.states[i]) for i in range(2)], dtype, for_gradient=True)
        ranks = [a.shape[0] for a, _ in adapters]
        # Cached activations: the SwiGLU backward can ride on the down projection's input-gradient GEMM
        # (`input_gradient_swiglu`, bit-identical). Measured inside a 7B step it gives back in that GEMM - which
        # then runs on 256 x 256 tiles with a long epilogue instead of 512 x 256 tiles - what the stand-alone kernel
        # cost (585-589 ms against 585-586 ms), so it is taken only on request (CT_B200_MLP_FUSED_BACKWARD=1).
        joined = (bool(ctx.cache) and rows > 0 and os.environ.get("CT_B200_MLP_FUSED_BACKWARD", "0") == "1"
                  and matrices[2].shape[1] % 32 == 0 and matrices[2].shape[0] % 8 == 0
                  and gated_supported(upstream, 0, ranks[2:], dtype))
        make = torch.empty if rows else torch.zeros
        wide = dict(device=x.device, dtype=torch.float32)
        # fp32 accumulators: d(a_gate) and d(a_up) stacked (one product over x yields both), the rest apart
        da_both = make((stacked.shape[0], flat.shape[1]), **wide)
        da_down = make(parameters[9].shape, **wide)
        db = [make(parameters[4 * i + 2].shape, **wide) for i in range(3)]
        step = max(1, min(ctx.tile, rows))
        held = min(step, rows)
        width = matrices[2].shape[1]
        workspace = torch.empty((3, held, width), device=x.device, dtype=dtype)
        xa_both = torch.empty((held, stacked.shape[0]), device=x.device, dtype=dtype)
        xa_down = torch.empty((held, ranks[2]), device=x.device, dtype=dtype)
        low_both = torch.empty((held, stacked.shape[0]), device=x.device, dtype=dtype)
        low_down = torch.empty((held, ranks[2]), device=x.device, dtype=dtype)
        for start in range(0, rows, step):
            stop = min(start + step, rows)
            count = stop - start
            part, dy = flat[start:stop], upstream[start:stop]
            gate, up, dh = workspace[0, :count], workspace[1, :count], workspace[2, :count]
            low = [low_both[:count, :ranks[0]], low_both[:count, ranks[0]:], low_down[:count]]
            if ctx.cache:
                xa = [saved[2][start:stop], saved[3][start:stop]]
            else:
                matmul(part, stacked.T, out=xa_both[:count])
                xa = [xa_both[:count, :ranks[0]], xa_both[:count, ranks[0]:]]
                if not gated:
                    pending.wait(0)
                    apply_projection(part, matrices[0], adapters[0][1], xa[0], out=gate)
                    pending.wait(1)
                    apply_projection(part, matrices[1], adapters[1][1], xa[1], out=up)
            matmul(dy, adapters[2][1], out=low[2])      # needs no base weight: runs beside the decodes
            pending.wait(2)
            if joined:
                # the gradient of hidden meets the kept gate and up in the epilogue of the GEMM that computes it:
                # it is never written, and (d_gate, d_up, hidden) land in the tile buffers; the saved tensors stay
                # untouched and survive a repeated backward pass
                hidden = input_gradient_swiglu(dy, matrices[2], adapters[2][0], low[2], saved[0][start:stop],
                                               saved[1][start:stop], gate, up, dh)
            else:
                input_gradient_with(dy, matrices[2], adapters[2][0], low[2], dh)
                if ctx.cache:
                    # Read the saved gate/up, write (d_gate, d_up, hidden) into the tile buffers: the saved
                    # tensors stay untouched and survive a repeated backward pass, without a copy.
                    _swiglu(saved[0][start:stop], saved[1][start:stop], dh, dh, gate, up, True)
                    hidden = dh
                elif gated:
                    # gate and up are recomputed tile by tile in the GEMM's accumulator and leave it as (d_gate,
                    # d_up, hidden): the activations themselves are never written
                    pending.wait(0)
                    pending.wait(1)
                    hidden = gated_projections(part, matrices[0], xa[0], xa[1], adapters[0][1], adapters[1][1],
                                               hidden=dh, gate=gate, up=up, gradient=dh)
                else:
                    hidden = activation(gate, up, dh)  # (gate, up, dh) now hold (d_gate, d_up, hidden)
            if len(saved) > 4:
                xa_low = saved[4][start:stop]
            else:
                xa_low = matmul(hidden, adapters[2][0].T, out=xa_down[:count])
            if want_dx:
                # gate and up share the input: one GEMM over [d_gate | low_g | d_up | low_u].
                pending.wait()
                if gradient_pair is not None:
                    gradient_pending.wait()
                    input_gradient_group((gate, up), gradient_pair, [adapters[0][0], adapters[1][0]],
                                         [adapters[0][1], adapters[1][1]], dx[start:stop], low[:2])
                elif gated:
                    gated_input_gradient(gate, up, matrices[0], adapters[0][0], adapters[1][0], adapters[0][1],
                                         adapters[1][1], dx[start:stop], low[:2])
                else:
                    input_gradient_group((gate, up), matrices[:2], [adapters[0][0], adapters[1][0]],
                                         [adapters[0][1], adapters[1][1]], dx[start:stop], low[:2])
            else:
                for index, signal in enumerate((gate, up)):
                    matmul(signal, adapters[index][1], out=low[index])
            # All five adapter-gradient products of the tile in one launch: d(a_down), d(b_down), the stacked
            # d(a_gate; a_up), d(b_gate), d(b_up). Apart they leave the machine between 22 % and 76 % occupied.
            token_gradients([(low[2], hidden, da_down), (dy, xa_low, db[2]), (low_both[:count], part, da_both),
                             (gate, xa[0], db[0]), (up, xa[1], db[1])], add=start > 0)
        da = [da_both[:ranks[0]], da_both[ranks[0]:], da_down]
        like = lambda value, parameter: value if parameter.dtype == torch.float32 else value.to(parameter.dtype)
        result = [value for i in range(3)
                  for value in (None, like(da[i], parameters[4 * i + 1]), like(db[i], parameters[4 * i + 2]), None)]
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
    _policy.keep_low_rank = bool(cache) and all(getattr(projection, "keep_low_rank", False) for projection in modules)
    try:
        output = _TiledLoRAMLP.apply(x, dtype, tile, tuple(states), residual, cache, *parameters)
    finally:
        _policy.keep_low_rank = False
    if not cache:
        _forward_into(output, x, dtype, tile, states, parameters, residual)
    return output
