"""Frozen-base projection with NF4 decode and rank-r LoRA, forward and analytic backward.

Drop-in for the reference's kernels/linear.py: the same module-level names with the same
arguments, ownership rules and error behaviour, so callers and tests written against the
reference work unchanged. The arithmetic runs in libct_b200.so:

* ``forward_linear``      -> ct_forward_linear   (xa = x.A^T, then ONE tcgen05 GEMM over the
                             concatenated contraction [x | xa].[W | B]^T with bias and
                             residual in the epilogue)
* ``input_gradient``      -> ct_input_gradient   (low = dy.B, then ONE GEMM [dy | low].[W ; A])
* ``parameter_gradients`` -> ct_parameter_gradients (token-contracted fp32 dA / dB, fixed
                             summation order)
* ``accumulate``          -> ct_matmul
* ``materialize``         -> ct_nf4_decode / ct_cast

Beyond the reference's names, for projections that share their input (q/k/v, gate/up):
``stack_adapters`` + ``matmul`` give all low-rank inputs from one product over x,
``apply_projection`` is ``forward_linear`` with that input already computed, ``token_gradient``
(ct_accumulate) gives the stacked dA, ``input_gradient_group`` one summed dX, and
``materialize_ahead`` decodes the base weights on a side stream beside those products.

Differences from the reference that callers can observe: outputs are rounded to the compute
dtype once per GEMM (the reference rounds after the base product and again after the
low-rank update), and `tile` only bounds workspaces - tile 0 runs all rows in one launch.
"""

import os
import threading

import torch

from .. import _lib
from . import core_cuda


# ---- tensor plumbing --------------------------------------------------------------------

def cast(tensor, dtype, out=None):
    """`tensor.to(dtype)` through ct_cast; returns the tensor itself when the dtype already matches.
    With `out` (contiguous, same shape) the values always land there."""
    if tensor is None or (tensor.dtype == dtype and out is None):
        return tensor
    _lib.require_cuda(tensor)
    source = tensor.contiguous()
    if out is not None and (out.shape != source.shape or out.dtype != dtype or not out.is_contiguous()):
        raise ValueError("cast destination must be contiguous with the source's shape")
    output = torch.empty(source.shape, device=source.device, dtype=dtype) if out is None else out
    count = source.numel()
    if count:
        with _lib.on_device(source):
            _lib.check(_lib.load().ct_cast(source.data_ptr(), _lib.code_of(source.dtype), count, output.data_ptr(),
                                          _lib.code_of(dtype), count, 1, count, _lib.stream_of(source)))
    return output


def cast_many(tensors, dtype, outs=None):
    """`cast` for several tensors at once: one launch per 32 tensors that need converting instead of
    one each. `outs[i]` (contiguous, same shape, `dtype`) receives tensor i when given; a tensor that
    already has `dtype` and no `out` is returned as it is, None stays None."""
    import ctypes
    results, jobs = [], {}
    for index, tensor in enumerate(tensors):
        out = None if outs is None else outs[index]
        if tensor is None or (tensor.dtype == dtype and out is None):
            results.append(tensor)
            continue
        _lib.require_cuda(tensor)
        source = tensor.contiguous()
        if out is None:
            out = torch.empty(source.shape, device=source.device, dtype=dtype)
        elif out.shape != source.shape or out.dtype != dtype or not out.is_contiguous():
            raise ValueError("cast destination must be contiguous with the source's shape")
        results.append(out)
        if source.numel():
            jobs.setdefault(source.dtype, []).append((source, out))
    for source_dtype, pairs in jobs.items():
        count = len(pairs)
        sources = (ctypes.c_void_p * count)(*[s.data_ptr() for s, _ in pairs])
        targets = (ctypes.c_void_p * count)(*[o.data_ptr() for _, o in pairs])
        sizes = (ctypes.c_int64 * count)(*[s.numel() for s, _ in pairs])
        with _lib.on_device(pairs[0][0]):
            _lib.check(_lib.load().ct_cast_many(count, sources, targets, sizes, _lib.code_of(source_dtype),
                                               _lib.code_of(dtype), _lib.stream_of(pairs[0][0])))
    return results


def _leading(tensor):
    """Leading dimension (elements between rows) of a 2-D tensor whose rows are contiguous."""
    return tensor.stride(0) if tensor.shape[0] > 1 else max(tensor.shape[1], 1)


def _readable(tensor):
    if tensor.dim() != 2:
        raise ValueError("expected a matrix")
    if tensor.shape[1] > 1 and tensor.stride(1) != 1 or (tensor.shape[0] > 1 and tensor.stride(0) < tensor.shape[1]):
        tensor = tensor.contiguous()
    return tensor


def _weight_operand(weight):
    """(tensor, row stride, column stride) of a [N, K] weight for the input-gradient products: row-major, or the
    `.T` view of a weight that was materialised transposed (unit row stride) - passed on as it is."""
    if weight.dim() != 2:
        raise ValueError("expected a matrix")
    if weight.shape[0] > 1 and weight.shape[1] > 1 and weight.stride(0) == 1 and weight.stride(1) >= weight.shape[0]:
        return weight, 1, weight.stride(1)
    weight = _readable(weight)
    return weight, _leading(weight), 1


def _writable(tensor, name):
    if tensor.dim() != 2 or (tensor.shape[1] > 1 and tensor.stride(1) != 1):
        raise ValueError(f"{name} must be a matrix with contiguous rows")
    return tensor


def _strides(tensor):
    """Element strides (row, column) with a unit stride wherever the extent is 1."""
    rs = tensor.stride(0) if tensor.shape[0] > 1 else None
    cs = tensor.stride(1) if tensor.shape[1] > 1 else None
    if rs is None and cs is None:
        return 1, 1
    if rs is None:
        return (tensor.shape[1] * cs if cs != 1 else tensor.shape[1]), cs
    if cs is None:
        return rs, (1 if rs != 1 else tensor.shape[0])
    return rs, cs


def matmul(left, right, *, out, add=False):
    """out[m, n] = (add ? out : 0) + left[m, k] @ right[k, n]; any strides, fp32 accumulation."""
    _lib.require_cuda(left, right, out)
    _writable(out, "out")
    if right.dtype != left.dtype:
        right = cast(right, left.dtype)
    (a_rs, a_cs), (b_rs, b_cs) = _strides(left), _strides(right)
    if a_rs != 1 and a_cs != 1:
        left = left.contiguous()
        a_rs, a_cs = _strides(left)
    if b_rs != 1 and b_cs != 1:
        right = right.contiguous()
        b_rs, b_cs = _strides(right)
    m, k = left.shape
    n = right.shape[1]
    if right.shape[0] != k or out.shape != (m, n):
        raise ValueError("matmul shape mismatch")
    with _lib.on_device(out):
        _lib.check(_lib.load().ct_matmul(left.data_ptr(), a_rs, a_cs, right.data_ptr(), b_rs, b_cs, out.data_ptr(),
                                        _leading(out), m, n, k, _lib.code_of(left.dtype), _lib.code_of(out.dtype),
                                        int(bool(add)), _lib.gemm_path, _lib.stream_of(out)))
    return out


def matmul_nf4(x, weight, state, *, out):
    """out = x @ dequantize_nf4(weight, state).T with the decode inside the GEMM (ct_matmul_nf4): the dense
    weight is never written. Bit-identical to decoding first. bf16, 64-element blocks, fp32 absmax; raises
    NotImplementedError otherwise. Every 256-row tile of x repeats the decode, so decoding once
    (`materialize`) is faster from a few hundred tokens up - which is what the operators do."""
    _lib.require_cuda(x, weight, out)
    if state.quant_type != "nf4" or bool(state.nested) or state.absmax.dtype != torch.float32:
        raise NotImplementedError("matmul_nf4 takes plain NF4 with fp32 absmax")
    if state.dtype not in (torch.bfloat16, torch.float32) or x.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise NotImplementedError("matmul_nf4 computes in bf16 (quant state bf16 or fp32)")
    x = _readable(x)
    _writable(out, "out")
    outer, inner = state.shape
    if x.shape[1] != inner or out.shape != (x.shape[0], outer):
        raise ValueError("matmul_nf4 shape mismatch")
    code = state.code if state.code.dtype == torch.float32 else state.code.float()
    with _lib.on_device(x):
        _lib.check(_lib.load().ct_matmul_nf4(x.data_ptr(), _leading(x), weight.data_ptr(), state.absmax.data_ptr(),
                                            code.data_ptr(), out.data_ptr(), _leading(out), x.shape[0], inner, outer,
                                            int(state.blocksize), _lib.code_of(x.dtype), _lib.stream_of(x)))
    return out


# ---- the reference's primitives -----------------------------------------------------------

def materialize(weight, state, dtype):
    """Dense `dtype` copy of a base weight: NF4 decode when `state` is given, else a cast.

    Mirrors kernels/linear.py:6-13. Without bitsandbytes there is exactly one quantised
    format: contiguous uint8 NF4 on a CUDA device; anything else is an error, not a fallback.
    """
    if state is not None:
        if weight.is_cuda and weight.dtype == torch.uint8 and weight.is_contiguous() and state.quant_type == "nf4":
            from .nf4_cuda import dequantize_nf4
            return dequantize_nf4(weight, state, dtype)
        raise RuntimeError("only contiguous uint8 NF4 weights on a CUDA device can be decoded")
    return cast(weight, dtype)


def materialize_for_gradient(weight, state, dtype):
    """`materialize` for a weight that only the input-gradient product dx = dy @ W will read. With
    CT_B200_DECODE_TRANSPOSED=1 an NF4 weight is decoded TRANSPOSED where the shapes allow it (same values; returned
    as the [N, K] view of a [K, N] buffer), which makes W the K-major operand of that GEMM. Timed alone in short
    bursts that orientation is up to 19 % faster (1555 against 1302 TFLOP/s at 16384 x 14336 x 4352); inside a
    training step, where the GPU sits at its power cap, the same launches take the same time either way (1461 and
    1465 us) and the transposed decode is the slower one, so the default is the plain decode."""
    if decodes_transposed(weight, state, dtype):
        from .nf4_cuda import dequantize_nf4_transposed
        return dequantize_nf4_transposed(weight, state, dtype)
    return materialize(weight, state, dtype)


def decodes_transposed(weight, state, dtype):
    """Whether `materialize_for_gradient` decodes this weight transposed."""
    if (state is None or not weight.is_cuda or weight.dtype != torch.uint8 or not weight.is_contiguous()
            or state.quant_type != "nf4" or _lib.gemm_path == _lib.PATH_SIMT
            or os.environ.get("CT_B200_DECODE_TRANSPOSED", "0") != "1"):
        return False
    from .nf4_cuda import transposable
    return transposable(state, dtype)


_side_streams = {}


class _Pending:
    """Decodes in flight on the side stream; `wait(i)` orders the current stream after the i-th
    matrix (and everything decoded before it), `wait()` after all of them."""

    def __init__(self, events, order):
        self.events, self.order, self.done = events, order, -1

    def wait(self, index=None):
        if not self.events:
            return
        position = len(self.order) - 1 if index is None else self.order.index(index)
        if position > self.done:
            torch.cuda.current_stream().wait_event(self.events[position])
            self.done = position


def materialize_into_pair(weight, state, pair, which):
    """`materialize(weight, state, pair.dtype)` written into the interleaved buffer `pair` [2 N, K]: rows
    [128 t, 128 t + 128) of the weight become rows [256 t + 128 * which, ... + 128) (which = 0: gate, 1: up),
    the layout the gated GEMM of the MLP reads its B operand in."""
    if state is not None:
        if weight.is_cuda and weight.dtype == torch.uint8 and weight.is_contiguous() and state.quant_type == "nf4":
            from .nf4_cuda import dequantize_nf4_blocks
            return dequantize_nf4_blocks(weight, state, pair, which)
        raise RuntimeError("only contiguous uint8 NF4 weights on a CUDA device can be decoded")
    outer, inner = weight.shape
    pair.view(outer // 128, 2, 128, inner)[:, which].copy_(weight.view(outer // 128, 128, inner))
    return pair


def materialize_ahead(pairs, dtype, order=None, *, interleave=False, for_gradient=False):
    """`materialize` for several (weight, quant_state) pairs with the NF4 decodes issued on a side
    stream in `order`, so that they run under whatever the caller launches next that does not need the
    dense weights (the low-rank products, which leave the decode most of the HBM bandwidth).
    Returns (matrices, pending); call `pending.wait(i)` before the first launch that reads matrix i.
    CT_B200_DECODE_AHEAD=0 decodes in stream order instead.
    interleave=True: pairs 0 and 1 (the gate and up weights of an MLP, equal shapes) share ONE buffer of
    interleaved 128-row blocks (`materialize_into_pair`); matrices[0] and matrices[1] are that buffer, complete
    once both have been waited for.
    for_gradient: True, or the indices of the matrices that only input-gradient products will read
    (`materialize_for_gradient`); the interleaved pair is never among them."""
    order = list(range(len(pairs))) if order is None else list(order)
    device = pairs[0][0].device
    shared = []

    def produce(index):
        weight, state = pairs[index]
        if interleave and index < 2:
            if not shared:
                outer, inner = pairs[0][0].shape if pairs[0][1] is None else pairs[0][1].shape
                shared.append(torch.empty((2 * outer, inner), device=device, dtype=dtype))
            return materialize_into_pair(weight, state, shared[0], index)
        gradient_only = for_gradient is True or (for_gradient and index in for_gradient)
        return (materialize_for_gradient if gradient_only else materialize)(weight, state, dtype)

    ahead = (device.type == "cuda" and (interleave or any(state is not None for _, state in pairs))
             and os.environ.get("CT_B200_DECODE_AHEAD", "1") != "0")
    if not ahead:
        return [produce(index) for index in range(len(pairs))], _Pending([], order)
    with torch.cuda.device(device):
        main = torch.cuda.current_stream()
        side = _side_streams.get(device.index)
        if side is None:
            side = _side_streams[device.index] = torch.cuda.Stream(device=device)
        side.wait_stream(main)        # everything enqueued so far (and the memory it frees) comes first
        matrices, events = [None] * len(pairs), []
        with torch.cuda.stream(side):
            for index in order:
                weight = pairs[index][0]
                matrices[index] = produce(index)
                if matrices[index] is not weight:
                    matrices[index].record_stream(main)   # consumed on `main`: hold the block until that work is done
                event = torch.cuda.Event()
                event.record(side)
                events.append(event)
    return matrices, _Pending(events, order)


def accumulate(output, left, right, *, add=True):
    """output (+)= left @ right with fp32 accumulation (kernels/linear.py:16-24). With add=False the
    previous contents of `output` are never read."""
    matmul(left, right, out=output, add=add)


def forward_linear(x, weight, a, b, *, out, xa, bias=None, residual=None):
    """out = x @ weight.T + bias + (x @ a.T) @ b.T [+ residual]; also leaves xa = x @ a.T.

    kernels/linear.py:27-33. `residual`, when given, is added to the rounded output and the sum
    rounded again - the result of the reference's separate in-place add (kernels/linear.py:90-91).
    """
    _lib.require_cuda(x, weight, out)
    x, weight = _readable(x), _readable(weight)
    _writable(out, "out")
    rows, inner = x.shape
    outer = weight.shape[0]
    rank = a.shape[0] if a is not None else 0
    if rank:
        a, b = a.contiguous(), b.contiguous()
        _writable(xa, "xa")
    if residual is not None:
        residual = _readable(residual)
    with _lib.on_device(x):
        _lib.check(_lib.load().ct_forward_linear(
            x.data_ptr(), _leading(x), weight.data_ptr(), _leading(weight), _lib.pointer(a if rank else None),
            _lib.pointer(b if rank else None), _lib.pointer(bias), _lib.pointer(residual),
            _leading(residual) if residual is not None else 0, out.data_ptr(), _leading(out),
            _lib.pointer(xa if rank else None), _leading(xa) if rank else 0, rows, inner, outer, rank,
            _lib.code_of(x.dtype), _lib.gemm_path, _lib.stream_of(x)))


def input_gradient(dy, weight, a, b, dx, low, *, add=False):
    """low = dy @ b; dx = (add ? dx : 0) + dy @ weight + low @ a (kernels/linear.py:36-39)."""
    _lib.require_cuda(dy, weight, dx, low)
    dy = _readable(dy)
    weight, w_rs, w_cs = _weight_operand(weight)
    _writable(dx, "dx")
    _writable(low, "low")
    a, b = a.contiguous(), b.contiguous()
    rows, outer = dy.shape
    inner, rank = weight.shape[1], a.shape[0]
    with _lib.on_device(dy):
        _lib.check(_lib.load().ct_input_gradient(
            dy.data_ptr(), _leading(dy), weight.data_ptr(), w_rs, w_cs, a.data_ptr(), b.data_ptr(),
            dx.data_ptr(), _leading(dx), low.data_ptr(), _leading(low), rows, inner, outer, rank, int(bool(add)),
            _lib.code_of(dy.dtype), _lib.gemm_path, _lib.stream_of(dy)))


def input_gradient_with(dy, weight, a, low, dx, *, add=False):
    """`input_gradient` with low = dy @ b already computed: dx = (add ? dx : 0) + dy @ weight + low @ a."""
    _lib.require_cuda(dy, weight, dx, low)
    dy, low = _readable(dy), _readable(low)
    weight, w_rs, w_cs = _weight_operand(weight)
    _writable(dx, "dx")
    a = a.contiguous()
    rows, outer = dy.shape
    inner, rank = weight.shape[1], a.shape[0]
    with _lib.on_device(dy):
        _lib.check(_lib.load().ct_input_gradient(
            dy.data_ptr(), _leading(dy), weight.data_ptr(), w_rs, w_cs, a.data_ptr(), None,
            dx.data_ptr(), _leading(dx), low.data_ptr(), _leading(low), rows, inner, outer, rank, int(bool(add)),
            _lib.code_of(dy.dtype), _lib.gemm_path, _lib.stream_of(dy)))


def input_gradient_group(dys, weights, a_list, b_list, dx, lows, *, add=False):
    """Input gradient of projections that share their input, in one GEMM:
    low_i = dy_i @ b_i and dx = (add ? dx : 0) + sum_i (dy_i @ weight_i + low_i @ a_i).
    Same arithmetic as calling `input_gradient` per projection with add=index > 0
    (kernels/linear.py:122), except that dx is rounded once."""
    import ctypes
    count = len(dys)
    _lib.require_cuda(dx, *dys, *weights, *lows)
    dys = [_readable(t) for t in dys]
    operands = [_weight_operand(t) for t in weights]
    weights = [operand[0] for operand in operands]
    a_list, b_list = [t.contiguous() for t in a_list], [t.contiguous() for t in b_list]
    _writable(dx, "dx")
    for low in lows:
        _writable(low, "low")
    pointers = lambda tensors: (ctypes.c_void_p * count)(*[t.data_ptr() for t in tensors])
    sizes = lambda values: (ctypes.c_int64 * count)(*values)
    rows, inner = dys[0].shape[0], weights[0].shape[1]
    with _lib.on_device(dx):
        _lib.check(_lib.load().ct_input_gradient_group(
            count, pointers(dys), sizes([_leading(t) for t in dys]), pointers(weights),
            sizes([operand[1] for operand in operands]), sizes([operand[2] for operand in operands]),
            pointers(a_list), pointers(b_list),
            sizes([t.shape[0] for t in weights]), sizes([t.shape[0] for t in a_list]), dx.data_ptr(), _leading(dx),
            pointers(lows), sizes([_leading(t) for t in lows]), rows, inner, int(bool(add)),
            _lib.code_of(dx.dtype), _lib.gemm_path, _lib.stream_of(dx)))


def gated_supported(x, width, ranks, dtype):
    """Whether the MLP's gate / up projections of `x` can run as one gated GEMM (ct_gated_forward): bf16 on the
    tcgen05 path, widths that are multiples of 128, rows and ranks in multiples of 8 elements."""
    return (dtype == torch.bfloat16 and x.is_cuda and _lib.gemm_path != _lib.PATH_SIMT and width % 128 == 0
            and x.shape[-1] % 8 == 0 and all(rank > 0 and rank % 8 == 0 for rank in ranks)
            and os.environ.get("CT_B200_MLP_FUSED", "1") != "0")


def gated_projections(x, pair, xa_gate, xa_up, b_gate, b_up, *, hidden, gate=None, up=None, gradient=None):
    """gate(x), up(x) and the SwiGLU between them in one launch over the interleaved weights `pair`.
    Forward (gradient None): hidden = silu(gate) * up; `gate` / `up`, when given, receive the two projections.
    Backward: `gradient` is d(hidden); (gate, up, hidden) receive (d_gate, d_up, hidden) - the in-place backward
    of `activation` without gate and up ever being stored. hidden may be the gradient's buffer."""
    _lib.require_cuda(x, pair, xa_gate, xa_up, b_gate, b_up, hidden, gate, up, gradient)
    x, xa_gate, xa_up = _readable(x), _readable(xa_gate), _readable(xa_up)
    b_gate, b_up = b_gate.contiguous(), b_up.contiguous()
    rows, inner = x.shape
    width = pair.shape[0] // 2
    outputs = [t for t in (hidden, gate, up, gradient) if t is not None]
    for tensor in outputs:
        if tensor.shape != (rows, width) or tensor.stride(1) != 1 or tensor.stride(0) != outputs[0].stride(0):
            raise ValueError("gated projections: hidden, gate, up and gradient must be [rows, width] with one leading dimension")
    if _leading(xa_gate) != _leading(xa_up):
        raise ValueError("gated projections: the two low-rank inputs must share a leading dimension")
    library = _lib.load()
    common = (x.data_ptr(), _leading(x), pair.data_ptr(), _leading(pair), xa_gate.data_ptr(), xa_up.data_ptr(),
              _leading(xa_gate), b_gate.data_ptr(), b_up.data_ptr())
    sizes = (_leading(hidden), rows, inner, width, b_gate.shape[1], b_up.shape[1], _lib.code_of(x.dtype),
             _lib.stream_of(x))
    with _lib.on_device(x):
        if gradient is None:
            _lib.check(library.ct_gated_forward(*common, hidden.data_ptr(), _lib.pointer(gate), _lib.pointer(up), *sizes))
        else:
            _lib.check(library.ct_gated_backward(*common, gradient.data_ptr(), hidden.data_ptr(), gate.data_ptr(),
                                                 up.data_ptr(), *sizes))
    return hidden


def gated_input_gradient(d_gate, d_up, pair, a_gate, a_up, b_gate, b_up, dx, lows, *, add=False):
    """`input_gradient_group` for the gate and up projections with their base weights read from the interleaved
    buffer `pair`: low_i = d_i @ b_i, dx = (add ? dx : 0) + sum_i (d_i @ weight_i + low_i @ a_i)."""
    _lib.require_cuda(d_gate, d_up, pair, dx, *lows)
    d_gate, d_up = _readable(d_gate), _readable(d_up)
    a_gate, a_up = a_gate.contiguous(), a_up.contiguous()
    _writable(dx, "dx")
    matmul(d_gate, b_gate, out=lows[0])
    matmul(d_up, b_up, out=lows[1])
    if _leading(d_gate) != _leading(d_up) or _leading(lows[0]) != _leading(lows[1]):
        raise ValueError("gated input gradient: the two signals (and the two low-rank gradients) must share a leading dimension")
    rows, inner = d_gate.shape[0], pair.shape[1]
    with _lib.on_device(dx):
        _lib.check(_lib.load().ct_gated_input_gradient(
            d_gate.data_ptr(), d_up.data_ptr(), _leading(d_gate), pair.data_ptr(), _leading(pair), lows[0].data_ptr(),
            lows[1].data_ptr(), _leading(lows[0]), a_gate.data_ptr(), a_up.data_ptr(), dx.data_ptr(), _leading(dx),
            rows, inner, pair.shape[0] // 2, a_gate.shape[0], a_up.shape[0], int(bool(add)),
            _lib.code_of(dx.dtype), _lib.stream_of(dx)))


def input_gradient_swiglu(dy, weight, a, low, gate, up, d_gate, d_up, hidden):
    """Backward pass of a SwiGLU whose gate and up were kept, inside the input-gradient GEMM of the projection that
    follows it: dh = dy @ weight + low @ a stays in the accumulator, and (d_gate, d_up, hidden) - the in-place
    backward of `activation(gate, up, dh)` - are written; gate and up are only read. `low` = dy @ b is an input."""
    _lib.require_cuda(dy, weight, a, low, gate, up, d_gate, d_up, hidden)
    dy, weight, low, gate, up = _readable(dy), _readable(weight), _readable(low), _readable(gate), _readable(up)
    a = a.contiguous()
    rows, width = dy.shape[0], weight.shape[1]
    for tensor in (gate, up, d_gate, d_up, hidden):
        if tensor.shape != (rows, width) or tensor.stride(1) != 1:
            raise ValueError("input_gradient_swiglu: gate, up and the outputs must be [rows, width] with unit column stride")
    if _leading(gate) != _leading(up) or len({_leading(t) for t in (d_gate, d_up, hidden)}) != 1:
        raise ValueError("input_gradient_swiglu: gate / up (and the three outputs) must share a leading dimension")
    with _lib.on_device(dy):
        _lib.check(_lib.load().ct_input_gradient_swiglu(
            dy.data_ptr(), _leading(dy), weight.data_ptr(), _leading(weight), a.data_ptr(), low.data_ptr(),
            _leading(low), gate.data_ptr(), up.data_ptr(), _leading(gate), d_gate.data_ptr(), d_up.data_ptr(),
            hidden.data_ptr(), _leading(hidden), rows, width, weight.shape[0], a.shape[0], _lib.code_of(dy.dtype),
            _lib.stream_of(dy)))
    return hidden


def stack_adapters(matrices, dtype, others=()):
    """Row-wise stack of the `a` matrices of projections that share their input, cast to `dtype`,
    and the row offset of each: one product x @ stack.T then yields every projection's low-rank
    input as a column slice, reading x once. `others` (b matrices, biases; None allowed) are cast in
    the same launch; returns (stacked, offsets, cast others)."""
    total = sum(m.shape[0] for m in matrices)
    stacked = torch.empty((total, matrices[0].shape[1]), device=matrices[0].device, dtype=dtype)
    offsets, slices, cursor = [], [], 0
    for matrix in matrices:
        slices.append(stacked[cursor:cursor + matrix.shape[0]])
        offsets.append(cursor)
        cursor += matrix.shape[0]
    converted = cast_many([*matrices, *others], dtype, [*slices, *([None] * len(others))])
    return stacked, offsets, converted[len(matrices):]


def apply_projection(x, weight, b, xa, *, out, bias=None, residual=None):
    """`forward_linear` with the low-rank input xa = x @ a.T already computed (a column slice of a
    stacked product): out = x @ weight.T + bias + xa @ b.T [+ residual]."""
    _lib.require_cuda(x, weight, out, xa)
    x, weight, xa = _readable(x), _readable(weight), _readable(xa)
    _writable(out, "out")
    b = b.contiguous()
    rows, inner = x.shape
    if residual is not None:
        residual = _readable(residual)
    with _lib.on_device(x):
        _lib.check(_lib.load().ct_forward_linear(
            x.data_ptr(), _leading(x), weight.data_ptr(), _leading(weight), None, b.data_ptr(), _lib.pointer(bias),
            _lib.pointer(residual), _leading(residual) if residual is not None else 0, out.data_ptr(), _leading(out),
            xa.data_ptr(), _leading(xa), rows, inner, weight.shape[0], b.shape[1], _lib.code_of(x.dtype),
            _lib.gemm_path, _lib.stream_of(x)))


def token_gradient(left, right, out, *, add=False):
    """out (+)= left.T @ right in fp32, contracted over the shared token dimension in the fixed slice
    order of `parameter_gradients` (kernels/linear.py:16-24 as called at :42-44). `left` may hold the
    low matrices of several projections side by side; `out` is then their stacked dA."""
    _lib.require_cuda(left, right, out)
    if out.dtype != torch.float32 or not out.is_contiguous():
        raise ValueError("token_gradient writes a contiguous fp32 matrix")
    left, right = _readable(left), _readable(right)
    tokens, rows = left.shape
    cols = right.shape[1]
    if right.shape[0] != tokens or out.shape != (rows, cols):
        raise ValueError("token_gradient shape mismatch")
    library = _lib.load()
    code = _lib.code_of(left.dtype)
    need = library.ct_accumulate_workspace(rows, cols, tokens, code, _lib.gemm_path)
    workspace = torch.empty(need, device=left.device, dtype=torch.uint8) if need else None
    with _lib.on_device(left):
        _lib.check(library.ct_accumulate(left.data_ptr(), _leading(left), right.data_ptr(), _leading(right),
                                         out.data_ptr(), rows, cols, tokens, int(bool(add)), code,
                                         _lib.pointer(workspace), _lib.gemm_path, _lib.stream_of(left)))


def token_gradients(problems, *, add=False):
    """Several `token_gradient` products over the same tokens in one launch: `problems` is a list of
    (left, right, out); every out_i (+)= left_i.T @ right_i in fp32 with the fixed slice order of the group
    (ct_token_gradients_group). The adapter gradients of one operator - its stacked dA and each projection's
    dB - have too few output tiles to fill the machine one by one; together they share its waves."""
    import ctypes
    problems = [(l, r, o) for l, r, o in problems if o.numel()]
    if not problems:
        return
    if len(problems) == 1 or len(problems) > 6:
        for left, right, out in problems:
            token_gradient(left, right, out, add=add)
        return
    prepared = []
    for left, right, out in problems:
        _lib.require_cuda(left, right, out)
        if out.dtype != torch.float32 or not out.is_contiguous():
            raise ValueError("token_gradients writes contiguous fp32 matrices")
        left, right = _readable(left), _readable(right)
        if right.shape[0] != left.shape[0] or out.shape != (left.shape[1], right.shape[1]):
            raise ValueError("token_gradients shape mismatch")
        if left.dtype != right.dtype or left.shape[0] != problems[0][0].shape[0] or left.dtype != problems[0][0].dtype:
            raise ValueError("token_gradients contracts operands of one dtype over one token count")
        prepared.append((left, right, out))
    count, tokens = len(prepared), prepared[0][0].shape[0]
    library, code = _lib.load(), _lib.code_of(prepared[0][0].dtype)
    longs = lambda values: (ctypes.c_int64 * count)(*values)
    pointers = lambda tensors: (ctypes.c_void_p * count)(*[t.data_ptr() for t in tensors])
    rows, cols = longs([o.shape[0] for _, _, o in prepared]), longs([o.shape[1] for _, _, o in prepared])
    need = library.ct_token_gradients_group_workspace(count, rows, cols, tokens, code, _lib.gemm_path)
    workspace = torch.empty(need, device=prepared[0][2].device, dtype=torch.uint8) if need else None
    with _lib.on_device(prepared[0][2]):
        _lib.check(library.ct_token_gradients_group(
            count, pointers([l for l, _, _ in prepared]), longs([_leading(l) for l, _, _ in prepared]),
            pointers([r for _, r, _ in prepared]), longs([_leading(r) for _, r, _ in prepared]),
            pointers([o for _, _, o in prepared]), rows, cols, tokens, (ctypes.c_int * count)(*([int(bool(add))] * count)),
            code, _lib.pointer(workspace), _lib.gemm_path, _lib.stream_of(prepared[0][2])))


def parameter_gradients(x, dy, da, db, low, xa, *, add):
    """da (+)= low.T @ x and db (+)= dy.T @ xa in fp32 (kernels/linear.py:42-44), summed in a fixed order."""
    _lib.require_cuda(x, dy, da, db, low, xa)
    if da.dtype != torch.float32 or db.dtype != torch.float32 or not (da.is_contiguous() and db.is_contiguous()):
        # Adapters kept in a 16-bit training dtype: accumulate in fp32 and round once.
        da32 = da.float() if add else torch.empty(da.shape, device=da.device, dtype=torch.float32)
        db32 = db.float() if add else torch.empty(db.shape, device=db.device, dtype=torch.float32)
        parameter_gradients(x, dy, da32, db32, low, xa, add=add)
        da.copy_(da32)
        db.copy_(db32)
        return
    if x.dtype == torch.bfloat16 and _lib.gemm_path != _lib.PATH_SIMT and x.shape[0]:
        token_gradients([(low, x, da), (dy, xa, db)], add=add)      # both products in one launch
        return
    x, dy, low, xa = _readable(x), _readable(dy), _readable(low), _readable(xa)
    rows, inner = x.shape
    outer, rank = dy.shape[1], low.shape[1]
    library = _lib.load()
    code = _lib.code_of(x.dtype)
    need = library.ct_parameter_gradients_workspace(rows, inner, outer, rank, code, _lib.gemm_path)
    workspace = torch.empty(need, device=x.device, dtype=torch.uint8) if need else None
    with _lib.on_device(x):
        _lib.check(library.ct_parameter_gradients(
            x.data_ptr(), _leading(x), dy.data_ptr(), _leading(dy), low.data_ptr(), _leading(low), xa.data_ptr(),
            _leading(xa), da.data_ptr(), db.data_ptr(), rows, inner, outer, rank, int(bool(add)), code,
            _lib.pointer(workspace), _lib.gemm_path, _lib.stream_of(x)))


def projection_parameters(module):
    """((weight, A, B, bias), quant_state or None) of a `Projection` (kernels/linear.py:47-50)."""
    weight = module.weight if module.quantized is None else module.quantized.weight
    state = None if module.quantized is None else weight.quant_state
    return (weight, module.lora_A, module.lora_B, module.bias), state


def can_fuse(module, x):
    """True when the fused operator applies: CUDA input, an adapter, frozen base weight and bias,
    trainable A and B (kernels/linear.py:53-56)."""
    return bool(x.is_cuda and module.rank and not (module.bias is not None and module.bias.requires_grad)
                and (module.weight is None or not module.weight.requires_grad)
                and module.lora_A.requires_grad and module.lora_B.requires_grad)


# Set by project_group around the call: the operator's positional signature mirrors the reference's
# and has no slot for this library's own execution option.
_policy = threading.local()


class _LoRAGroup(torch.autograd.Function):
    """One to three projections that share their input (q/k/v, or a single o/gate/up/down).

    Saves only the input, the rotary table and the parameters (kernels/linear.py:62). The
    backward pass decodes a base weight again only if the input gradient is wanted, rotates
    upstream q/k gradients back into a private buffer, sums the input gradients of the group
    and returns fp32 adapter gradients.
    """

    @staticmethod
    def forward(ctx, x, dtype, tile, states, cosine, sine, head_dim, residual, *parameters):
        _lib.require_cuda(x)
        ctx.dtype, ctx.states, ctx.head_dim = dtype, states, head_dim
        flat = cast(x.reshape(-1, x.shape[-1]), dtype)
        rows = flat.shape[0]
        ctx.tile = tile
        step = max(1, min(tile, rows) if tile else rows)
        widest = max(parameters[4 * i + 1].shape[0] for i in range(len(states)))
        workspace = torch.empty((min(step, rows), widest), device=x.device, dtype=dtype)
        fuse_residual = residual is not None and not head_dim
        shortcut = residual.reshape(rows, residual.shape[-1]) if fuse_residual else None
        outputs = []
        stacked = len(states) > 1 and step >= rows > 0
        keep = bool(getattr(_policy, "keep_low_rank", False)) and step >= rows > 0
        kept = ()         # with `keep`: (low-rank inputs, cast a [stacked], cast b per projection) for backward
        decoded = None
        if stacked:
            # Untiled group (q/k/v): the low-rank inputs of all projections in one product over x,
            # with the base weights decoding beside it.
            decoded, pending = materialize_ahead([(parameters[4 * i], state) for i, state in enumerate(states)], dtype)
            count = len(states)
            a_all, offsets, others = stack_adapters(
                [parameters[4 * i + 1] for i in range(count)], dtype,
                [parameters[4 * i + 2] for i in range(count)] + [parameters[4 * i + 3] for i in range(count)])
            b_cast, bias_cast = others[:count], others[count:]
            xa_all = torch.empty((rows, a_all.shape[0]), device=x.device, dtype=dtype)
            matmul(flat, a_all.T, out=xa_all)
            if keep:
                kept = (xa_all, a_all, *b_cast)
            del a_all
            pending.wait()
        elif keep:
            workspace = torch.empty((rows, widest), device=x.device, dtype=dtype)   # its own buffer: it outlives the call
        for index, state in enumerate(states):
            weight, a, b, bias = parameters[4 * index:4 * index + 4]
            matrix = decoded[index] if decoded is not None else materialize(weight, state, dtype)
            if stacked:
                out = torch.empty((rows, matrix.shape[0]), device=x.device, dtype=dtype)
                apply_projection(flat, matrix, b_cast[index], xa_all[:, offsets[index]:offsets[index] + a.shape[0]],
                                 out=out, bias=bias_cast[index])
                outputs.append(out.reshape(*x.shape[:-1], matrix.shape[0]))
                decoded[index] = None
                del matrix
                continue
            a16, b16, bias16 = cast_many((a, b, bias), dtype)
            out = torch.empty((rows, matrix.shape[0]), device=x.device, dtype=dtype)
            for start in range(0, rows, step):
                stop = min(start + step, rows)
                forward_linear(flat[start:stop], matrix, a16, b16, bias=bias16, out=out[start:stop],
                               xa=workspace[:stop - start, :a.shape[0]],
                               residual=shortcut[start:stop] if fuse_residual and index == 0 else None)
            outputs.append(out.reshape(*x.shape[:-1], matrix.shape[0]))
            if keep and len(states) == 1:
                kept = (workspace[:, :a.shape[0]], a16, b16)
            del matrix, a16, b16
        # Saved through autograd (not as attributes) so that checkpointing and saved-tensor hooks see them.
        ctx.kept = len(kept)
        ctx.save_for_backward(x, cosine, sine, *parameters, *kept)
        if head_dim:
            core_cuda.rotate_owned_qk(outputs[0], outputs[1], cosine, sine, head_dim)
        if residual is not None and not fuse_residual:
            _add_inplace(outputs[0], residual)
        return tuple(outputs)

    @staticmethod
    def backward(ctx, *grad_outputs):
        x, cosine, sine, *parameters = ctx.saved_tensors
        kept = tuple(parameters[len(parameters) - ctx.kept:]) if ctx.kept else ()
        if ctx.kept:
            parameters = parameters[:len(parameters) - ctx.kept]
        dtype, states = ctx.dtype, ctx.states
        flat = cast(x.reshape(-1, x.shape[-1]), dtype)
        rows = flat.shape[0]
        want_dx = ctx.needs_input_grad[0]
        dx = torch.empty_like(flat) if want_dx else None
        step = max(1, min(ctx.tile, rows) if ctx.tile else rows)
        if ctx.head_dim:
            cosine, sine = (value.reshape(-1, value.shape[-1]) for value in (cosine, sine))
        widest = max(parameters[4 * i + 1].shape[0] for i in range(len(states)))
        workspace = torch.empty((2, min(step, rows), widest), device=x.device, dtype=dtype)
        rotary = None
        if ctx.head_dim:
            width = max(parameters[4 * i + 2].shape[0] for i in range(min(2, len(states))))
            rotary = torch.empty(min(step, rows) * width, device=x.device, dtype=dtype)
        results = []
        if want_dx and len(states) > 1 and step >= rows > 0:
            # Untiled group (q/k/v): one GEMM sums the input gradients of all projections.
            prepared = []
            if kept:
                xa_kept, a_all, b_cast = kept[0], kept[1], list(kept[2:])
                offsets, cursor = [], 0
                for i in range(len(states)):
                    offsets.append(cursor)
                    cursor += parameters[4 * i + 1].shape[0]
            else:
                xa_kept = None
                a_all, offsets, b_cast = stack_adapters([parameters[4 * i + 1] for i in range(len(states))], dtype,
                                                        [parameters[4 * i + 2] for i in range(len(states))])
            total = a_all.shape[0]
            low_all = torch.empty((rows, total), device=x.device, dtype=dtype)
            decoded, pending = materialize_ahead([(parameters[4 * i], state) for i, state in enumerate(states)], dtype,
                                                 for_gradient=True)
            for index, (state, grad) in enumerate(zip(states, grad_outputs)):
                weight, a, b, _ = parameters[4 * index:4 * index + 4]
                signal = cast(grad.reshape(-1, grad.shape[-1]), dtype).contiguous()
                if ctx.head_dim and index < 2:
                    signal = core_cuda.inverse_rope_tile(signal, cosine, sine, ctx.head_dim, torch.empty_like(signal))
                span = slice(offsets[index], offsets[index] + a.shape[0])
                prepared.append((decoded[index], a_all[span], b_cast[index], signal, low_all[:, span]))
            del decoded
            pending.wait()
            input_gradient_group([p[3] for p in prepared], [p[0] for p in prepared], [p[1] for p in prepared],
                                 [p[2] for p in prepared], dx, [p[4] for p in prepared])
            # One product recomputes every projection's low-rank input, one more gives the stacked dA
            # (each reads x once); dB is per projection.
            xa_all = xa_kept
            if xa_all is None:
                xa_all = torch.empty((rows, total), device=x.device, dtype=dtype)
                matmul(flat, a_all.T, out=xa_all)
            da_all = torch.empty((total, flat.shape[1]), device=x.device, dtype=torch.float32)
            contractions, db_all = [(low_all, flat, da_all)], []
            for index, (matrix, a16, b16, signal, low) in enumerate(prepared):
                b = parameters[4 * index + 2]
                span = slice(offsets[index], offsets[index] + parameters[4 * index + 1].shape[0])
                db_all.append(torch.empty(b.shape, device=x.device, dtype=torch.float32))
                contractions.append((signal, xa_all[:, span], db_all[-1]))
            token_gradients(contractions)        # the stacked dA and every dB in one launch
            for index in range(len(prepared)):
                a, b = parameters[4 * index + 1], parameters[4 * index + 2]
                span = slice(offsets[index], offsets[index] + a.shape[0])
                da, db = da_all[span], db_all[index]
                results.extend((None, da if a.dtype == torch.float32 else da.to(a.dtype),
                                db if b.dtype == torch.float32 else db.to(b.dtype), None))
            del prepared
            residual_grad = grad_outputs[0] if ctx.needs_input_grad[7] else None
            return (cast(dx.reshape(x.shape), x.dtype), None, None, None, None, None, None, residual_grad, *results)
        for index, (state, grad) in enumerate(zip(states, grad_outputs)):
            weight, a, b, _ = parameters[4 * index:4 * index + 4]
            matrix = materialize_for_gradient(weight, state, dtype) if want_dx else None
            a16, b16 = (kept[1], kept[2]) if kept and len(states) == 1 else cast_many((a, b), dtype)
            dy = cast(grad.reshape(-1, grad.shape[-1]), dtype).contiguous()
            make = torch.empty_like if rows else torch.zeros_like
            da, db = make(a), make(b)
            rotate = bool(ctx.head_dim) and index < 2
            for start in range(0, rows, step):
                stop = min(start + step, rows)
                signal = dy[start:stop]
                if rotate:
                    target = rotary[:signal.numel()].view_as(signal)
                    signal = core_cuda.inverse_rope_tile(signal, cosine[start:stop], sine[start:stop], ctx.head_dim,
                                                         target)
                low = workspace[0, :stop - start, :a.shape[0]]
                xa = workspace[1, :stop - start, :a.shape[0]]
                if want_dx:
                    input_gradient(signal, matrix, a16, b16, dx[start:stop], low, add=index > 0)
                else:
                    matmul(signal, b16, out=low)
                if kept and len(states) == 1:
                    xa = kept[0]               # kept by the forward pass (untiled: one slice)
                else:
                    matmul(flat[start:stop], a16.T, out=xa)
                parameter_gradients(flat[start:stop], signal, da, db, low, xa, add=start > 0)
            results.extend((None, da, db, None))
            del matrix, a16, b16, dy
        residual_grad = grad_outputs[0] if ctx.needs_input_grad[7] else None
        dx_out = None if dx is None else cast(dx.reshape(x.shape), x.dtype)
        return (dx_out, None, None, None, None, None, None, residual_grad, *results)


def _add_inplace(target, other):
    other = other.contiguous()
    with _lib.on_device(target):
        _lib.check(_lib.load().ct_add_inplace(target.data_ptr(), other.data_ptr(), target.numel(),
                                             _lib.code_of(target.dtype), _lib.stream_of(target)))
    return target


def project_group(modules, x, tile=0, *, rotary=None, residual=None):
    """Apply one to three LoRA projections to the same input (kernels/linear.py:133-148).

    rotary = (cosine[..., half], sine[..., half], head_dim) rotates outputs 0 and 1 in place
    before they become visible; `residual` is fused only for a single projection whose output
    matches it in shape and dtype, otherwise it is added outside the operator.
    """
    if residual is not None:
        if len(modules) != 1:
            raise ValueError("Residual fusion requires one output projection")
        shape = (*x.shape[:-1], len(modules[0].lora_B))
        if residual.shape != shape or residual.dtype != modules[0].compute_dtype:
            return (project_group(modules, x, tile, rotary=rotary)[0] + residual,)
    parameters, states = [], []
    for module in modules:
        values, state = projection_parameters(module)
        parameters.extend(values)
        states.append(state)
    cosine, sine, head_dim = (None, None, 0) if rotary is None else rotary
    if rotary is not None:
        cosine, sine = cosine.contiguous(), sine.contiguous()
    _policy.keep_low_rank = torch.is_grad_enabled() and all(getattr(module, "keep_low_rank", False) for module in modules)
    try:
        return _LoRAGroup.apply(x, modules[0].compute_dtype, tile, tuple(states), cosine, sine, head_dim, residual,
                                *parameters)
    finally:
        _policy.keep_low_rank = False
