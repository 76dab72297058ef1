"""NF4 decode in one launch (drop-in for the reference's kernels/nf4_cuda.py)."""

import torch

from .. import _lib


def _statistics(weight, state):
    """(absmax, code, (code2, absmax2, offset) or Nones, nested, auxiliary) as contiguous tensors of the types
    the decode kernels read."""
    if weight.dtype != torch.uint8 or not weight.is_contiguous():
        raise ValueError("packed NF4 weights must be a contiguous uint8 tensor")
    nested = bool(state.nested)
    auxiliary = state.state2 if nested else None
    code = state.code if state.code.dtype == torch.float32 else state.code.float()
    absmax = state.absmax
    if nested:
        if absmax.dtype != torch.uint8:
            raise ValueError("nested NF4 statistics must be uint8")
        code2 = auxiliary.code if auxiliary.code.dtype == torch.float32 else auxiliary.code.float()
        absmax2 = auxiliary.absmax if auxiliary.absmax.dtype == torch.float32 else auxiliary.absmax.float()
        offset = state.offset if state.offset.dtype == torch.float32 else state.offset.float()
        extras = (code2.contiguous(), absmax2.contiguous(), offset.contiguous())
    else:
        if absmax.dtype != torch.float32:
            absmax = absmax.float()
        extras = (None, None, None)
    return absmax.contiguous(), code.contiguous(), extras, nested, auxiliary


BLOCK_ROWS = 128   # row-block size of the interleaved gate / up buffer (half the column width of a GEMM tile)


def dequantize_nf4_blocks(weight, state, pair, which):
    """Decode `weight` [N, K] into the interleaved buffer `pair` [2 N, K]: its rows [128 t, 128 t + 128) become
    rows [256 t + 128 * which, ... + 128) of `pair` (which = 0 for the gate weight, 1 for the up weight) - the B
    operand of the MLP's gated GEMM. Values are those of ``dequantize_nf4(weight, state, pair.dtype)``."""
    _lib.require_cuda(weight, pair)
    outer, inner = state.shape
    if pair.shape != (2 * outer, inner) or not pair.is_contiguous() or outer % BLOCK_ROWS:
        raise ValueError("the interleaved buffer must be a contiguous [2 N, K] tensor with N a multiple of 128")
    absmax, code, extras, nested, auxiliary = _statistics(weight, state)
    chunk = BLOCK_ROWS * inner
    with _lib.on_device(weight):
        _lib.check(_lib.load().ct_nf4_decode_chunks(
            weight.data_ptr(), absmax.data_ptr(), code.data_ptr(), *(_lib.pointer(t) for t in extras),
            pair.data_ptr() + which * chunk * pair.element_size(), outer * inner, int(state.blocksize),
            int(auxiliary.blocksize) if nested else 0, int(nested), _lib.code_of(state.dtype),
            _lib.code_of(pair.dtype), chunk, 2 * chunk, _lib.stream_of(weight)))
    return pair


def transposable(state, dtype):
    """Whether `dequantize_nf4_transposed` can produce this weight: bf16, both extents multiples of 64, block size a
    multiple of 16."""
    shape = tuple(state.shape)
    return (dtype == torch.bfloat16 and len(shape) == 2 and shape[0] % 64 == 0 and shape[1] % 64 == 0
            and 0 < shape[0] // 64 <= 65535 and int(state.blocksize) % 16 == 0)


def dequantize_nf4_transposed(weight, state, dtype):
    """The values of ``dequantize_nf4(weight, state, dtype)`` stored transposed: returns the [N, K] view `.T` of a
    contiguous [K, N] buffer. The input-gradient product dx = dy @ W contracts over N; with this storage W is the
    K-major operand of that GEMM (the operators pass the view straight to `input_gradient`)."""
    _lib.require_cuda(weight)
    if not transposable(state, dtype):
        raise ValueError("transposed decode needs bf16 and extents that are multiples of 64")
    absmax, code, extras, nested, auxiliary = _statistics(weight, state)
    outer, inner = state.shape
    output = torch.empty((inner, outer), device=weight.device, dtype=dtype)
    with _lib.on_device(weight):
        _lib.check(_lib.load().ct_nf4_decode_transposed(
            weight.data_ptr(), absmax.data_ptr(), code.data_ptr(), *(_lib.pointer(t) for t in extras),
            output.data_ptr(), outer, inner, outer, int(state.blocksize), int(auxiliary.blocksize) if nested else 0,
            int(nested), _lib.code_of(state.dtype), _lib.code_of(dtype), _lib.stream_of(weight)))
    return output.T


def dequantize_nf4(weight, state, dtype):
    """Decode packed NF4 `weight` (uint8, two codes per byte) into a dense `dtype` tensor of `state.shape`.

    Same contract as the reference's ``dequantize_nf4`` (kernels/nf4_cuda.py:32-43): plain or
    nested (8-bit) absmax statistics, the fp32 product rounded to ``state.dtype`` and then to
    ``dtype``, bit-exact with the reference decode.
    """
    _lib.require_cuda(weight)
    absmax, code, extras, nested, auxiliary = _statistics(weight, state)
    output = torch.empty(state.shape, device=weight.device, dtype=dtype)
    with _lib.on_device(weight):
        _lib.check(_lib.load().ct_nf4_decode(
            weight.data_ptr(), absmax.data_ptr(), code.data_ptr(), *(_lib.pointer(t) for t in extras),
            output.data_ptr(), output.numel(), int(state.blocksize), int(auxiliary.blocksize) if nested else 0,
            int(nested), _lib.code_of(state.dtype), _lib.code_of(dtype), _lib.stream_of(weight)))
    return output
