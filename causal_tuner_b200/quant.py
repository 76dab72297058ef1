"""NF4 quantisation of frozen base weights and the quant-state record the decode kernel reads.

Quantisation is set-up work done once per weight: `ct_nf4_encode` / `ct_nf4_nest` for a weight
on a GPU, the same rule in plain tensor ops for a host tensor (the two agree bit for bit); only
decoding is on the training path. The layout is the one the
reference consumes (kernels/nf4_cuda.py:9-29): blocks of `blocksize` consecutive elements
of the flattened weight share one fp32 absmax; element 2j of the flattened weight sits in
the high nibble of byte j, element 2j+1 in the low nibble. With `nested=True` the absmax
values are themselves stored as 8-bit indices into a 256-entry table with one fp32 scale
per `blocksize2` blocks plus a common offset (their mean).
"""

from dataclasses import dataclass, field

import torch

# The sixteen NormalFloat-4 levels of the QLoRA paper (Dettmers et al., 2023, appendix E).
NF4_LEVELS = (
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
    -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
    0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
    0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0)


def nf4_code(device=None):
    return torch.tensor(NF4_LEVELS, dtype=torch.float32, device=device)


def scale_code(device=None):
    """256-level table for nested absmax statistics: signed, denser near zero."""
    steps = torch.linspace(-1.0, 1.0, 256, dtype=torch.float64)
    return (steps.sign() * steps.abs().pow(2)).to(torch.float32).to(device)


@dataclass
class NestedState:
    code: torch.Tensor
    absmax: torch.Tensor
    blocksize: int


@dataclass
class QuantState:
    """Attribute-compatible with the quant-state object the reference reads
    (kernels/nf4_cuda.py:33-41, kernels/linear.py:8,49)."""
    shape: torch.Size
    dtype: torch.dtype
    blocksize: int
    absmax: torch.Tensor
    code: torch.Tensor
    quant_type: str = "nf4"
    nested: bool = False
    offset: torch.Tensor | None = None
    state2: NestedState | None = None
    extra: dict = field(default_factory=dict)

    def to(self, device):
        self.absmax, self.code = self.absmax.to(device), self.code.to(device)
        if self.nested:
            self.offset = self.offset.to(device)
            self.state2.code, self.state2.absmax = self.state2.code.to(device), self.state2.absmax.to(device)
        return self


def _nearest(values, table):
    """Index of the nearest table entry (lowest index on ties); table is sorted ascending."""
    midpoints = (table[1:] + table[:-1]) / 2
    return torch.bucketize(values, midpoints, right=False)


def quantize_nf4(weight, blocksize=64, nested=False, blocksize2=256):
    """Return (packed uint8 [ceil(n/2), 1], QuantState) for a floating-point weight."""
    if blocksize <= 0 or blocksize % 2:
        raise ValueError("blocksize must be a positive even number")
    device = weight.device
    if weight.is_cuda and _device_encoder_takes(weight, blocksize, blocksize2):
        return _quantize_on_device(weight, blocksize, nested, blocksize2)
    flat = weight.detach().reshape(-1).to(torch.float32)
    n = flat.numel()
    blocks = -(-n // blocksize)
    padded = torch.zeros(blocks * blocksize, dtype=torch.float32, device=device)
    padded[:n] = flat
    padded = padded.view(blocks, blocksize)
    absmax = padded.abs().amax(dim=1)
    scaled = padded / absmax.clamp_min(torch.finfo(torch.float32).tiny)[:, None]
    code = nf4_code(device)
    indices = _nearest(scaled.reshape(-1), code)[:n + (n & 1)].to(torch.uint8)
    if n & 1 and indices.numel() < n + 1:
        indices = torch.cat((indices, indices.new_zeros(1)))
    packed = (indices[0::2] << 4) | indices[1::2]
    state = QuantState(shape=weight.shape, dtype=weight.dtype, blocksize=blocksize, absmax=absmax, code=code)
    if nested:
        offset = absmax.double().mean().float()   # fp64 accumulation: the value does not depend on the summation order
        centred = absmax - offset
        groups = -(-blocks // blocksize2)
        grid = torch.zeros(groups * blocksize2, dtype=torch.float32, device=device)
        grid[:blocks] = centred
        grid = grid.view(groups, blocksize2)
        absmax2 = grid.abs().amax(dim=1)
        table = scale_code(device)
        normal = grid / absmax2.clamp_min(torch.finfo(torch.float32).tiny)[:, None]
        state.absmax = _nearest(normal.reshape(-1), table)[:blocks].to(torch.uint8)
        state.nested, state.offset = True, offset.reshape(())
        state.state2 = NestedState(code=table, absmax=absmax2, blocksize=blocksize2)
    return packed.reshape(-1, 1).contiguous(), state


def _device_encoder_takes(weight, blocksize, blocksize2):
    return (weight.dtype in (torch.float32, torch.bfloat16, torch.float16) and 8 <= blocksize <= 256
            and blocksize & (blocksize - 1) == 0 and blocksize2 > 0)


def _quantize_on_device(weight, blocksize, nested, blocksize2):
    """`quantize_nf4` through the CUDA encoder; same outputs as the tensor-op rule above."""
    from . import _lib
    device = weight.device
    flat = weight.detach().reshape(-1).contiguous()
    n = flat.numel()
    blocks = -(-n // blocksize)
    packed = torch.empty((n + 1) // 2, dtype=torch.uint8, device=device)
    absmax = torch.empty(blocks, dtype=torch.float32, device=device)
    code = nf4_code(device)
    library = _lib.load()
    with _lib.on_device(flat):
        stream = _lib.stream_of(flat)
        _lib.check(library.ct_nf4_encode(flat.data_ptr(), n, _lib.code_of(flat.dtype), blocksize, code.data_ptr(),
                                         packed.data_ptr(), absmax.data_ptr(), stream))
        state = QuantState(shape=weight.shape, dtype=weight.dtype, blocksize=blocksize, absmax=absmax, code=code)
        if nested:
            groups = -(-blocks // blocksize2)
            table = scale_code(device)
            quantised = torch.empty(blocks, dtype=torch.uint8, device=device)
            absmax2 = torch.empty(groups, dtype=torch.float32, device=device)
            offset = torch.empty((), dtype=torch.float32, device=device)
            _lib.check(library.ct_nf4_nest(absmax.data_ptr(), blocks, blocksize2, table.data_ptr(),
                                           quantised.data_ptr(), absmax2.data_ptr(), offset.data_ptr(), stream))
            state.absmax, state.nested, state.offset = quantised, True, offset
            state.state2 = NestedState(code=table, absmax=absmax2, blocksize=blocksize2)
    return packed.reshape(-1, 1), state
