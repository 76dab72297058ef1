"""NF4 decode (and a simple encoder) in numpy. Test infrastructure - see oracle/__init__.py."""

import numpy as np
import torch

# NormalFloat-4 levels as published in the QLoRA paper (Dettmers et al. 2023, appendix E).
NF4_LEVELS = np.array([
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
    -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
    0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
    0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0], dtype=np.float32)


def _round(values, dtype):
    """fp32 numpy array -> rounded to a torch dtype (nearest even) -> back to fp32 numpy."""
    if dtype == torch.float32:
        return values.astype(np.float32)
    return torch.from_numpy(np.ascontiguousarray(values, dtype=np.float32)).to(dtype).float().numpy()


def decode(packed, absmax, code, n, blocksize, *, nested=False, code2=None, absmax2=None, offset=None,
           blocksize2=256, state_dtype=torch.float32, out_dtype=torch.float32):
    """Restates kernels/nf4_cuda.py:9-29.

    group g covers elements [g*blocksize, (g+1)*blocksize); byte j holds element 2j in its high
    nibble and 2j+1 in its low nibble (:21-27, `tl.interleave(high, low)`); scale is absmax[g]
    or, nested, code2[absmax[g]] * absmax2[g // blocksize2] + offset with the product and the
    sum rounded separately (:16-19, fp fusion disabled at :42); the fp32 product
    code * scale is cast to the state dtype, then to the output dtype (:29 and tl.store).
    """
    packed = np.asarray(packed, dtype=np.uint8).reshape(-1)[:(n + 1) // 2].astype(np.int32)
    code = np.asarray(code, dtype=np.float32)
    groups = (n + blocksize - 1) // blocksize
    if nested:
        decoded = np.asarray(code2, dtype=np.float32)[np.asarray(absmax, dtype=np.uint8)[:groups].astype(np.int32)]
        maximum = np.asarray(absmax2, dtype=np.float32)[np.arange(groups) // blocksize2]
        product = (decoded * maximum).astype(np.float32)
        scale = (product + np.float32(offset)).astype(np.float32)
    else:
        scale = np.asarray(absmax, dtype=np.float32)[:groups]
    values = np.stack((code[packed >> 4], code[packed & 15]), axis=-1).reshape(-1)[:n]
    scales = np.repeat(scale, blocksize)[:n]
    product = (values.astype(np.float32) * scales.astype(np.float32)).astype(np.float32)
    return _round(_round(product, state_dtype), out_dtype)


def encode(weight, blocksize=64):
    """Per-block absmax, nearest NF4 level (lowest index on ties). Not pinned by the reference."""
    flat = np.asarray(weight, dtype=np.float32).reshape(-1)
    n = flat.size
    groups = (n + blocksize - 1) // blocksize
    padded = np.zeros(groups * blocksize, dtype=np.float32)
    padded[:n] = flat
    padded = padded.reshape(groups, blocksize)
    absmax = np.abs(padded).max(axis=1).astype(np.float32)
    scaled = padded / np.maximum(absmax, np.finfo(np.float32).tiny)[:, None]
    midpoints = (NF4_LEVELS[1:] + NF4_LEVELS[:-1]) / 2
    indices = np.searchsorted(midpoints, scaled.reshape(-1), side="left").astype(np.uint8)[:n + (n & 1)]
    packed = (indices[0::2] << 4) | indices[1::2]
    return packed.astype(np.uint8), absmax


def scale_levels():
    """The 256-level table of the nested statistics: sign(s) * s^2 for 256 evenly spaced s in [-1, 1]."""
    steps = np.linspace(-1.0, 1.0, 256, dtype=np.float64)
    return (np.sign(steps) * np.abs(steps) ** 2).astype(np.float32)


def encode_statistics(absmax, blocksize2=256, code2=None):
    """Nested statistics of the per-block absmax values: (uint8 indices, absmax2, offset).
    offset = mean in fp64 rounded to fp32; the centred values are scaled by their group's
    largest magnitude and mapped to the nearest table level (lowest index on ties).
    Not pinned by the reference (the rule lives in bitsandbytes)."""
    absmax = np.asarray(absmax, dtype=np.float32)
    code2 = scale_levels() if code2 is None else np.asarray(code2, dtype=np.float32)
    blocks = absmax.size
    offset = np.float32(absmax.astype(np.float64).mean())
    centred = (absmax - offset).astype(np.float32)
    groups = (blocks + blocksize2 - 1) // blocksize2
    grid = np.zeros(groups * blocksize2, dtype=np.float32)
    grid[:blocks] = centred
    grid = grid.reshape(groups, blocksize2)
    absmax2 = np.abs(grid).max(axis=1).astype(np.float32)
    normal = (grid / np.maximum(absmax2, np.finfo(np.float32).tiny)[:, None]).astype(np.float32)
    midpoints = ((code2[1:] + code2[:-1]) / 2).astype(np.float32)
    indices = np.searchsorted(midpoints, normal.reshape(-1), side="left").astype(np.uint8)[:blocks]
    return indices, absmax2, offset
