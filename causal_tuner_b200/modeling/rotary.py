"""Partial adjacent-pair RoPE at the requested logical positions (modeling/rotary.py:6-24)."""

import torch

from ..kernels.core_cuda import PartialRoPE, position_values


def rotary_values(positions, config, dtype):
    channel = torch.arange(0, config.rotary_dim, 2, device=positions.device, dtype=torch.float32)
    inverse = 1.0 / (config.rope_theta ** (channel / config.rotary_dim))
    return position_values(positions, inverse, dtype)


def rotate(x, cosine, sine):
    if not x.is_cuda:
        raise RuntimeError("causal_tuner_b200 rotate runs on CUDA tensors only; there is no CPU path")
    return PartialRoPE.apply(x, cosine.contiguous(), sine.contiguous())
