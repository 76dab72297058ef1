"""`Projection`: a frozen base weight (dense or NF4) with a unit-scale rank-r adapter.

Drop-in for the reference's modeling/lora.py:9-62. Differences: NF4 packing is done by this
package's own quantiser (no bitsandbytes), and the forward pass has no CPU branch - a
non-CUDA input is an error.
"""

import math

import torch
from torch import nn

from ..quant import quantize_nf4


class _PackedWeight(nn.Module):
    """Holder of the packed NF4 bytes; `weight.quant_state` is what the operators read
    (kernels/linear.py:47-50 of the reference)."""

    def __init__(self, packed, state):
        super().__init__()
        self.weight = nn.Parameter(packed, requires_grad=False)
        self.weight.quant_state = state

    def _apply(self, fn, recurse=True):
        state = self.weight.quant_state
        super()._apply(fn, recurse)
        self.weight.quant_state = state.to(self.weight.device)
        return self


class Projection(nn.Module):
    def __init__(self, inputs, outputs, *, bias=False, rank=0, base_dtype=torch.bfloat16,
                 train_dtype=torch.float32, compute_dtype=torch.bfloat16, device=None):
        super().__init__()
        self.compute_dtype, self.rank = compute_dtype, rank
        self.weight = nn.Parameter(torch.empty(outputs, inputs, dtype=base_dtype, device=device),
                                   requires_grad=not rank)
        self.bias = nn.Parameter(torch.zeros(outputs, dtype=base_dtype, device=device),
                                 requires_grad=not rank) if bias else None
        self.quantized = None
        if rank:
            self.lora_A = nn.Parameter(torch.empty(rank, inputs, dtype=train_dtype, device=device))
            self.lora_B = nn.Parameter(torch.zeros(outputs, rank, dtype=train_dtype, device=device))
            bound = math.sqrt(6 / inputs)
            nn.init.uniform_(self.lora_A, -bound, bound)
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x):
        from ..kernels.linear import can_fuse, project_group
        if not x.is_cuda:
            raise RuntimeError("causal_tuner_b200.Projection runs on CUDA tensors only; there is no CPU path")
        if can_fuse(self, x):
            return project_group((self,), x)[0]
        raise NotImplementedError(
            "causal_tuner_b200 covers the fused adapter path only: rank > 0, frozen base weight and bias, "
            "trainable lora_A and lora_B")

    def install_nf4(self, weight, device, *, blocksize=64, nested=True):
        """Replace the dense base weight by its NF4 packing on `device` (modeling/lora.py:41-56)."""
        if not self.rank or weight.requires_grad:
            raise ValueError("NF4 is restricted to frozen adapter base projections")
        if torch.device(device).type != "cuda":
            raise ValueError("NF4 requires a CUDA device")
        packed, state = quantize_nf4(weight.detach().to(device), blocksize=blocksize, nested=nested)
        self.quantized = _PackedWeight(packed, state)
        self.register_parameter("weight", None)

    def base_weight(self):
        if self.quantized is None:
            return self.weight
        from ..kernels.nf4_cuda import dequantize_nf4
        packed = self.quantized.weight
        return dequantize_nf4(packed.data, packed.quant_state, packed.quant_state.dtype)
