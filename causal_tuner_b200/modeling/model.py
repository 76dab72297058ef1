"""`Runtime` and the SwiGLU `MLP` block of the decoder (the callers of the two fused operators).

Drop-in for the parts of the reference's modeling/model.py that sit on the projection / MLP
path: `Runtime` (:18-36) and `MLP` (:111-139). The decoder around them (attention, norms,
embedding, checkpoint policy) is outside this package.
"""

from dataclasses import dataclass

import torch
from torch import nn

from .lora import Projection


@dataclass
class Runtime:
    rank: int = 256
    base_dtype: torch.dtype = torch.bfloat16
    train_dtype: torch.dtype = torch.float32
    compute_dtype: torch.dtype = torch.bfloat16
    train_embed: bool = False
    train_head: bool = False
    frozen: tuple = ()
    attention: str = "flash_attention_2"
    mlp_tile: int | None = None
    mlp_cache_budget_bytes: int | None = None
    attention_cache_budget_bytes: int | None = None
    projection_tile: int = 0
    checkpoint: bool = True
    adaptive: bool = False
    group_size: int = 1
    inner_checkpoint: bool = True
    gpu_budget_bytes: int | None = None


class MLP(nn.Module):
    """down(silu(gate(x)) * up(x)); `config` needs `hidden_size` and `intermediate_size`."""

    def __init__(self, config, runtime, device):
        super().__init__()
        self.tile = runtime.mlp_tile
        self.cache_intermediates = False
        kwargs = dict(rank=runtime.rank, base_dtype=runtime.base_dtype, train_dtype=runtime.train_dtype,
                      compute_dtype=runtime.compute_dtype, device=device)
        hidden, inner = config.hidden_size, config.intermediate_size
        self.gate_proj = Projection(hidden, inner, **kwargs)
        self.up_proj = Projection(hidden, inner, **kwargs)
        self.down_proj = Projection(inner, hidden, **kwargs)

    def cache_bytes(self, rows):
        """Bytes the cache=True mode retains for `rows` tokens: gate, up and their low-rank inputs."""
        size = torch.empty((), dtype=self.gate_proj.compute_dtype).element_size()
        return rows * size * sum(p.lora_B.shape[0] + p.rank for p in (self.gate_proj, self.up_proj))

    def untiled(self, x):
        """The same block as three separate autograd nodes that store gate and up (the store-
        activations baseline the recompute mode is compared against)."""
        from ..kernels.mlp_cuda import silu_multiply
        return self.down_proj(silu_multiply(self.gate_proj(x), self.up_proj(x)))

    def forward(self, x, *, residual=None, tile=None, cache=None):
        from ..kernels.linear import can_fuse
        from ..kernels.mlp_cuda import tiled_lora_mlp
        if not x.is_cuda:
            raise RuntimeError("causal_tuner_b200.MLP runs on CUDA tensors only; there is no CPU path")
        if all(can_fuse(module, x) for module in (self.gate_proj, self.up_proj, self.down_proj)):
            return tiled_lora_mlp(self, x, residual, tile=tile, cache=cache)
        raise NotImplementedError("causal_tuner_b200.MLP needs adapters on gate_proj, up_proj and down_proj")
