"""The decoder around the two fused operators: `Runtime`, `RMSNorm`, `Attention`, `MLP`, `Layer`,
`CausalLM`.

Class names, constructor arguments and attributes are those of the reference's modeling/model.py
(:18-279) because callers and checkpoints address them by name; the bodies call this package's
operators only. Adapter training is covered (rank > 0, frozen base weights); the execution policy
is explicit in `Runtime` (layer checkpointing on or off, an MLP activation-cache byte budget, kept
low-rank inputs) instead of being derived from free memory, and nothing is offloaded.
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
    # Keep the low-rank inputs x @ A.T of q/k/v/o (and, in layers that cache their MLP activations,
    # of the down projection) between forward and backward - 2 bytes x rank per token and
    # projection - instead of recomputing them; the reference always recomputes (False).
    keep_low_rank: bool = False
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
        for projection in (self.gate_proj, self.up_proj, self.down_proj):
            projection.keep_low_rank = getattr(runtime, "keep_low_rank", False)

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


# ---- the decoder around the two operators ------------------------------------------------------
# RMSNorm, Attention, Layer and CausalLM follow modeling/model.py:39-279 of the reference with the
# execution policy made explicit: `runtime.checkpoint` recomputes each layer in backward, the MLP
# always recomputes gate/up unless `layer.mlp.cache_intermediates` is set, nothing is offloaded.

class RMSNorm(nn.Module):
    """RMS normalisation with a weight per channel (modeling/model.py:39-66 of the reference).

    A frozen bf16 norm that hands its input gradient buffer back (`reuse_grad`) also uses the
    output-reconstruction mode when every weight magnitude lies in [1/256, 256]: the backward pass
    then needs the output only, which the following projection keeps anyway."""

    def __init__(self, size, eps, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(size, dtype=dtype, device=device))
        self.eps = eps
        self._reconstruction_cache = None

    def _can_reconstruct(self, dtype):
        weight = self.weight
        if dtype != torch.bfloat16 or weight.requires_grad or torch.is_inference(weight):
            return False
        key = (weight.data_ptr(), weight._version, dtype)
        cached = self._reconstruction_cache
        if cached is None or cached[0] != key:
            if torch.cuda.is_current_stream_capturing():
                return False            # the check below reads a value back to the host
            magnitude = weight.detach().to(dtype).abs()
            cached = self._reconstruction_cache = (key, bool(((magnitude >= 1 / 256) & (magnitude <= 256)).all()))
        return cached[1]

    def _require_cuda(self, x):
        if not x.is_cuda:
            raise RuntimeError("causal_tuner_b200.RMSNorm runs on CUDA tensors only; there is no CPU path")

    def forward(self, x, *, reuse_grad=False):
        from ..kernels.core_cuda import RMS
        self._require_cuda(x)
        reconstruct = reuse_grad and torch.is_grad_enabled() and self._can_reconstruct(x.dtype)
        return RMS.apply(x, self.weight, self.eps, reuse_grad, reconstruct)

    def with_shortcut(self, x):
        """(norm(x), x) for `x + block(norm(x))`; with a frozen weight the two gradients of x are summed
        inside the norm's backward kernel instead of by a separate add."""
        from ..kernels.core_cuda import RMS, RMSWithShortcut
        self._require_cuda(x)
        if self.weight.requires_grad:
            return RMS.apply(x, self.weight, self.eps, False, False), x
        reconstruct = torch.is_grad_enabled() and self._can_reconstruct(x.dtype)
        return RMSWithShortcut.apply(x, self.weight, self.eps, reconstruct)


class Attention(nn.Module):
    def __init__(self, config, runtime, device):
        super().__init__()
        self.config, self.runtime = config, runtime
        kwargs = dict(rank=runtime.rank, base_dtype=runtime.base_dtype, train_dtype=runtime.train_dtype,
                      compute_dtype=runtime.compute_dtype, device=device)
        h, d = config.hidden_size, config.head_dim
        self.q_proj = Projection(h, h, bias=True, **kwargs)
        self.k_proj = Projection(h, d, bias=True, **kwargs)
        self.v_proj = Projection(h, d, bias=True, **kwargs)
        self.o_proj = Projection(h, h, **kwargs)
        for projection in (self.q_proj, self.k_proj, self.v_proj, self.o_proj):
            projection.keep_low_rank = runtime.keep_low_rank

    def forward(self, x, cosine, sine, segments, spans, layout=None, *, residual=None):
        from ..kernels.attention import dense_attention, flash_dense
        from ..kernels.linear import project_group
        b, s, _ = x.shape
        c, r = self.config, self.runtime
        q, k, v = project_group((self.q_proj, self.k_proj, self.v_proj), x, r.projection_tile,
                                rotary=(cosine, sine, c.head_dim))
        q, k = q.reshape(b, s, c.num_attention_heads, c.head_dim), k.reshape(b, s, 1, c.head_dim)
        v = v.reshape(b, s, 1, c.head_dim)
        if r.attention == "vanilla":
            y = dense_attention(q, k, v, segments)
        else:
            y = flash_dense(q, k, v, spans, layout=layout)
        return project_group((self.o_proj,), y.reshape(b, s, -1), r.projection_tile, residual=residual)[0]


class Layer(nn.Module):
    def __init__(self, config, runtime, device):
        super().__init__()
        self.self_attn = Attention(config, runtime, device)
        self.mlp = MLP(config, runtime, device)
        self.input_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps, runtime.base_dtype, device)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps, runtime.base_dtype, device)

    def forward(self, x, *args, mlp_tile=None, mlp_cache=None):
        # Both norms feed operators that return private input gradients, so the norm backward may
        # write over its upstream gradient, and it adds the residual path's gradient while it does.
        normed, shortcut = self.input_layernorm.with_shortcut(x)
        x = self.self_attn(normed, *args, residual=shortcut)
        normed, shortcut = self.post_attention_layernorm.with_shortcut(x)
        return self.mlp(normed, residual=shortcut, tile=mlp_tile, cache=mlp_cache)


class Decoder(nn.Module):
    def __init__(self, config, runtime, device):
        super().__init__()
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, padding_idx=config.pad_token_id,
                                         dtype=runtime.base_dtype, device=device)
        self.layers = nn.ModuleList([Layer(config, runtime, device) for _ in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps, runtime.base_dtype, device)


class CausalLM(nn.Module):
    """Adapter-training decoder: base weights, biases and norms are frozen; lora_A / lora_B of the
    seven projections per layer train in `runtime.train_dtype`, and so do the embedding and the head
    when `runtime.train_embed` / `runtime.train_head` ask for it (modeling/model.py:185-193 of the
    reference)."""

    def __init__(self, config, runtime, device=None):
        super().__init__()
        if not runtime.rank:
            raise NotImplementedError("causal_tuner_b200 covers adapter training (rank > 0) only")
        self.config, self.runtime = config, runtime
        self.last_execution = {}
        self.model = Decoder(config, runtime, device)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False, dtype=runtime.base_dtype,
                                 device=device)
        for name, param in self.named_parameters():
            trainable = ("lora_" in name or ("embed_tokens" in name and runtime.train_embed)
                         or (name.startswith("lm_head") and runtime.train_head))
            param.requires_grad_(trainable)
            if trainable:
                param.data = param.data.to(runtime.train_dtype)

    def install_nf4(self, *, blocksize=64, nested=False):
        """Pack every projection's base weight to NF4 in place (weights must already be on a CUDA device)."""
        for layer in self.model.layers:
            for projection in (layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj,
                               layer.self_attn.o_proj, layer.mlp.gate_proj, layer.mlp.up_proj, layer.mlp.down_proj):
                weight = projection.weight.detach()
                projection.install_nf4(weight, weight.device, blocksize=blocksize, nested=nested)
        return self

    def adapter_parameters(self):
        return [p for p in self.parameters() if p.requires_grad]

    def forward(self, batch):
        from torch.utils.checkpoint import checkpoint
        from ..kernels.attention import prepare_dense_layout
        from ..segments import canonical_segments, position_ids, runs
        from .rotary import rotary_values
        r = self.runtime
        segments = canonical_segments(batch["attention_mask"], batch.get("segment_ids"))
        positions = batch.get("position_ids")
        if positions is None:
            positions = position_ids(segments)
        if (positions < 0).any() or (positions >= self.config.max_position_embeddings).any():
            raise ValueError("position_ids exceed the model's logical position range")
        spans = batch.get("_spans") or runs(segments)
        cosine, sine = rotary_values(positions, self.config, r.compute_dtype)
        x = self.model.embed_tokens(batch["input_ids"]).to(r.compute_dtype)
        layout = prepare_dense_layout(x.shape[:2], spans, x.device) if r.attention == "flash_attention_2" else None
        recompute = r.checkpoint and self.training and torch.is_grad_enabled()
        # MLP activation cache: layers keep gate/up (instead of recomputing them in backward) while
        # the byte budget lasts, last layers first (modeling/model.py:228-239 of the reference).
        remaining = r.mlp_cache_budget_bytes or 0
        if not torch.is_grad_enabled() or recompute:
            remaining = 0
        tokens = x.numel() // x.shape[-1]
        retained = 0
        for layer in reversed(self.model.layers):
            cost = layer.mlp.cache_bytes(tokens) if remaining else 0
            layer.mlp.cache_intermediates = bool(cost and cost <= remaining)
            if layer.mlp.cache_intermediates:
                remaining -= cost
                retained += cost
        self.last_execution = dict(rows=tokens, checkpoint=recompute, mlp_cache_bytes=retained,
                                   mlp_cache_layers=sum(l.mlp.cache_intermediates for l in self.model.layers))
        for layer in self.model.layers:
            run = lambda z, layer=layer: layer(z, cosine, sine, segments, spans, layout, mlp_tile=r.mlp_tile,
                                                mlp_cache=layer.mlp.cache_intermediates)
            x = checkpoint(run, x, use_reentrant=False, preserve_rng_state=False) if recompute else run(x)
        return self.model.norm(x)
