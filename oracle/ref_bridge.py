"""Bridge to the installed reference (oracle/_ref): import it, and give it this library's weights.

TEST INFRASTRUCTURE ONLY. Used by tests/ (parity against the reference's own CUDA path) and
by bench.py's reported baselines; nothing under causal_tuner_b200/ imports it.

The reference packs NF4 through bitsandbytes (modeling/lora.py:41-56), which is not
installed; everything after packing reads a duck-typed object (`module.quantized.weight`
with a `.quant_state`, kernels/linear.py:47-50, kernels/nf4_cuda.py:32-43). `share_nf4` hands
a reference `Projection` the very bytes and quant state this library's `Projection` holds, so
both sides decode the same packed weights and the encoder cannot affect a comparison.
"""

import os
import sys
from types import SimpleNamespace

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")


def available():
    return os.path.exists(os.path.join(REF_ROOT, "causal_tuner", "kernels", "linear.py"))


def load():
    """Put oracle/_ref on sys.path and return the reference package."""
    if not available():
        raise FileNotFoundError(
            "oracle/_ref is missing: run `python oracle/make_ref.py` on a machine that has the reference checkout")
    if REF_ROOT not in sys.path:
        sys.path.insert(0, REF_ROOT)
    import causal_tuner
    return causal_tuner


def share_nf4(reference_projection, holder):
    """Make a reference `Projection` read `holder` (an nn.Module whose `.weight` is the packed
    uint8 tensor carrying `.quant_state`) as its quantised base weight."""
    reference_projection.quantized = holder
    reference_projection.register_parameter("weight", None)


def mirror_projection(ours, device=None):
    """A reference `Projection` with the same base weight (dense or NF4), bias and adapters as `ours`."""
    load()
    from causal_tuner.modeling.lora import Projection
    packed = ours.quantized is not None
    rows, cols = ours.lora_B.shape[0], ours.lora_A.shape[1]
    device = device or ours.lora_A.device
    base_dtype = ours.bias.dtype if ours.bias is not None else (torch.bfloat16 if packed else ours.weight.dtype)
    module = Projection(cols, rows, bias=ours.bias is not None, rank=ours.rank, base_dtype=base_dtype,
                        train_dtype=ours.lora_A.dtype, compute_dtype=ours.compute_dtype,
                        device="meta" if packed else device)
    if packed:
        module = module.to_empty(device=device)
        share_nf4(module, ours.quantized)
    with torch.no_grad():
        if not packed:
            module.weight.copy_(ours.weight)
        module.lora_A.copy_(ours.lora_A)
        module.lora_B.copy_(ours.lora_B)
        if ours.bias is not None:
            module.bias.copy_(ours.bias)
    return module


def mirror_model(ours, **runtime_overrides):
    """A reference `CausalLM` that shares every frozen tensor of `ours` (packed NF4 weights, biases,
    norms, embedding, head) and starts from copies of its adapters. Built on the meta device first,
    so no dense base weight is ever allocated."""
    load()
    from causal_tuner.modeling.config import ModelConfig
    from causal_tuner.modeling.model import CausalLM, Runtime
    config = ModelConfig(**{name: getattr(ours.config, name) for name in
                            ("hidden_size", "intermediate_size", "vocab_size", "num_hidden_layers",
                             "num_attention_heads", "head_dim", "partial_rotary_factor", "rope_theta", "rms_norm_eps",
                             "max_position_embeddings", "pad_token_id", "eos_token_id")})
    r = ours.runtime
    settings = dict(rank=r.rank, base_dtype=r.base_dtype, train_dtype=r.train_dtype, compute_dtype=r.compute_dtype,
                    attention=r.attention, mlp_tile=r.mlp_tile, mlp_cache_budget_bytes=r.mlp_cache_budget_bytes,
                    projection_tile=r.projection_tile, checkpoint=r.checkpoint)
    settings.update(runtime_overrides)
    model = CausalLM(config, Runtime(**settings), "meta")
    own_modules = dict(ours.named_modules())
    own_parameters = dict(ours.named_parameters())
    for name, module in model.named_modules():
        mine = own_modules.get(name)
        if mine is not None and getattr(mine, "quantized", None) is not None and hasattr(module, "lora_A"):
            share_nf4(module, mine.quantized)
    for name, parameter in list(model.named_parameters()):
        if ".quantized." in name:
            continue
        source = own_parameters[name]
        owner = model.get_submodule(name.rpartition(".")[0]) if "." in name else model
        data = source.detach().clone() if parameter.requires_grad else source.detach()
        setattr(owner, name.rpartition(".")[2], torch.nn.Parameter(data, requires_grad=parameter.requires_grad))
    for name, parameter in model.named_parameters():
        if parameter.is_meta:
            raise RuntimeError(f"reference parameter {name} was not materialised")
    return model


def trainer_arguments(**overrides):
    """The argument record `Trainer` and `make_optimizer` of the reference read (training/engine.py:10-107),
    with the defaults of its arguments.json except that packs are never re-grouped."""
    values = dict(learning_rate=2e-5, learning_rate_end=0.0, weight_decay=0.0, adam_beta1=0.9, adam_beta2=0.999,
                  adam_epsilon=1e-8, warmup_steps=0, scheduler="constant", microbatch_token_budget=0,
                  data_buffer_budget_mib=1024, loss_token_budget=128, loss_implementation="fused", cut_chunk_size=0,
                  max_grad_norm=1.0)
    values.update(overrides)
    return SimpleNamespace(**values)


def reference_trainer(model, device, **overrides):
    load()
    from causal_tuner.training.engine import Trainer, make_optimizer
    arguments = trainer_arguments(**overrides)
    return Trainer(model, make_optimizer(model, arguments), arguments, device=device)
