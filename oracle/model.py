"""The reference decoder and one optimizer step, restated with plain torch on the CPU.
Test infrastructure - see oracle/__init__.py. Pinned by tests/golden/step_tiny_b*.npz.

`params` maps the reference's parameter names (model.layers.0.self_attn.q_proj.weight, ...) to
CPU tensors; adapters (lora_A / lora_B) may require grad.
"""

import torch
from torch.nn import functional as F

from . import ops


def rms_norm(x, weight, eps):
    """modeling/model.py:65-66 (CPU branch of RMSNorm.forward)."""
    normalized = x.float() * torch.rsqrt(x.float().square().mean(-1, keepdim=True) + eps)
    return normalized.to(x.dtype) * weight.to(x.dtype)


def segments_of(mask, labels):
    """data/segments.py:6-17."""
    valid = mask.bool()
    previous = F.pad(valid[:, :-1], (1, 0), value=False)
    changed = F.pad(labels[:, 1:] != labels[:, :-1], (1, 0), value=True)
    return (valid & (~previous | changed)).to(torch.int32).cumsum(1).to(torch.int32) * valid


def positions_of(segments):
    """data/segments.py:20-24."""
    index = torch.arange(segments.shape[1]).expand_as(segments)
    previous = F.pad(segments[:, :-1], (1, 0))
    starts = torch.where((segments != previous) & (segments > 0), index, 0)
    return torch.where(segments > 0, index - starts.cummax(1).values, 0)


def dense_attention(q, k, v, segments):
    """kernels/reference.py:11-27: same document, causal, fp32 softmax."""
    s = q.shape[1]
    index = torch.arange(s)
    mask = ((segments[:, :, None] == segments[:, None, :]) & (segments[:, :, None] > 0)
            & (index[None, None, :] <= index[None, :, None]))[:, None]
    score = torch.einsum("bqhd,bkd->bhqk", q.float(), k[:, :, 0].float()) / q.shape[-1] ** 0.5
    score = score.masked_fill(~mask, -torch.inf)
    score = torch.where(mask.any(-1, keepdim=True), score, 0)
    probs = torch.softmax(score, -1) * mask
    return torch.einsum("bhqk,bkd->bqhd", probs, v[:, :, 0].float()).to(q.dtype)


def project(params, prefix, x, dtype):
    return ops.projection(x, params[prefix + ".weight"], params[prefix + ".lora_A"], params[prefix + ".lora_B"],
                          params.get(prefix + ".bias"), dtype)


def layer(params, prefix, x, cosine, sine, segments, heads, head_dim, eps, dtype):
    """modeling/model.py:150-156 with Attention (:81-108) and MLP.untiled (:127-131)."""
    b, s, _ = x.shape
    y = rms_norm(x, params[prefix + ".input_layernorm.weight"], eps)
    q = ops.rotate(project(params, prefix + ".self_attn.q_proj", y, dtype).reshape(b, s, heads, head_dim), cosine, sine)
    k = ops.rotate(project(params, prefix + ".self_attn.k_proj", y, dtype).reshape(b, s, 1, head_dim), cosine, sine)
    v = project(params, prefix + ".self_attn.v_proj", y, dtype).reshape(b, s, 1, head_dim)
    attended = dense_attention(q, k, v, segments).reshape(b, s, -1)
    x = x + project(params, prefix + ".self_attn.o_proj", attended, dtype)
    y = rms_norm(x, params[prefix + ".post_attention_layernorm.weight"], eps)
    hidden = F.silu(project(params, prefix + ".mlp.gate_proj", y, dtype)) * project(params, prefix + ".mlp.up_proj", y, dtype)
    return x + project(params, prefix + ".mlp.down_proj", hidden, dtype)


def forward(params, batch, *, layers, heads, head_dim, rotary_dim, theta, eps, dtype=torch.float32):
    """modeling/model.py:195-279 without checkpointing: final-norm hidden states."""
    segments = segments_of(batch["attention_mask"], batch["segment_ids"])
    positions = positions_of(segments)
    channel = torch.arange(0, rotary_dim, 2, dtype=torch.float32)
    angle = positions.float()[..., None] * (1.0 / (theta ** (channel / rotary_dim)))
    cosine, sine = angle.cos().to(dtype), angle.sin().to(dtype)
    x = F.embedding(batch["input_ids"], params["model.embed_tokens.weight"]).to(dtype)
    for index in range(layers):
        x = layer(params, f"model.layers.{index}", x, cosine, sine, segments, heads, head_dim, eps, dtype)
    return rms_norm(x, params["model.norm.weight"], eps), segments


def step_loss(params, batch, **config):
    """Weighted next-token loss of training/engine.py:68-87 with data/segments.py:41-58:
    returns (sum of weighted CE, total weight)."""
    dtype = config.get("dtype", torch.float32)
    hidden, segments = forward(params, batch, **config)
    ids, valid = batch["input_ids"], batch["attention_mask"].bool()
    edges = valid[:, :-1] & valid[:, 1:] & (segments[:, :-1] == segments[:, 1:])
    targets = F.pad(ids[:, 1:], (0, 1))
    weights = F.pad(edges.float(), (0, 1))
    logits = F.linear(hidden.to(dtype), params["lm_head.weight"].to(dtype)).float()
    losses = F.cross_entropy(logits.flatten(0, 1), targets.flatten(), reduction="none") * weights.flatten()
    return losses.sum(), weights.sum()
