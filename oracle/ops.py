"""Projection, SwiGLU MLP and RoPE on the CPU with torch. Test infrastructure - see oracle/__init__.py.

All functions take and return CPU tensors. `dtype` is the compute dtype; with bfloat16 every
matrix product rounds to bf16 where the reference's CPU branch does.
"""

import torch
from torch.nn import functional as F


def projection(x, weight, a, b, bias=None, dtype=torch.float32):
    """Restates the non-fused branch of Projection.forward, modeling/lora.py:29-39:
    F.linear(x, W, bias) + F.linear(F.linear(x, A), B), everything cast to the compute dtype."""
    x = x.to(dtype)
    out = F.linear(x, weight.to(dtype), None if bias is None else bias.to(dtype))
    if a is not None:
        out = out + F.linear(F.linear(x, a.to(dtype)), b.to(dtype))
    return out


def projection_backward(x, weight, a, b, dy, dtype=torch.float32):
    """Restates _LoRAGroup.backward for one projection, kernels/linear.py:107-126:
    low = dy.B, dx = dy.W + low.A, xa = x.A^T, dA = low^T.x, dB = dy^T.xa (dA, dB in fp32,
    kernels/linear.py:16-24)."""
    x, dy, w, ac, bc = x.to(dtype), dy.to(dtype), weight.to(dtype), a.to(dtype), b.to(dtype)
    low = dy @ bc
    dx = dy @ w + low @ ac
    xa = x @ ac.T
    da = low.float().T @ x.float()
    db = dy.float().T @ xa.float()
    return dx, da, db


def swiglu(gate, up):
    """Restates kernels/mlp_cuda.py:12-25, forward: round(g * sigmoid(g)) * u in the tensor dtype."""
    g = gate.float()
    activated = (g * torch.sigmoid(g)).to(gate.dtype).float()
    return (activated * up.float()).to(gate.dtype)


def swiglu_backward(gate, up, grad):
    """Restates kernels/mlp_cuda.py:18-23: returns (d_gate, d_up)."""
    g, u, dh = gate.float(), up.float(), grad.float()
    s = torch.sigmoid(g)
    activated = (g * s).to(gate.dtype).float()
    product_grad = (dh * u).to(gate.dtype).float()
    dgate = product_grad * (s * (1 + g * (1 - s)))
    return dgate.to(gate.dtype), (dh * activated).to(gate.dtype)


def mlp(x, gate, up, down, dtype=torch.float32):
    """Restates MLP.untiled on the CPU, modeling/model.py:127-131:
    down(silu(gate(x)) * up(x)); each of gate/up/down is a (weight, A, B) triple."""
    g = projection(x, *gate, dtype=dtype)
    u = projection(x, *up, dtype=dtype)
    return projection(F.silu(g) * u, *down, dtype=dtype)


def rotate(x, cosine, sine, inverse=False):
    """Restates modeling/rotary.py:16-24 (adjacent-pair partial RoPE on x[..., heads, head_dim]);
    in a 16-bit dtype every product rounds before the add, as kernels/core_cuda.py:134-142 does.
    inverse=True negates the sine (the backward rotation, kernels/core_cuda.py:136-137)."""
    size = cosine.shape[-1] * 2
    cosine, sine = cosine.unsqueeze(-2), sine.unsqueeze(-2)
    if inverse:
        sine = -sine
    even, odd = x[..., :size:2], x[..., 1:size:2]
    paired = torch.stack((even * cosine - odd * sine, odd * cosine + even * sine), dim=-1)
    return torch.cat((paired.flatten(-2), x[..., size:]), dim=-1)
