"""The CPU restatement of the decoder step (oracle/model.py) against the fixture produced by the reference."""

import numpy as np
import pytest
import torch

from oracle import model as oracle_model
from oracle import nf4 as oracle_nf4

CONFIG = dict(layers=2, heads=4, head_dim=64, rotary_dim=32, theta=1e4, eps=1e-5)


def params_of(g):
    params = {}
    for key in g:
        kind, _, rest = key.partition("__")
        name = rest.replace("__", ".")
        if kind in ("a", "b"):
            params[name] = torch.from_numpy(g[key]).clone().requires_grad_(True)
        elif kind == "v":
            params[name] = torch.from_numpy(g[key])
        elif kind == "q":
            scale = g["s__" + rest]
            shape = {"model.embed_tokens.weight": (1024, 256), "lm_head.weight": (1024, 256)}.get(name)
            values = oracle_nf4.decode(g[key], scale, oracle_nf4.NF4_LEVELS, g[key].size * 2, 64)
            params[name] = (torch.from_numpy(values), shape)
    widths = {"q_proj": (256, 256), "k_proj": (64, 256), "v_proj": (64, 256), "o_proj": (256, 256),
              "gate_proj": (688, 256), "up_proj": (688, 256), "down_proj": (256, 688)}
    for name, value in list(params.items()):
        if isinstance(value, tuple):
            flat, shape = value
            shape = shape or widths[name.split(".")[-2]]
            params[name] = flat.reshape(shape)
    return params


@pytest.mark.parametrize("variant", [0, 1])
def test_step_loss_and_adapter_gradients(golden, variant):
    g = golden(f"step_tiny_b{variant}.npz")
    params = params_of(g)
    ids = torch.from_numpy(g["input_ids"])
    batch = {"input_ids": ids, "attention_mask": torch.ones_like(ids), "segment_ids": torch.from_numpy(g["segment_ids"])}
    total, weight = oracle_model.step_loss(params, batch, **CONFIG)
    assert weight.item() == float(g["effective_weight"])
    assert abs((total / weight).item() - float(g["loss"])) / float(g["loss"]) < 1e-6
    names = [n for n, p in params.items() if p.requires_grad]
    grads = torch.autograd.grad(total, [params[n] for n in names])
    norm = torch.sqrt(sum((gr / weight).square().sum() for gr in grads)).item()
    assert abs(norm - float(g["grad_norm"])) / float(g["grad_norm"]) < 1e-4
    for name, grad in zip(names, grads):
        expected = torch.from_numpy(g["g__" + name.replace(".", "__")])
        torch.testing.assert_close(grad / weight, expected, rtol=1e-4, atol=1e-8 + 1e-5 * expected.abs().max().item())
