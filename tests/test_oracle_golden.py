"""The CPU oracle against fixtures produced by the reference's own code (tests/golden/make_golden.py)."""

import glob
import os

import numpy as np
import pytest
import torch

from oracle import nf4, ops
from conftest import GOLDEN

NF4_FILES = sorted(os.path.basename(p) for p in glob.glob(os.path.join(GOLDEN, "nf4_*.npz")))
PROJECTION_FILES = sorted(os.path.basename(p) for p in glob.glob(os.path.join(GOLDEN, "projection_*.npz")))
ROPE_FILES = sorted(os.path.basename(p) for p in glob.glob(os.path.join(GOLDEN, "rope_*.npz")))


def tensor(array, bf16=False):
    t = torch.from_numpy(np.ascontiguousarray(array))
    return t.bfloat16() if bf16 else t


def test_fixture_inventory():
    assert len(NF4_FILES) == 8 and len(PROJECTION_FILES) == 4 and len(ROPE_FILES) == 3


@pytest.mark.parametrize("name", NF4_FILES)
def test_nf4_decode_matches_reference_kernel_bit_for_bit(golden, name):
    g = golden(name)
    nested = bool(g["nested"])
    extra = dict(code2=g["code2"], absmax2=g["absmax2"], offset=g["offset"], blocksize2=int(g["blocksize2"])) if nested else {}
    out = nf4.decode(g["packed"], g["absmax"], g["code"], int(g["n"]), int(g["blocksize"]), nested=nested, **extra)
    assert out.dtype == np.float32
    assert np.array_equal(out, g["out"])


def test_nf4_levels_match_fixture_table(golden):
    assert np.array_equal(golden(NF4_FILES[0])["code"], nf4.NF4_LEVELS)


def test_nf4_encoder_agrees_with_package_quantiser():
    from causal_tuner_b200.quant import quantize_nf4
    weight = torch.randn(37, 64) * 0.02
    packed, state = quantize_nf4(weight, blocksize=64)
    expected_packed, expected_absmax = nf4.encode(weight.numpy(), 64)
    assert np.array_equal(packed.reshape(-1).numpy(), expected_packed)
    assert np.array_equal(state.absmax.numpy(), expected_absmax)
    decoded = nf4.decode(expected_packed, expected_absmax, nf4.NF4_LEVELS, weight.numel(), 64)
    # 4-bit round trip: every element lands within half the widest level gap of its block scale
    error = np.abs(decoded.reshape(37, 64) - weight.numpy())
    assert (error <= 0.16 * expected_absmax[:, None] + 1e-8).all()


@pytest.mark.parametrize("blocks,blocksize2", [(917, 256), (256, 256), (5, 64)])
def test_nested_statistics_agree_with_package_quantiser(blocks, blocksize2):
    from causal_tuner_b200.quant import quantize_nf4, scale_code
    weight = torch.randn(blocks, 64) * torch.rand(blocks, 1) * 0.05
    packed, state = quantize_nf4(weight, blocksize=64, nested=True, blocksize2=blocksize2)
    _, absmax = nf4.encode(weight.numpy(), 64)
    indices, absmax2, offset = nf4.encode_statistics(absmax, blocksize2)
    assert np.array_equal(scale_code().numpy(), nf4.scale_levels())
    assert np.array_equal(state.absmax.numpy(), indices)
    assert np.array_equal(state.state2.absmax.numpy(), absmax2)
    assert np.float32(state.offset) == offset
    # the decoded scale lands within half the widest table gap (2 / 255, doubled by the square) of the true one
    decoded = nf4.scale_levels()[indices] * np.repeat(absmax2, blocksize2)[:blocks] + offset
    assert (np.abs(decoded - absmax) <= np.repeat(absmax2, blocksize2)[:blocks] * 8e-3 + 1e-9).all()


@pytest.mark.parametrize("name", PROJECTION_FILES)
def test_projection_forward_and_backward(golden, name):
    g = golden(name)
    bf16 = bool(g["bf16"])
    dtype = torch.bfloat16 if bf16 else torch.float32
    x, w, a, b, dy = (tensor(g[k]) for k in ("x", "weight", "a", "b", "dy"))
    bias = tensor(g["bias"]) if "bias" in g else None
    y = ops.projection(x, w, a, b, bias, dtype)
    flat = lambda t: t.reshape(-1, t.shape[-1])
    dx, da, db = ops.projection_backward(flat(x), w, a, b, flat(dy), dtype)
    tolerance = dict(rtol=2e-2, atol=2e-2) if bf16 else dict(rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(y.float(), tensor(g["y"]), **(dict(rtol=0, atol=0) if not bf16 else tolerance))
    torch.testing.assert_close(dx.float().reshape(g["dx"].shape), tensor(g["dx"]), **tolerance)
    torch.testing.assert_close(da, tensor(g["da"]), **tolerance)
    torch.testing.assert_close(db, tensor(g["db"]), **tolerance)


@pytest.mark.parametrize("name", ["mlp_fp32.npz", "mlp_bf16.npz"])
def test_mlp_forward_and_autograd(golden, name):
    g = golden(name)
    bf16 = bool(g["bf16"])
    dtype = torch.bfloat16 if bf16 else torch.float32
    params = {k[2:]: tensor(v).requires_grad_(k.endswith(("lora_A", "lora_B"))) for k, v in g.items() if k.startswith("p_")}
    triple = lambda p: (params[f"{p}_weight"], params[f"{p}_lora_A"], params[f"{p}_lora_B"])
    x = tensor(g["x"]).requires_grad_(True)
    y = ops.mlp(x, triple("gate_proj"), triple("up_proj"), triple("down_proj"), dtype)
    tolerance = dict(rtol=3e-2, atol=3e-3) if bf16 else dict(rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(y.float(), tensor(g["y"]), **tolerance)
    names = [k for k in params if k.endswith(("lora_A", "lora_B"))]
    grads = torch.autograd.grad(y, (x, *(params[k] for k in names)), tensor(g["dy"]).to(y.dtype))
    torch.testing.assert_close(grads[0].float(), tensor(g["dx"]), **tolerance)
    for key, grad in zip(names, grads[1:]):
        torch.testing.assert_close(grad.float(), tensor(g["g_" + key]), **tolerance)


def test_swiglu_closed_form_matches_autograd():
    gate = torch.linspace(-30, 30, 7 * 131).reshape(7, -1).requires_grad_(True)
    up = torch.randn_like(gate).requires_grad_(True)
    signal = torch.randn_like(gate)
    expected = torch.nn.functional.silu(gate) * up
    torch.testing.assert_close(ops.swiglu(gate.detach(), up.detach()), expected.detach(), rtol=3e-6, atol=3e-6)
    eg, eu = torch.autograd.grad(expected, (gate, up), signal)
    dg, du = ops.swiglu_backward(gate.detach(), up.detach(), signal)
    torch.testing.assert_close(dg, eg, rtol=3e-5, atol=3e-6)
    torch.testing.assert_close(du, eu, rtol=3e-5, atol=3e-6)


@pytest.mark.parametrize("name", ROPE_FILES)
def test_rope_bit_exact_forward_and_inverse(golden, name):
    g = golden(name)
    bf16 = bool(g["bf16"])
    x, c, s, dy = (tensor(g[k], bf16) for k in ("x", "cosine", "sine", "dy"))
    assert torch.equal(ops.rotate(x, c, s).float(), tensor(g["y"]))
    # The gradient of a rotation is the inverse rotation of the upstream gradient.
    assert torch.equal(ops.rotate(dy, c, s, inverse=True).float(), tensor(g["dx"]))
