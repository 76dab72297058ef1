"""SwiGLU, RoPE, casts and the residual add against the CPU oracle and reference fixtures."""

import glob
import os

import numpy as np
import pytest
import torch

from causal_tuner_b200.kernels import core_cuda, linear, mlp_cuda
from oracle import ops
from conftest import GOLDEN

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("gpu_guard")]

ROPE_FILES = sorted(os.path.basename(p) for p in glob.glob(os.path.join(GOLDEN, "rope_*.npz")))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_extreme_inputs_and_tail_tiles(dtype):
    gate = torch.linspace(-30, 30, 7 * 13569, device="cuda", dtype=dtype).reshape(7, -1).requires_grad_(True)
    up = torch.randn_like(gate, requires_grad=True)
    actual = mlp_cuda.silu_multiply(gate, up)
    signal = torch.randn_like(actual.T).contiguous().T
    original_signal = signal.clone()
    expected = ops.swiglu(gate.detach().cpu(), up.detach().cpu())
    tolerance = dict(rtol=.02, atol=.002) if dtype == torch.bfloat16 else dict(rtol=3e-5, atol=3e-6)
    torch.testing.assert_close(actual.detach().cpu(), expected, **tolerance)
    gradients = torch.autograd.grad(actual, (gate, up), signal, retain_graph=True)
    oracle = ops.swiglu_backward(gate.detach().cpu(), up.detach().cpu(), signal.cpu())
    for result, reference in zip(gradients, oracle):
        torch.testing.assert_close(result.cpu(), reference, **tolerance)
    for repeat, first in zip(torch.autograd.grad(actual, (gate, up), signal), gradients):
        assert torch.equal(repeat, first)
    assert torch.equal(signal, original_signal)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activation_in_place_backward_rewrites_all_three_buffers(dtype):
    gate = torch.randn(33, 257, device="cuda", dtype=dtype)
    up, grad = torch.randn_like(gate), torch.randn_like(gate)
    saved = (gate.clone(), up.clone(), grad.clone())
    hidden_forward = mlp_cuda.activation(gate.clone(), up.clone())
    returned = mlp_cuda.activation(gate, up, grad)
    assert returned.data_ptr() == grad.data_ptr()
    assert torch.equal(grad, hidden_forward)  # the gradient buffer now holds the forward product
    dg, du = ops.swiglu_backward(*(t.cpu() for t in saved))
    tolerance = dict(rtol=.02, atol=.002) if dtype == torch.bfloat16 else dict(rtol=3e-5, atol=3e-6)
    torch.testing.assert_close(gate.cpu(), dg, **tolerance)
    torch.testing.assert_close(up.cpu(), du, **tolerance)
    # forward into a caller-provided buffer, including gate itself
    target = torch.empty_like(gate)
    assert mlp_cuda.activation(saved[0], saved[1], out=target) is target
    alias = saved[0].clone()
    mlp_cuda.activation(alias, saved[1], out=alias)
    assert torch.equal(alias, target) and torch.equal(target, hidden_forward)


@pytest.mark.parametrize("name", ROPE_FILES)
def test_rope_fixture_bit_exact(golden, name):
    g = golden(name)
    dtype = torch.bfloat16 if int(g["bf16"]) else torch.float32
    x, c, s, dy = (torch.from_numpy(g[k]).to(dtype).cuda() for k in ("x", "cosine", "sine", "dy"))
    x.requires_grad_(True)
    y = core_cuda.PartialRoPE.apply(x, c, s)
    tolerance = 0 if dtype == torch.bfloat16 else 2e-6
    torch.testing.assert_close(y.float().cpu(), torch.from_numpy(g["y"]), rtol=tolerance, atol=tolerance)
    dx, = torch.autograd.grad(y, x, dy)
    torch.testing.assert_close(dx.float().cpu(), torch.from_numpy(g["dx"]), rtol=tolerance, atol=tolerance)
    heads, head_dim = x.shape[-2], x.shape[-1]
    rotary = c.shape[-1] * 2
    assert torch.equal(y[..., rotary:], x[..., rotary:])
    # owned in-place rotation of a (query, key) pair equals the out-of-place one
    query = x.detach().reshape(14, heads * head_dim).clone()
    key = x.detach()[..., 0, :].reshape(14, head_dim).clone()
    core_cuda.rotate_owned_qk(query, key, c, s, head_dim)
    assert torch.equal(query, y.detach().reshape(14, -1))
    assert torch.equal(key, y.detach()[..., 0, :].reshape(14, head_dim))
    # inverse into a private tile leaves the source untouched
    source = dy.reshape(14, -1).clone()
    keep = source.clone()
    tile = torch.empty_like(source)
    assert core_cuda.inverse_rope_tile(source, c.reshape(14, -1), s.reshape(14, -1), head_dim, tile) is tile
    assert torch.equal(source, keep) and torch.equal(tile, dx.reshape(14, -1))


def test_rope_many_rows_and_heads_bit_exact_bf16():
    rows, heads, head_dim, rotary = 4099, 32, 128, 64
    x = torch.randn(rows, heads, head_dim, device="cuda", dtype=torch.bfloat16)
    angles = torch.randn(rows, rotary // 2, device="cuda") * 1000
    c, s = angles.cos().bfloat16(), angles.sin().bfloat16()
    expected = ops.rotate(x.cpu(), c.cpu(), s.cpu())
    assert torch.equal(core_cuda.PartialRoPE.apply(x, c, s).cpu(), expected)


@pytest.mark.parametrize("shape", [(5, 7), (256, 4096), (3, 8)])
def test_cast_and_residual_add(shape):
    source = torch.randn(*shape, device="cuda")
    assert torch.equal(linear.cast(source, torch.bfloat16), source.bfloat16())
    assert linear.cast(source, torch.float32) is source
    strided = torch.randn(shape[1], shape[0], device="cuda").T
    assert torch.equal(linear.cast(strided, torch.bfloat16), strided.bfloat16())
    for dtype in (torch.bfloat16, torch.float32):
        y, r = torch.randn(*shape, device="cuda", dtype=dtype), torch.randn(*shape, device="cuda", dtype=dtype)
        expected = y + r
        linear._add_inplace(y, r)
        assert torch.equal(y, expected)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_position_table_full_range(dtype):
    from causal_tuner_b200.kernels.core_cuda import position_values
    # ordinary packed positions and very long logical ones (argument reduction far outside [-pi, pi])
    positions = torch.cat((torch.arange(0, 4096), torch.tensor([131071, 1 << 20, 12345678, (1 << 31) + 5]))).cuda()
    positions = positions.reshape(2, -1)
    inverse = (1.0 / (1e6 ** (torch.arange(0, 64, 2, dtype=torch.float32) / 64))).cuda()
    cosine, sine = position_values(positions, inverse, dtype)
    assert cosine.shape == (*positions.shape, 32) and cosine.dtype == dtype and sine.dtype == dtype
    angle = (positions.float()[..., None] * inverse).double()      # the fp32 product, evaluated exactly
    tolerance = {torch.float32: 5e-7, torch.bfloat16: 4e-3, torch.float16: 5e-4}[dtype]
    assert (cosine.double() - angle.cos()).abs().max() <= tolerance
    assert (sine.double() - angle.sin()).abs().max() <= tolerance
    # same values as the plain tensor expression of the reference's CPU branch (modeling/rotary.py:20-24)
    plain = positions.float()[..., None] * inverse
    assert (cosine.float() - plain.cos().to(dtype).float()).abs().max() <= tolerance
    empty = position_values(positions[:, :0], inverse, dtype)
    assert empty[0].shape == (2, 0, 32)


def test_owned_rotary_beyond_512k_rows():
    # One token more than 2^19: exercises the tail after 65,536 position tiles (the reference checks the same
    # size); every token and head is compared with a bounded plain-PyTorch bf16 expression.
    rows, head_dim, rotary_dim = 524289, 128, 64
    query = torch.randn(rows, 3 * head_dim, device="cuda", dtype=torch.bfloat16)
    key = torch.randn(rows, head_dim, device="cuda", dtype=torch.bfloat16)
    original = (query.clone(), key.clone())
    angles = torch.randn(rows, rotary_dim // 2, device="cuda")
    cosine, sine = angles.cos().bfloat16(), angles.sin().bfloat16()
    core_cuda.rotate_owned_qk(query, key, cosine, sine, head_dim)
    for actual, raw in zip((query, key), original):
        for start in range(0, rows, 65536):
            source = raw[start:start + 65536].reshape(-1, raw.shape[-1] // head_dim, head_dim)
            expected = source.clone()
            c, s = cosine[start:start + 65536, None], sine[start:start + 65536, None]
            even, odd = source[..., :rotary_dim:2], source[..., 1:rotary_dim:2]
            expected[..., :rotary_dim:2] = even * c - odd * s
            expected[..., 1:rotary_dim:2] = odd * c + even * s
            assert torch.equal(actual[start:start + 65536].reshape_as(expected), expected)


def test_swiglu_and_add_index_past_two_to_the_31():
    # 2^31 + 4104 bf16 elements per buffer (4.3 GB each): element offsets no longer fit 32 bits.
    total = (1 << 31) + 4104
    gate = torch.empty(total, device="cuda", dtype=torch.bfloat16)
    up = torch.empty_like(gate)
    for buffer, seed in ((gate, 1), (up, 2)):
        generator = torch.Generator(device="cuda").manual_seed(seed)
        pattern = torch.randn(1 << 20, device="cuda", generator=generator).bfloat16()
        buffer.view(-1)[:(total // pattern.numel()) * pattern.numel()].view(-1, pattern.numel()).copy_(pattern)
        buffer[(total // pattern.numel()) * pattern.numel():] = pattern[:total % pattern.numel()]
    hidden = mlp_cuda.activation(gate.view(1, -1), up.view(1, -1)).view(-1)
    for start in (0, (1 << 31) - 2048, total - 4096):
        g, u = gate[start:start + 4096].float(), up[start:start + 4096].float()
        expected = ((g * torch.sigmoid(g)).bfloat16().float() * u).bfloat16()
        assert (hidden[start:start + 4096].float() - expected.float()).abs().max() <= 0.02 * expected.float().abs().max()
    assert bool((hidden[-8:] != 0).any())
    tail = slice(total - 4096, total)
    before = hidden[tail].clone()
    linear._add_inplace(hidden, up)
    assert torch.equal(hidden[tail], (before.float() + up[tail].float()).bfloat16())
    del gate, up, hidden
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype,width", [(torch.bfloat16, 4096), (torch.bfloat16, 8200), (torch.bfloat16, 68), (torch.float32, 96)])
def test_norm_with_shortcut_sums_both_gradients_like_autograd(dtype, width):
    rows = 37
    weight = (1 + .1 * torch.randn(width, device="cuda")).to(dtype)
    x = torch.randn(rows, width, device="cuda", dtype=dtype, requires_grad=True)
    y = x.detach().clone().requires_grad_(True)
    g_normed, g_shortcut = torch.randn_like(x), torch.randn_like(x)
    # separate: RMS(x) and x used twice, autograd adds the two gradients with its own kernel
    plain = core_cuda.RMS.apply(y, weight, 1e-6, False, False)
    expected, = torch.autograd.grad((plain, y * 1), y, (g_normed, g_shortcut))
    normed, shortcut = core_cuda.RMSWithShortcut.apply(x, weight, 1e-6)
    assert torch.equal(normed, plain) and shortcut.data_ptr() == x.data_ptr()
    keep = g_shortcut.clone()
    actual, = torch.autograd.grad((normed, shortcut * 1), x, (g_normed.clone(), g_shortcut))
    assert torch.equal(actual, expected) and torch.equal(g_shortcut, keep)
    # one branch only
    normed, shortcut = core_cuda.RMSWithShortcut.apply(x, weight, 1e-6)
    only_norm, = torch.autograd.grad(normed, x, g_normed.clone())
    assert torch.equal(only_norm, torch.autograd.grad(core_cuda.RMS.apply(y, weight, 1e-6, False, False), y, g_normed)[0])
    normed, shortcut = core_cuda.RMSWithShortcut.apply(x, weight, 1e-6)
    only_shortcut, = torch.autograd.grad(shortcut * 2, x, g_shortcut)
    assert torch.equal(only_shortcut, 2 * g_shortcut)


def test_cast_many_equals_one_cast_each():
    generator = torch.Generator().manual_seed(2)
    shapes = [(256, 4096), (5, 7), (1,), (4096,), (33, 17)] + [(16, 8)] * 40        # more than one launch carries (32)
    sources = [torch.randn(shape, generator=generator).cuda() for shape in shapes]
    sources[3] = None
    sources[6] = sources[6].bfloat16()                    # already in the target dtype: returned as it is
    before = _launches()
    results = linear.cast_many(sources, torch.bfloat16)
    assert _launches() - before == 2
    for source, result in zip(sources, results):
        if source is None:
            assert result is None
        elif source.dtype == torch.bfloat16:
            assert result is source
        else:
            assert torch.equal(result, source.bfloat16())
    # into caller-provided slices of one buffer, same dtype (a plain copy) and fp16
    stacked = torch.empty(3 * 5, 7, device="cuda")
    pieces = [torch.randn(5, 7, device="cuda") for _ in range(3)]
    linear.cast_many(pieces, torch.float32, [stacked[0:5], stacked[5:10], stacked[10:15]])
    assert torch.equal(stacked, torch.cat(pieces))
    halves = linear.cast_many(pieces, torch.float16)
    assert all(torch.equal(h, p.half()) for h, p in zip(halves, pieces))
    with pytest.raises(ValueError):
        linear.cast_many(pieces[:1], torch.float32, [stacked[0:4]])


def _launches():
    from causal_tuner_b200 import _lib
    return _lib.launch_count()
