"""project_group / _LoRAGroup on the GPU against the CPU oracle, the reference-generated fixtures
and the ownership rules the reference's own tests pin (tests/test_fast_training.py,
tests/test_kernel_workspaces.py, tests/test_recompute_and_layout.py of the reference)."""

import copy
import glob
import os

import pytest
import torch

from causal_tuner_b200 import _lib
from causal_tuner_b200.kernels import core_cuda, linear
from causal_tuner_b200.kernels.linear import project_group
from causal_tuner_b200.modeling.lora import Projection
from oracle import ops
from conftest import GOLDEN

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("gpu_guard")]

PROJECTION_FILES = sorted(os.path.basename(p) for p in glob.glob(os.path.join(GOLDEN, "projection_*.npz")))


def relative(actual, expected):
    actual, expected = actual.float(), expected.float()
    return ((actual - expected).norm() / expected.norm().clamp_min(1e-20)).item()


def oracle_projection(module, x):
    """The reference's non-fused composition (modeling/lora.py:29-39) on the module's current weights."""
    return ops.projection(x, module.base_weight().detach(), module.lora_A, module.lora_B,
                          None if module.bias is None else module.bias.detach(), module.compute_dtype)


@pytest.mark.parametrize("name", PROJECTION_FILES)
@pytest.mark.parametrize("tile", [0, 5])
def test_reference_fixture(golden, name, tile):
    g = golden(name)
    dtype = torch.bfloat16 if int(g["bf16"]) else torch.float32
    outputs, inputs = g["weight"].shape
    module = Projection(inputs, outputs, bias="bias" in g, rank=g["a"].shape[0], base_dtype=dtype, compute_dtype=dtype,
                        device="cuda")
    with torch.no_grad():
        module.weight.copy_(torch.from_numpy(g["weight"]))
        module.lora_A.copy_(torch.from_numpy(g["a"]))
        module.lora_B.copy_(torch.from_numpy(g["b"]))
        if "bias" in g:
            module.bias.copy_(torch.from_numpy(g["bias"]))
    x = torch.from_numpy(g["x"]).to(dtype).cuda().requires_grad_(True)
    y = project_group((module,), x, tile)[0]
    dx, da, db = torch.autograd.grad(y, (x, module.lora_A, module.lora_B), torch.from_numpy(g["dy"]).to(dtype).cuda())
    assert da.dtype == db.dtype == torch.float32 and y.dtype == dx.dtype == dtype
    for actual, key in ((y, "y"), (dx, "dx"), (da, "da"), (db, "db")):
        expected = torch.from_numpy(g[key])
        if dtype == torch.float32:
            torch.testing.assert_close(actual.cpu(), expected, rtol=3e-5, atol=3e-6)
        else:
            assert relative(actual.cpu(), expected) < 2e-2, key


@pytest.mark.parametrize("path", ["auto", "simt"])
def test_full_width_bf16_against_independent_autograd(path, monkeypatch):
    if path == "simt":
        monkeypatch.setattr(_lib, "gemm_path", _lib.PATH_SIMT)
    torch.manual_seed(1701)
    module = Projection(4096, 4096, rank=256, device="cuda")
    torch.nn.init.normal_(module.lora_B, std=.005)
    rows = 4099 if path == "auto" else 515
    x = torch.randn(1, rows, 4096, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    saved = x.detach().clone()
    y = x.detach().clone().requires_grad_(True)
    before = _lib.tcgen05_launch_count()
    actual = project_group((module,), x, 0)[0]
    expected = oracle_projection(module, y)
    parameters = (module.lora_A, module.lora_B)
    signal = torch.randn_like(actual)
    gradients = torch.autograd.grad(actual, (x, *parameters), signal, retain_graph=True)
    repeated = torch.autograd.grad(actual, (x, *parameters), signal)
    reference = torch.autograd.grad(expected, (y, *parameters), signal)
    for left, right in zip((actual, *gradients), (expected, *reference)):
        assert torch.isfinite(left).all()
        assert relative(left, right) < .02
    for left, right in zip(gradients, repeated):
        assert torch.equal(left, right)
    assert all(gradient.dtype == torch.float32 for gradient in gradients[1:])
    assert torch.equal(x, saved)
    assert (_lib.tcgen05_launch_count() > before) == (path == "auto")


@pytest.mark.parametrize("ranks", [(4, 4, 4), (3, 5, 7), (8, 16, 8)])
def test_shared_qkv_with_bias_and_fp32_adapter_accumulation(ranks):
    modules = [Projection(32, out, bias=True, rank=rank, compute_dtype=torch.bfloat16, device="cuda")
               for out, rank in zip((32, 8, 8), ranks)]
    for module in modules:
        torch.nn.init.normal_(module.lora_B, std=.1)
        torch.nn.init.normal_(module.bias, std=.1)
    reference = copy.deepcopy(modules)
    x = torch.randn(2, 9, 32, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = x.detach().clone().requires_grad_(True)
    outputs = project_group(modules, x, tile=4)
    targets = [oracle_projection(module, y) for module in reference]
    signals = [torch.randn_like(out) for out in outputs]
    torch.autograd.backward(outputs, signals)
    torch.autograd.backward(targets, signals)
    torch.testing.assert_close(x.grad, y.grad, rtol=.05, atol=.02)
    for index, (module, oracle) in enumerate(zip(modules, reference)):
        torch.testing.assert_close(outputs[index], targets[index], rtol=.03, atol=.02)
        dy = signals[index].flatten(0, 1)
        expected_b = dy.float().T @ (x.detach().flatten(0, 1) @ module.lora_A.detach().bfloat16().T).float()
        torch.testing.assert_close(module.lora_B.grad, expected_b, rtol=2e-5, atol=2e-5)
        torch.testing.assert_close(module.lora_A.grad, oracle.lora_A.grad, rtol=.05, atol=.02)
        assert module.weight.grad is module.bias.grad is None


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tile", [0, 5])
@pytest.mark.parametrize("head_dim,rotary_dim", [(8, 4), (128, 64)])
def test_owned_rotary_preserves_shared_gradients(dtype, tile, head_dim, rotary_dim, monkeypatch):
    width = head_dim * 4
    modules = [Projection(width, out, bias=True, rank=rank, base_dtype=dtype, compute_dtype=dtype, device="cuda")
               for out, rank in zip((width, head_dim, head_dim), (3, 5, 7))]
    for module in modules:
        torch.nn.init.normal_(module.lora_B, std=.03)
        torch.nn.init.normal_(module.bias, std=.1)
    x = torch.randn(2, 7, width, device="cuda", dtype=dtype, requires_grad=True)
    original_input = x.detach().clone()
    angles = torch.arange(14, device="cuda").reshape(2, 7, 1) * 60000 * torch.rand(rotary_dim // 2, device="cuda")
    cosine, sine = angles.cos().to(dtype), angles.sin().to(dtype)
    actual = project_group(modules, x, tile, rotary=(cosine, sine, head_dim))
    raw = project_group(modules, x, tile)
    rotate = lambda t: core_cuda.PartialRoPE.apply(t.reshape(2, 7, -1, head_dim), cosine, sine).reshape_as(t)
    expected = tuple(rotate(t) if i < 2 else t for i, t in enumerate(raw))
    tolerance = dict(rtol=0, atol=0) if dtype == torch.bfloat16 else dict(rtol=2e-6, atol=2e-6)
    for a, e in zip(actual, expected):
        torch.testing.assert_close(a, e, **tolerance)
    # and against the CPU oracle's rotation of the raw outputs
    for a, r in zip(actual[:2], raw[:2]):
        oracle = ops.rotate(r.detach().cpu().reshape(2, 7, -1, head_dim), cosine.cpu(), sine.cpu()).reshape(r.shape)
        torch.testing.assert_close(a.detach().cpu(), oracle, **tolerance)
        assert torch.equal(a.reshape(2, 7, -1, head_dim)[..., rotary_dim:], r.reshape(2, 7, -1, head_dim)[..., rotary_dim:])
    shared = torch.randn_like(actual[0])
    signals = (shared, shared[..., :head_dim], shared[..., :head_dim])
    saved_signal = shared.clone()
    parameters = (x, *(p for module in modules for p in module.parameters() if p.requires_grad))
    largest_tile = 0
    original_inverse = core_cuda.inverse_rope_tile

    def bounded_inverse(grad, *args):
        nonlocal largest_tile
        largest_tile = max(largest_tile, len(grad))
        return original_inverse(grad, *args)
    monkeypatch.setattr(core_cuda, "inverse_rope_tile", bounded_inverse)
    ag = torch.autograd.grad(actual, parameters, signals, retain_graph=True)
    eg = torch.autograd.grad(expected, parameters, signals)
    repeated = torch.autograd.grad(actual, parameters, signals)
    assert 0 < largest_tile <= (tile or 4096)
    for a, e, r in zip(ag, eg, repeated):
        torch.testing.assert_close(a, e, **tolerance)
        assert torch.equal(a, r)
    assert torch.equal(shared, saved_signal) and torch.equal(x, original_input)


@pytest.mark.parametrize("alias", [False, True])
def test_owned_residual_preserves_inputs_and_repeated_gradients(alias):
    module = Projection(32, 32, rank=4, device="cuda")
    torch.nn.init.normal_(module.lora_B, std=.1)
    x = torch.randn(2, 7, 32, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    residual = x if alias else torch.randn_like(x, requires_grad=True)
    saved_x, saved_residual = x.detach().clone(), residual.detach().clone()
    forward = lambda r: project_group((module,), x, 5, residual=r)[0]
    actual, expected = forward(residual), forward(None) + residual
    assert torch.equal(actual, expected)
    signal = torch.randn_like(actual)
    original_signal = signal.clone()
    parameters = (x, *(() if alias else (residual,)), module.lora_A, module.lora_B)
    first = torch.autograd.grad(actual, parameters, signal, retain_graph=True)
    second = torch.autograd.grad(actual, parameters, signal)
    oracle = torch.autograd.grad(expected, parameters, signal)
    for a, b, c in zip(first, second, oracle):
        assert torch.equal(a, b) and torch.equal(a, c)
    assert torch.equal(x, saved_x) and torch.equal(residual, saved_residual) and torch.equal(signal, original_signal)


def test_residual_of_other_dtype_or_shape_is_added_outside():
    module = Projection(32, 32, rank=4, device="cuda")
    x = torch.randn(2, 7, 32, device="cuda", dtype=torch.bfloat16)
    residual = torch.randn(2, 7, 32, device="cuda", dtype=torch.float32)
    out = project_group((module,), x, residual=residual)[0]
    assert out.dtype == torch.float32
    assert torch.equal(out, project_group((module,), x)[0] + residual)


def nf4_module(inputs, outputs, rank, **kwargs):
    module = Projection(inputs, outputs, rank=rank, device="cuda", **kwargs)
    module.install_nf4(module.weight.detach().clone(), "cuda")
    torch.nn.init.normal_(module.lora_B, std=.1)
    return module


def test_nf4_projection_matches_oracle_on_decoded_weights():
    module = nf4_module(64, 48, 8, bias=True)
    assert module.weight is None and module.quantized.weight.dtype == torch.uint8
    x = torch.randn(2, 13, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = x.detach().clone().requires_grad_(True)
    actual = project_group((module,), x, 5)[0]
    expected = oracle_projection(module, y)
    signal = torch.randn_like(actual)
    ag = torch.autograd.grad(actual, (x, module.lora_A, module.lora_B), signal)
    eg = torch.autograd.grad(expected, (y, module.lora_A, module.lora_B), signal)
    torch.testing.assert_close(actual, expected, rtol=.04, atol=.003)
    for a, e in zip(ag, eg):
        torch.testing.assert_close(a, e.to(a.dtype), rtol=.05, atol=.003)


def test_backward_without_input_gradient_does_not_decode_the_base(monkeypatch):
    module = nf4_module(32, 32, 4)
    x = torch.randn(2, 7, 32, device="cuda", dtype=torch.bfloat16)
    actual = project_group((module,), x, 5)[0]

    def forbidden(*args):
        raise AssertionError("Adapter-only backward must not dequantize the frozen base")
    monkeypatch.setattr(linear, "materialize", forbidden)
    actual.sum().backward()
    assert module.lora_A.grad.abs().sum() > 0 and module.lora_B.grad.abs().sum() > 0


def test_empty_input_returns_zero_parameter_gradients():
    module = Projection(32, 32, rank=4, device="cuda")
    x = torch.empty(2, 0, 32, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    output = project_group((module,), x, 5)[0]
    gradients = torch.autograd.grad(output.sum(), (x, module.lora_A, module.lora_B))
    assert gradients[0].shape == x.shape
    assert all(torch.count_nonzero(gradient) == 0 for gradient in gradients)


def test_projection_module_forward_uses_the_fused_operator():
    module = Projection(64, 32, bias=True, rank=8, device="cuda")
    torch.nn.init.normal_(module.lora_B, std=.1)
    x = torch.randn(3, 5, 64, device="cuda", dtype=torch.bfloat16)
    assert relative(module(x), oracle_projection(module, x)) < 2e-2
    module.lora_A.requires_grad_(False)
    with pytest.raises(NotImplementedError):
        module(x)


def test_config2_full_size_nf4_projection():
    """Single fused NF4+LoRA projection at M = 16384, K = 4096, N = 14336, rank 256: forward Y and
    backward dX, dA, dB within 2e-2 relative Frobenius error of a bf16 PyTorch composition on the
    same decoded weights; repeated backward bit-identical; tcgen05 kernel in use."""
    torch.manual_seed(5)
    rows, inner, outer, rank = 16384, 4096, 14336, 256
    module = Projection(inner, outer, rank=rank, device="cuda")
    module.install_nf4(module.weight.detach().clone(), "cuda", nested=False)
    torch.nn.init.normal_(module.lora_A, std=.02)
    torch.nn.init.normal_(module.lora_B, std=.01)
    x = torch.randn(rows, inner, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn(rows, outer, device="cuda", dtype=torch.bfloat16)
    before = _lib.tcgen05_launch_count()
    y = project_group((module,), x)[0]
    grads = torch.autograd.grad(y, (x, module.lora_A, module.lora_B), dy, retain_graph=True)
    again = torch.autograd.grad(y, (x, module.lora_A, module.lora_B), dy)
    assert _lib.tcgen05_launch_count() - before >= 10
    z = x.detach().clone().requires_grad_(True)
    expected = oracle_projection(module, z)
    reference = torch.autograd.grad(expected, (z, module.lora_A, module.lora_B), dy)
    for name, left, right in zip(("y", "dx", "da", "db"), (y, *grads), (expected, *reference)):
        assert torch.isfinite(left).all(), name
        assert relative(left, right) < 2e-2, name
    for left, right in zip(grads, again):
        assert torch.equal(left, right)


@pytest.mark.parametrize("ranks", [(8, 16, 8), (3, 5, 7), (256, 256, 256)])
def test_untiled_group_shares_its_low_rank_products_and_may_keep_them(ranks):
    # q/k/v on one input, all rows at once: stacked x.A^T and stacked dA. Keeping the low-rank inputs for
    # backward changes what is retained, never a value; the tiled path (separate products) agrees within
    # the accumulation-order tolerance of fp32.
    inner = 64 if ranks[0] < 256 else 512
    modules = [Projection(inner, out, bias=True, rank=rank, compute_dtype=torch.bfloat16, device="cuda")
               for out, rank in zip((inner, 16, 16), ranks)]
    for module in modules:
        torch.nn.init.normal_(module.lora_B, std=.1)
    x = torch.randn(3, 100, inner, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    parameters = [p for module in modules for p in (module.lora_A, module.lora_B)]

    def run(tile, keep):
        for module in modules:
            module.keep_low_rank = keep
        before = torch.cuda.memory_allocated()
        outputs = project_group(modules, x, tile=tile)
        retained = torch.cuda.memory_allocated() - before - sum(o.numel() * o.element_size() for o in outputs)
        signals = [torch.full_like(o, .01) * (i + 1) for i, o in enumerate(outputs)]
        first = torch.autograd.grad(outputs, (x, *parameters), signals, retain_graph=True)
        again = torch.autograd.grad(outputs, (x, *parameters), signals)
        assert all(torch.equal(a, b) for a, b in zip(first, again))
        return outputs, first, retained

    plain_out, plain_grads, plain_retained = run(0, False)
    kept_out, kept_grads, kept_retained = run(0, True)
    tiled_out, tiled_grads, _ = run(32, False)
    assert all(torch.equal(a, b) for a, b in zip(plain_out, kept_out))
    assert all(torch.equal(a, b) for a, b in zip(plain_grads, kept_grads))
    assert kept_retained - plain_retained >= 300 * sum(ranks) * 2      # the stacked [rows, sum of ranks] bf16 block
    assert all(torch.equal(a, b) for a, b in zip(plain_out, tiled_out))
    for a, b in zip(plain_grads, tiled_grads):
        assert relative(a, b) < (4e-3 if a.dtype == torch.bfloat16 else 1e-5)
    assert all(g.dtype == torch.float32 for g in plain_grads[1:])


def test_single_projection_may_keep_its_low_rank_input():
    module = Projection(256, 128, rank=16, compute_dtype=torch.bfloat16, device="cuda")
    torch.nn.init.normal_(module.lora_B, std=.1)
    x = torch.randn(70, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    residual = torch.randn(70, 128, device="cuda", dtype=torch.bfloat16)
    results = []
    for keep in (False, True):
        module.keep_low_rank = keep
        out = project_group((module,), x, residual=residual)[0]
        results.append((out, torch.autograd.grad(out, (x, module.lora_A, module.lora_B), torch.ones_like(out))))
    assert torch.equal(results[0][0], results[1][0])
    assert all(torch.equal(a, b) for a, b in zip(results[0][1], results[1][1]))
    with torch.no_grad():            # nothing is kept when no graph is recorded
        module.keep_low_rank = True
        assert torch.equal(project_group((module,), x, residual=residual)[0], results[0][0])
