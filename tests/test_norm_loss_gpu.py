"""RMSNorm (trainable weight, output-reconstruction mode, fused shortcut) and the tiled lm_head loss with a
trainable head, against plain PyTorch formulas. The cases follow what the reference's own tests pin
(tests/test_fused_core.py:28-76, tests/test_kernel_workspaces.py:109-122,162-253,282-419,
tests/test_operators.py:70-106 of the reference); tolerances are written at each comparison."""

import pytest
import torch
from torch.nn import functional as F

from causal_tuner_b200.kernels.core_cuda import RMS, RMSWithShortcut
from causal_tuner_b200.kernels.loss import active_rows, projection_loss
from causal_tuner_b200.kernels.loss_cuda import weighted_ce
from causal_tuner_b200.modeling.model import RMSNorm

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("gpu_guard")]


def torch_rms(x, weight, eps, dtype):
    """round(x * rstd) * round(w) with a straight-through rounding of w, so that autograd sees the fp32 weight."""
    rounded = weight + (weight.to(dtype).float() - weight).detach()
    normalized = (x.float() * torch.rsqrt(x.float().square().mean(-1, keepdim=True) + eps)).to(dtype)
    return (normalized.float() * rounded).to(dtype)


@pytest.mark.parametrize("dtype,weight_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.float32),
                                               (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("width", [33, 4096])
@pytest.mark.parametrize("train_input", [False, True])
def test_trainable_weight_gradient(dtype, weight_dtype, width, train_input):
    x = torch.randn(257, width, device="cuda", dtype=dtype, requires_grad=train_input)
    weight = torch.empty(width, device="cuda", dtype=weight_dtype).uniform_(.5, 1.5)
    weight[:3] = torch.tensor([0., -1., 2.], device="cuda")
    weight.requires_grad_(True)
    oracle_x = x.detach().clone().requires_grad_(train_input)
    oracle_w = weight.detach().float().requires_grad_(True)
    expected = torch_rms(oracle_x, oracle_w, 1e-6, dtype)
    actual = RMS.apply(x, weight, 1e-6, True, True)      # reuse / reconstruction are ignored for a trainable weight
    upstream = torch.randn_like(actual.T).contiguous().T
    kept = upstream.clone()
    tolerance = dict(rtol=.02, atol=.04) if dtype == torch.bfloat16 else dict(rtol=3e-5, atol=2e-5)
    torch.testing.assert_close(actual, expected, **tolerance)
    inputs, oracles = ((x, weight), (oracle_x, oracle_w)) if train_input else ((weight,), (oracle_w,))
    first = torch.autograd.grad(actual, inputs, upstream, retain_graph=True)
    for mine, reference in zip(first, torch.autograd.grad(expected, oracles, upstream)):
        assert mine.dtype in (dtype, weight_dtype)
        torch.testing.assert_close(mine, reference.to(mine.dtype), **tolerance)
    for mine, again in zip(first, torch.autograd.grad(actual, inputs, upstream)):
        assert torch.equal(mine, again)                   # fixed summation order
    assert torch.equal(upstream, kept)                    # the upstream gradient is never written


def test_trainable_weight_with_no_rows():
    weight = torch.ones(33, device="cuda", requires_grad=True)
    x = torch.empty(0, 33, device="cuda", requires_grad=True)
    dx, dw = torch.autograd.grad(RMS.apply(x, weight, 1e-6).sum(), (x, weight))
    assert dx.shape == x.shape and dw.shape == weight.shape and not dw.any()


@pytest.mark.parametrize("width", [32, 4096, 4100])
def test_reconstruction_mode_saves_the_output_and_bounds_the_gradient_error(width):
    norm = RMSNorm(width, 1e-6, torch.bfloat16, "cuda")
    norm.weight.requires_grad_(False)
    torch.nn.init.uniform_(norm.weight, .5, 1.5)
    x = torch.randn(2, 7, width, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    saved = []
    with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(t) or t, lambda t: t):
        output = norm(x, reuse_grad=True)
    assert saved[0].data_ptr() == output.data_ptr() != x.data_ptr()
    exact = norm(x)
    assert torch.equal(output, exact)
    signal = torch.randn_like(output)
    expected = torch.autograd.grad(exact, x, signal)[0].float()
    handed_over = signal.clone()
    actual = torch.autograd.grad(output, x, handed_over)[0]
    assert actual.data_ptr() == handed_over.data_ptr()    # reuse_grad: written over the private upstream gradient
    # the bounds of the reference's own test (tests/test_kernel_workspaces.py:236-253)
    assert ((actual.float() - expected).norm() / expected.norm()).item() < .003
    assert (actual.float() - expected).abs().max().item() < .05


@pytest.mark.parametrize("bad", [0., 1e-9, 1e9, float("inf"), float("nan")])
def test_reconstruction_is_refused_for_weights_outside_its_range(bad):
    norm = RMSNorm(32, 1e-6, torch.bfloat16, "cuda")
    norm.weight.requires_grad_(False)
    x = torch.randn(2, 7, 32, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    assert norm._can_reconstruct(x.dtype)
    norm.weight[0] = bad                                   # bumps the version: the cached verdict is stale
    saved = []
    with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(t) or t, lambda t: t):
        norm(x, reuse_grad=True)
    assert not norm._can_reconstruct(x.dtype)
    assert saved[0].data_ptr() == x.data_ptr()
    assert not RMSNorm(32, 1e-6, torch.float32, "cuda")._can_reconstruct(torch.float32)


@pytest.mark.parametrize("reconstruct", [False, True])
def test_fused_shortcut_equals_norm_gradient_plus_residual_gradient(reconstruct):
    torch.manual_seed(3)
    weight = torch.empty(4096, device="cuda", dtype=torch.bfloat16).uniform_(.5, 1.5)
    x = torch.randn(37, 4096, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    other = x.detach().clone().requires_grad_(True)
    normed, shortcut = RMSWithShortcut.apply(x, weight, 1e-6, reconstruct)
    plain = RMS.apply(other, weight, 1e-6, False, reconstruct)
    assert torch.equal(normed, plain) and shortcut.data_ptr() == x.data_ptr()
    g_norm, g_short = torch.randn_like(normed), torch.randn_like(normed)
    fused = torch.autograd.grad((normed, shortcut), x, (g_norm.clone(), g_short))[0]
    separate = torch.autograd.grad(plain, other, g_norm.clone())[0]
    assert torch.equal(fused, separate + g_short)          # round(round(norm gradient) + shortcut gradient)


@pytest.mark.parametrize("reuse", [False, True])
def test_gradient_ownership_with_zero_weights(reuse):
    x = torch.randn(3, 4096, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    weight = torch.randn(4096, device="cuda", dtype=torch.bfloat16)
    weight[:64] = 0
    signal = torch.randn_like(x)
    kept = signal.clone()
    expected = torch.autograd.grad(RMS.apply(x, weight, 1e-6), x, kept)[0]
    result = torch.autograd.grad(RMS.apply(x, weight, 1e-6, reuse), x, signal)[0]
    assert torch.equal(result, expected)
    assert (result.data_ptr() == signal.data_ptr()) == reuse
    assert reuse or torch.equal(signal, kept)


# ---- lm_head loss ------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("reuse", [False, True])
@pytest.mark.parametrize("layout", ["all", "interval", "gaps", "empty"])
def test_trainable_head_gradients_for_every_row_layout(dtype, reuse, layout):
    values = torch.randn(17, 32, device="cuda", dtype=dtype)
    leaf = values.clone().requires_grad_(True)
    hidden = leaf + 0 if reuse else leaf
    head = torch.randn(259, 32, device="cuda", requires_grad=True)
    weights = torch.rand(17)
    if layout == "interval":
        weights[:3] = weights[-2:] = 0
    elif layout == "gaps":
        weights[::3] = 0
    elif layout == "empty":
        weights.zero_()
    selection = active_rows(weights, "cuda")
    assert isinstance(selection, slice) == (layout != "gaps")
    targets = torch.randint(259, (17,), device="cuda")
    weights = weights.cuda()
    oracle_x, oracle_head = values.clone().requires_grad_(True), head.detach().clone().requires_grad_(True)
    logits = F.linear(oracle_x, oracle_head.to(dtype)).float()
    expected = (F.cross_entropy(logits, targets, reduction="none") * weights).sum()
    actual = projection_loss(hidden, head, targets, weights, token_budget=5, compute_dtype=dtype, reuse_hidden=reuse,
                             rows=selection)
    torch.testing.assert_close(actual, expected, rtol=2e-5, atol=2e-5)
    first = torch.autograd.grad(actual, (leaf, head), retain_graph=True)
    bound = .03 if dtype == torch.bfloat16 else 3e-5
    for mine, reference in zip(first, torch.autograd.grad(expected, (oracle_x, oracle_head))):
        torch.testing.assert_close(mine, reference, rtol=bound, atol=bound)
    assert first[1].dtype == torch.float32
    for mine, again in zip(first, torch.autograd.grad(actual, (leaf, head), retain_graph=True)):
        assert torch.equal(mine, again)
    assert torch.equal(leaf.detach(), values)
    doubled = torch.autograd.grad(actual * 2, (leaf, head))
    assert all(torch.equal(twice, once * 2) for twice, once in zip(doubled, first))


def test_head_gradient_accumulates_in_fp32_across_tiles():
    """bf16 operands, fp32 head gradient (kernels/loss_cuda.py:120-121): summing the tiles in bf16 would round
    differently (tests/test_operators.py:88-106 of the reference)."""
    hidden = torch.randn(2, 7, 8, dtype=torch.bfloat16, device="cuda", requires_grad=True)
    head = torch.randn(19, 8, device="cuda", requires_grad=True)
    targets = torch.randint(0, 19, (2, 7), device="cuda")
    weights = torch.rand(2, 7, device="cuda")
    projection_loss(hidden, head, targets, weights, token_budget=2, compute_dtype=torch.bfloat16).backward()
    x = hidden.detach().flatten(0, 1)
    derivative = F.linear(x, head.detach().bfloat16()).float().softmax(-1)
    derivative[torch.arange(len(x), device="cuda"), targets.flatten()] -= 1
    derivative = (derivative * weights.flatten()[:, None]).bfloat16()
    expected = derivative.float().T @ x.float()
    torch.testing.assert_close(head.grad, expected, rtol=1e-6, atol=1e-6)
    assert not torch.equal(head.grad, expected.bfloat16().float())


def test_unsupervised_batch_touches_neither_the_head_nor_the_logits(monkeypatch):
    hidden = torch.randn(2, 7, 32, device="cuda", requires_grad=True)
    head = torch.randn(97, 32, device="cuda", requires_grad=True)
    from causal_tuner_b200.kernels import loss_cuda

    def forbidden(*args, **kwargs):
        raise AssertionError("an unsupervised batch must not cast the head or form logits")
    monkeypatch.setattr(loss_cuda, "cast", forbidden)
    monkeypatch.setattr(loss_cuda, "matmul", forbidden)
    loss = projection_loss(hidden, head, torch.full((2, 7), -100, device="cuda"), torch.zeros(2, 7, device="cuda"))
    gradients = torch.autograd.grad(loss, (hidden, head))
    assert loss.item() == 0 and all(not g.any() for g in gradients)


def test_ignore_index_on_unweighted_rows_is_never_dereferenced():
    """Targets outside [0, vocab) - the usual -100 - on rows of weight 0 select nothing: loss 0, zero gradient row."""
    logits = torch.randn(6, 4099, device="cuda").bfloat16()
    reference = logits.clone()
    targets = torch.tensor([5, -100, 4098, 4099, 7, -1], device="cuda")
    weights = torch.tensor([1., 0., .5, 0., 2., 0.], device="cuda")
    losses = weighted_ce(logits, targets, weights, gradient=True)
    valid = weights > 0
    expected = F.cross_entropy(reference[valid].float(), targets[valid], reduction="none") * weights[valid]
    torch.testing.assert_close(losses[valid], expected, rtol=2e-6, atol=1e-5)
    assert not losses[~valid].any() and not logits[~valid].any() and torch.isfinite(logits.float()).all()
