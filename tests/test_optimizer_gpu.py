"""ct_grad_norm + ct_adamw_update (FusedAdamW.scale_clip_step) against the reference's sequence
`_foreach_div_` -> `clip_grad_norm_` -> `torch.optim.AdamW.step()` (training/engine.py:97-107) on the
same seeded tensors. fp32 throughout; the two differ only in rounding order (true division vs
reciprocal multiply, one fused expression vs separate passes), hence rtol 2e-5 on parameters and moments."""

import copy

import pytest
import torch

from causal_tuner_b200.optim import FusedAdamW

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("gpu_guard")]

# more tensors than one launch carries (40), sizes that are not multiples of 4 or of a 4096 chunk
SIZES = [(256, 512), (130, 3), (1,), (4096,), (4097,), (64, 64, 5)] + [(33, 17)] * 45


def make_parameters(sizes, seed):
    generator = torch.Generator().manual_seed(seed)
    return [torch.nn.Parameter(torch.randn(size, generator=generator).cuda()) for size in sizes]


def close(actual, expected, rtol):
    """Relative to the tensor's scale: entries near zero come from cancellation and carry the absolute
    rounding error of their operands."""
    torch.testing.assert_close(actual, expected, rtol=rtol, atol=1e-6 * float(expected.detach().abs().max()))


def groups_of(parameters, weight_decay):
    return [{"params": [p for p in parameters if p.ndim > 1], "weight_decay": weight_decay},
            {"params": [p for p in parameters if p.ndim <= 1], "weight_decay": 0.0}]


@pytest.mark.parametrize("max_norm,scale", [(1.0, 3.0), (1.0, 1e-4), (0.0, 1.0)])
def test_three_updates_match_the_reference_sequence(max_norm, scale):
    ours, theirs = make_parameters(SIZES, 1), make_parameters(SIZES, 1)
    hyper = dict(lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    fused = FusedAdamW(groups_of(ours, 0.1), **hyper)
    reference = torch.optim.AdamW(groups_of(theirs, 0.1), foreach=False, fused=True, **hyper)
    generator = torch.Generator().manual_seed(7)
    for step in range(3):
        divisor = torch.tensor(37.0 + step, device="cuda")
        for a, b in zip(ours, theirs):
            gradient = (torch.randn(a.shape, generator=generator) * scale * 37).cuda()
            a.grad, b.grad = gradient.clone(), gradient.clone()
        norm = fused.scale_clip_step(divisor, max_norm)
        torch._foreach_div_([p.grad for p in theirs], float(divisor))
        if max_norm:
            expected_norm = torch.nn.utils.clip_grad_norm_(theirs, max_norm, error_if_nonfinite=True, foreach=True)
        else:
            expected_norm = torch.sqrt(sum(p.grad.double().square().sum() for p in theirs)).float()
        reference.step()
        torch.testing.assert_close(norm[0], expected_norm, rtol=2e-6, atol=0)
        for a, b in zip(ours, theirs):
            close(a.grad, b.grad, 2e-6)   # what is left in .grad
            close(a, b, 2e-5)
            close(fused.state[a]["exp_avg"], reference.state[b]["exp_avg"], 2e-5)
            close(fused.state[a]["exp_avg_sq"], reference.state[b]["exp_avg_sq"], 2e-5)
            assert int(fused.state[a]["step"]) == step + 1


def test_norm_is_reproducible_and_gradients_can_be_left_alone():
    parameters = make_parameters(SIZES, 3)
    for p in parameters:
        p.grad = torch.randn_like(p)
    kept = [p.grad.clone() for p in parameters]
    first = FusedAdamW(parameters, lr=0.0).scale_clip_step(None, 1.0, write_grads=False).clone()
    second = FusedAdamW(parameters, lr=0.0).scale_clip_step(None, 1.0, write_grads=False)
    assert torch.equal(first, second)
    assert all(torch.equal(p.grad, g) for p, g in zip(parameters, kept))
    torch.testing.assert_close(first[1], torch.clamp(1.0 / (first[0] + 1e-6), max=1.0), rtol=1e-6, atol=0)


def test_plain_step_is_adamw():
    ours, theirs = make_parameters(SIZES[:8], 5), make_parameters(SIZES[:8], 5)
    fused = FusedAdamW(ours, lr=1e-2, weight_decay=0.01)
    reference = torch.optim.AdamW(theirs, lr=1e-2, weight_decay=0.01, foreach=True)
    for _ in range(2):
        for a, b in zip(ours, theirs):
            a.grad = torch.randn_like(a)
            b.grad = a.grad.clone()
        fused.step()
        reference.step()
    for a, b in zip(ours, theirs):
        close(a, b, 2e-5)


def test_non_finite_norm_steps_nothing():
    parameters = make_parameters(SIZES[:6], 9)
    before = [p.detach().clone() for p in parameters]
    for p in parameters:
        p.grad = torch.randn_like(p)
    parameters[2].grad[0] = float("inf")
    kept = [p.grad.clone() for p in parameters]
    optimizer = FusedAdamW(parameters, lr=1e-2)
    norm = optimizer.scale_clip_step(torch.tensor(2.0, device="cuda"), 1.0)
    assert not torch.isfinite(norm[0])
    optimizer.rollback()
    for p, b, g in zip(parameters, before, kept):
        assert torch.equal(p, b) and torch.equal(p.grad, g)
        assert int(optimizer.state[p]["step"]) == 0
        assert not optimizer.state[p]["exp_avg"].any() and not optimizer.state[p]["exp_avg_sq"].any()


def test_state_dict_round_trip_continues_the_run():
    ours, resumed = make_parameters(SIZES[:6], 11), make_parameters(SIZES[:6], 11)
    first, second = FusedAdamW(ours, lr=1e-2), FusedAdamW(resumed, lr=1e-2)
    generator = torch.Generator().manual_seed(4)
    gradients = [[torch.randn(p.shape, generator=generator).cuda() for p in ours] for _ in range(2)]
    for p, g in zip(ours, gradients[0]):
        p.grad = g.clone()
    first.scale_clip_step(None, 1.0)
    with torch.no_grad():
        for p, q in zip(ours, resumed):
            q.copy_(p)
    second.load_state_dict(copy.deepcopy(first.state_dict()))   # as read back from a checkpoint
    for p, q, g in zip(ours, resumed, gradients[1]):
        p.grad, q.grad = g.clone(), g.clone()
    first.scale_clip_step(None, 1.0)
    second.scale_clip_step(None, 1.0)
    for p, q in zip(ours, resumed):
        assert torch.equal(p, q)


def test_rejects_what_it_cannot_step():
    parameter = torch.nn.Parameter(torch.randn(8, device="cuda", dtype=torch.bfloat16))
    parameter.grad = torch.randn_like(parameter)
    with pytest.raises(TypeError):
        FusedAdamW([parameter]).scale_clip_step(None, 1.0)


def test_update_of_128m_values_matches_and_leaves_the_cache_behind():
    # 32 tensors of 4 M values: 2 GB of parameters, gradients and moments per side, far beyond the 126 MB L2.
    sizes = [(2048, 2048)] * 32
    ours = [torch.nn.Parameter(torch.randn(size, device="cuda")) for size in sizes]
    theirs = [torch.nn.Parameter(p.detach().clone()) for p in ours]
    fused = FusedAdamW(ours, lr=1e-3, weight_decay=0.01)
    reference = torch.optim.AdamW(theirs, lr=1e-3, weight_decay=0.01, foreach=False, fused=True)
    divisor = torch.tensor(16384.0, device="cuda")
    for _ in range(2):
        for a, b in zip(ours, theirs):
            a.grad = torch.randn_like(a) * 100
            b.grad = a.grad.clone()
        norm = fused.scale_clip_step(divisor, 1.0)
        torch._foreach_div_([p.grad for p in theirs], float(divisor))
        expected_norm = torch.nn.utils.clip_grad_norm_(theirs, 1.0, error_if_nonfinite=True, foreach=True)
        reference.step()
        torch.testing.assert_close(norm[0], expected_norm, rtol=2e-6, atol=0)
    for a, b in zip(ours[::8], theirs[::8]):
        close(a, b, 2e-5)
        close(fused.state[a]["exp_avg_sq"], reference.state[b]["exp_avg_sq"], 2e-5)
