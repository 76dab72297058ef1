"""One whole optimizer step of the tiny decoder on the GPU against the fixture the reference produced on
CPU (tests/golden/make_golden_step.py): loss, gradient norm, every adapter gradient and every updated
adapter. Plus RMSNorm and the tiled lm_head loss against plain PyTorch formulas."""

import numpy as np
import pytest
import torch
from torch.nn import functional as F

from causal_tuner_b200.kernels.core_cuda import RMS
from causal_tuner_b200.kernels.loss import active_rows, projection_loss
from causal_tuner_b200.kernels.loss_cuda import weighted_ce
from causal_tuner_b200.kernels.nf4_cuda import dequantize_nf4
from causal_tuner_b200.modeling.config import ModelConfig
from causal_tuner_b200.modeling.model import CausalLM, Runtime
from causal_tuner_b200.quant import QuantState, nf4_code
from causal_tuner_b200.training import Trainer, make_optimizer

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("gpu_guard")]

CONFIG = dict(hidden_size=256, intermediate_size=688, vocab_size=1024, num_hidden_layers=2, num_attention_heads=4,
              head_dim=64, rope_theta=1e4, rms_norm_eps=1e-5, pad_token_id=0, eos_token_id=1)


def load_model(g, runtime, nf4):
    model = CausalLM(ModelConfig(**CONFIG), runtime, "cuda")
    packed_projections = []
    with torch.no_grad():
        for name, parameter in model.named_parameters():
            key = name.replace(".", "__")
            if "a__" + key in g:
                parameter.copy_(torch.from_numpy(g["a__" + key]))
            elif "b__" + key in g:
                parameter.copy_(torch.from_numpy(g["b__" + key]))
            elif "v__" + key in g:
                parameter.copy_(torch.from_numpy(g["v__" + key]))
            else:   # frozen matrix stored as NF4 codes: decode with the CUDA kernel
                state = QuantState(shape=parameter.shape, dtype=torch.float32, blocksize=64,
                                   absmax=torch.from_numpy(g["s__" + key]).cuda(), code=nf4_code("cuda"))
                packed = torch.from_numpy(g["q__" + key]).cuda()
                parameter.copy_(dequantize_nf4(packed, state, torch.float32))
    if nf4:
        model.install_nf4(blocksize=64, nested=False)   # re-packing decoded NF4 values is lossless
    return model


def batch_of(g):
    ids = torch.from_numpy(g["input_ids"])
    return {"input_ids": ids, "attention_mask": torch.ones_like(ids), "segment_ids": torch.from_numpy(g["segment_ids"])}


@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("checkpoint", [False, True])
def test_fp32_step_matches_the_reference_fixture(golden, variant, checkpoint):
    g = golden(f"step_tiny_b{variant}.npz")
    runtime = Runtime(rank=16, base_dtype=torch.float32, train_dtype=torch.float32, compute_dtype=torch.float32,
                      attention="vanilla", checkpoint=checkpoint)
    model = load_model(g, runtime, nf4=False)
    optimizer = make_optimizer(model, learning_rate=1e-4)
    metrics = Trainer(model, optimizer, device="cuda", loss_token_budget=128).update([batch_of(g)])
    assert abs(metrics["loss"] - float(g["loss"])) / float(g["loss"]) < 1e-5
    assert abs(metrics["grad_norm"] - float(g["grad_norm"])) / float(g["grad_norm"]) < 1e-3
    assert metrics["effective_weight"] == float(g["effective_weight"]) and metrics["valid_tokens"] == int(g["valid_tokens"])
    for name, parameter in model.named_parameters():
        if parameter.requires_grad:
            key = name.replace(".", "__")
            expected_grad, expected_value = torch.from_numpy(g["g__" + key]), torch.from_numpy(g["u__" + key])
            scale = expected_grad.abs().max().item()
            torch.testing.assert_close(parameter.grad.cpu(), expected_grad, rtol=2e-3, atol=2e-4 * scale + 1e-9, msg=name)
            # AdamW's first step moves every element by ~lr * sign(grad): compare the values themselves
            torch.testing.assert_close(parameter.detach().cpu(), expected_value, rtol=0, atol=2.5e-5, msg=name)


def test_bf16_nf4_flash_step_tracks_the_bf16_reference_fixture(golden):
    """Same step in the production arithmetic (NF4 base decoded to bf16, bf16 compute, FlashAttention-2, layer
    checkpointing) against the fixture the reference produced with ITS bf16 arithmetic on the CPU
    (make_golden_step.py --dtype bfloat16): loss within 1e-3 relative - the bound stated for per-step losses -
    and gradients within 5e-2 relative Frobenius error over all adapters (every layer's bf16 rounding adds up)."""
    pytest.importorskip("flash_attn")
    g = golden("step_tiny_bf16.npz")
    runtime = Runtime(rank=16, base_dtype=torch.float32, compute_dtype=torch.bfloat16, checkpoint=True)
    model = load_model(g, runtime, nf4=True)       # fp32 NF4 values re-pack without loss; decode rounds to bf16 once
    optimizer = make_optimizer(model, learning_rate=1e-4)
    metrics = Trainer(model, optimizer, device="cuda").update([batch_of(g)])
    assert abs(metrics["loss"] - float(g["loss"])) / float(g["loss"]) < 1e-3
    assert abs(metrics["grad_norm"] - float(g["grad_norm"])) / float(g["grad_norm"]) < 2e-2
    actual = torch.cat([p.grad.flatten().cpu() for n, p in model.named_parameters() if p.requires_grad])
    expected = torch.cat([torch.from_numpy(g["g__" + n.replace(".", "__")]).flatten()
                          for n, p in model.named_parameters() if p.requires_grad])
    assert ((actual - expected).norm() / expected.norm()).item() < 5e-2
    assert all(p.grad.dtype == torch.float32 for p in model.adapter_parameters())


@pytest.mark.parametrize("policy", ["reference", "kept"])
def test_updates_are_reproducible_and_independent_of_what_is_kept(golden, policy, monkeypatch):
    """Three updates in the production configuration, run twice from the same state: bit-identical
    losses and adapters (fixed summation orders, side-stream decodes ordered by events). Keeping MLP
    activations and low-rank inputs, or decoding in stream order, changes memory and time, never a value."""
    pytest.importorskip("flash_attn")
    g = golden("step_tiny_b1.npz")

    def run(keep, ahead="1"):
        monkeypatch.setenv("CT_B200_DECODE_AHEAD", ahead)
        runtime = Runtime(rank=16, base_dtype=torch.bfloat16, compute_dtype=torch.bfloat16, checkpoint=False,
                          keep_low_rank=keep, mlp_cache_budget_bytes=(1 << 30) if keep else None)
        model = load_model(g, runtime, nf4=True)
        with torch.no_grad():
            for name, parameter in model.named_parameters():
                if name.endswith("lora_B"):
                    parameter.copy_(torch.linspace(-.02, .02, parameter.numel(), device="cuda").view_as(parameter))
        trainer = Trainer(model, make_optimizer(model, learning_rate=1e-3), device="cuda")
        losses = [trainer.update([batch_of(g)])["loss"] for _ in range(3)]
        return losses, [p.detach().clone() for p in model.adapter_parameters()]

    keep = policy == "kept"
    first, again, in_order = run(keep), run(keep), run(keep, ahead="0")
    other = run(not keep)
    for losses, adapters in (again, in_order, other):
        assert losses == first[0]
        assert all(torch.equal(a, b) for a, b in zip(adapters, first[1]))
    assert first[0][2] < first[0][0]


def test_two_microbatches_equal_one_concatenated_batch(golden):
    g = golden("step_tiny_b1.npz")
    runtime = Runtime(rank=16, base_dtype=torch.float32, train_dtype=torch.float32, compute_dtype=torch.float32,
                      attention="vanilla", checkpoint=False)
    whole, split = load_model(g, runtime, nf4=False), load_model(g, runtime, nf4=False)
    batch = batch_of(g)
    halves = [{k: v[i:i + 1] for k, v in batch.items()} for i in range(2)]
    a = Trainer(whole, make_optimizer(whole, learning_rate=1e-4), device="cuda").update([batch])
    b = Trainer(split, make_optimizer(split, learning_rate=1e-4), device="cuda").update(halves)
    assert abs(a["loss"] - b["loss"]) / a["loss"] < 1e-6 and b["microbatches"] == 2
    for p, q in zip(whole.adapter_parameters(), split.adapter_parameters()):
        torch.testing.assert_close(p.grad, q.grad, rtol=2e-4, atol=1e-7)


@pytest.mark.parametrize("dtype,weight_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                               (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("width", [32, 33, 4096])
@pytest.mark.parametrize("reuse", [False, True])
def test_rmsnorm_forward_and_input_gradient(dtype, weight_dtype, width, reuse):
    x = torch.randn(2, 17, width, device="cuda", dtype=dtype, requires_grad=True)
    reference = x.detach().clone().requires_grad_(True)
    weight = (torch.rand(width, device="cuda") + .5).to(weight_dtype)
    weight[:2] = torch.tensor([0., -1.], device="cuda").to(weight_dtype)
    normalized = (reference.float() * torch.rsqrt(reference.float().square().mean(-1, keepdim=True) + 1e-6)).to(dtype)
    expected = normalized * weight.to(dtype)
    actual = RMS.apply(x, weight, 1e-6, reuse)
    tolerance = dict(rtol=.02, atol=.02) if dtype == torch.bfloat16 else dict(rtol=3e-5, atol=3e-6)
    torch.testing.assert_close(actual, expected, **tolerance)
    signal = torch.randn_like(x)
    original = signal.clone()
    result = torch.autograd.grad(actual, x, signal)[0]
    oracle = torch.autograd.grad(expected, reference, original)[0]
    torch.testing.assert_close(result, oracle, **(dict(rtol=.03, atol=.03) if dtype == torch.bfloat16 else tolerance))
    assert (result.data_ptr() == signal.data_ptr()) == reuse
    if not reuse:
        assert torch.equal(signal, original)


@pytest.mark.parametrize("vocab", [97, 4096, 4097, 49152])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_weighted_ce_targets_at_boundaries_and_in_place_gradient(vocab, dtype):
    logits = (torch.randn(5, vocab, device="cuda") * 4).to(dtype)
    targets = torch.tensor([0, min(4095, vocab - 1), min(4096, vocab - 1), vocab // 2, vocab - 1], device="cuda")
    weights = torch.tensor([0, .125, 1, 2, .5], device="cuda")
    reference = logits.float().requires_grad_(True)
    loss = (F.cross_entropy(reference, targets, reduction="none") * weights).sum()
    expected_grad, = torch.autograd.grad(loss, reference)
    for gradient in (False, True):
        workspace = logits.clone()
        actual = weighted_ce(workspace, targets, weights, gradient=gradient).sum()
        torch.testing.assert_close(actual, loss, rtol=2e-6, atol=1e-5)
        if gradient:
            tolerance = .008 if dtype == torch.bfloat16 else 2e-6
            torch.testing.assert_close(workspace, expected_grad.to(dtype), rtol=tolerance, atol=1e-7)
        else:
            assert torch.equal(workspace, logits)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout", ["all", "interval", "gaps", "empty"])
@pytest.mark.parametrize("reuse", [False, True])
def test_projection_loss_against_full_logits(dtype, layout, reuse):
    values = torch.randn(17, 64, device="cuda", dtype=dtype)
    leaf = values.clone().requires_grad_(True)
    hidden = leaf + 0 if reuse else leaf
    head = torch.randn(259, 64, device="cuda", dtype=torch.float32)
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
    oracle_input = values.clone().requires_grad_(True)
    logits = F.linear(oracle_input, head.to(dtype)).float()
    expected = (F.cross_entropy(logits, targets, reduction="none") * weights).sum()
    actual = projection_loss(hidden, head, targets, weights, token_budget=5, compute_dtype=dtype, reuse_hidden=reuse,
                             rows=selection)
    torch.testing.assert_close(actual, expected, rtol=2e-5 if dtype == torch.float32 else 2e-3, atol=2e-5)
    gradient, = torch.autograd.grad(actual, leaf, retain_graph=True)
    oracle, = torch.autograd.grad(expected, oracle_input)
    tolerance = .03 if dtype == torch.bfloat16 else 3e-5
    torch.testing.assert_close(gradient, oracle, rtol=tolerance, atol=tolerance)
    again, = torch.autograd.grad(actual * 2, leaf)
    assert torch.equal(again, gradient * 2)
    assert torch.equal(leaf, values)
