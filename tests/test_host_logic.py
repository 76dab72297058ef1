"""Host-side logic of the operator layer that needs no GPU: fusion predicate, argument
guards, cache accounting, quantiser round trips and module surface."""

import inspect

import numpy as np
import pytest
import torch

from causal_tuner_b200.kernels import core_cuda, linear, mlp_cuda, nf4_cuda
from causal_tuner_b200.modeling.lora import Projection
from causal_tuner_b200.modeling.model import MLP, Runtime
from causal_tuner_b200.quant import quantize_nf4, NF4_LEVELS
from oracle import nf4 as oracle_nf4


class TinyConfig:
    hidden_size, intermediate_size = 32, 68


def test_operator_surface_matches_the_reference_signatures():
    expected = {
        linear.materialize: ["weight", "state", "dtype"],
        linear.accumulate: ["output", "left", "right", "add"],
        linear.forward_linear: ["x", "weight", "a", "b", "out", "xa", "bias", "residual"],
        linear.input_gradient: ["dy", "weight", "a", "b", "dx", "low", "add"],
        linear.input_gradient_group: ["dys", "weights", "a_list", "b_list", "dx", "lows", "add"],
        linear.parameter_gradients: ["x", "dy", "da", "db", "low", "xa", "add"],
        linear.projection_parameters: ["module"],
        linear.can_fuse: ["module", "x"],
        linear.project_group: ["modules", "x", "tile", "rotary", "residual"],
        mlp_cuda.activation: ["gate", "up", "gradient", "out"],
        mlp_cuda.silu_multiply: ["gate", "up"],
        mlp_cuda._forward_into: ["output", "x", "dtype", "tile", "states", "parameters", "residual", "save"],
        mlp_cuda.tiled_lora_mlp: ["module", "x", "residual", "tile", "cache"],
        nf4_cuda.dequantize_nf4: ["weight", "state", "dtype"],
        core_cuda.rotate_owned_qk: ["query", "key", "cosine", "sine", "head_dim"],
        core_cuda.inverse_rope_tile: ["grad", "cosine", "sine", "head_dim", "output"],
    }
    for function, names in expected.items():
        target = getattr(function, "__wrapped__", function)
        assert list(inspect.signature(target).parameters) == names, function.__name__
    assert inspect.signature(linear.accumulate).parameters["add"].default is True
    assert inspect.signature(linear.project_group).parameters["tile"].default == 0
    assert issubclass(linear._LoRAGroup, torch.autograd.Function)
    assert issubclass(mlp_cuda._TiledLoRAMLP, torch.autograd.Function)


def test_can_fuse_predicate():
    module = Projection(8, 8, bias=True, rank=2, device="cpu")

    class Cuda:
        is_cuda = True
    assert linear.can_fuse(module, Cuda())
    assert not linear.can_fuse(module, torch.zeros(1))
    module.bias.requires_grad_(True)
    assert not linear.can_fuse(module, Cuda())
    module.bias.requires_grad_(False)
    module.lora_A.requires_grad_(False)
    assert not linear.can_fuse(module, Cuda())
    assert not linear.can_fuse(Projection(8, 8, rank=0, device="cpu"), Cuda())


def test_projection_parameters_and_initialisation():
    module = Projection(64, 16, bias=True, rank=4, device="cpu")
    (weight, a, b, bias), state = linear.projection_parameters(module)
    assert state is None and weight is module.weight and bias is module.bias
    assert a.dtype == b.dtype == torch.float32 and a.shape == (4, 64) and b.shape == (16, 4)
    assert not b.any() and a.abs().max() <= (6 / 64) ** .5
    assert not weight.requires_grad and not bias.requires_grad and a.requires_grad and b.requires_grad


def test_residual_needs_a_single_projection():
    modules = [Projection(8, 8, rank=2, device="cpu") for _ in range(2)]
    with pytest.raises(ValueError, match="Residual fusion requires one output projection"):
        linear.project_group(modules, torch.zeros(1, 3, 8), residual=torch.zeros(1, 3, 8))


def test_nf4_install_is_restricted_like_the_reference():
    module = Projection(8, 8, rank=2, device="cpu")
    with pytest.raises(ValueError, match="CUDA"):
        module.install_nf4(module.weight.detach().clone(), "cpu")
    with pytest.raises(ValueError, match="frozen adapter"):
        Projection(8, 8, rank=0, device="cpu").install_nf4(torch.zeros(8, 8), "cuda")


def test_mlp_cache_bytes_counts_gate_up_and_their_low_rank_inputs():
    module = MLP(TinyConfig, Runtime(rank=4, mlp_tile=5), "cpu")
    assert module.cache_bytes(14) == 14 * 2 * (2 * 68 + 2 * 4)
    assert module.tile == 5 and module.cache_intermediates is False


@pytest.mark.parametrize("shape,blocksize,nested", [((71, 96), 64, False), ((71, 96), 128, True), ((17, 19), 64, True),
                                                    ((5, 4096), 4096, False)])
def test_quantiser_layout_round_trips_through_the_oracle_decode(shape, blocksize, nested):
    weight = torch.randn(*shape) * 0.02
    packed, state = quantize_nf4(weight, blocksize=blocksize, nested=nested)
    n = weight.numel()
    assert packed.shape == ((n + 1) // 2, 1) and packed.dtype == torch.uint8
    assert state.shape == weight.shape and state.quant_type == "nf4" and state.blocksize == blocksize
    assert tuple(state.code.tolist()) == tuple(np.float32(v) for v in NF4_LEVELS)
    extra = {}
    if nested:
        assert state.absmax.dtype == torch.uint8
        extra = dict(nested=True, code2=state.state2.code.numpy(), absmax2=state.state2.absmax.numpy(),
                     offset=float(state.offset), blocksize2=state.state2.blocksize)
    decoded = oracle_nf4.decode(packed.numpy(), state.absmax.numpy(), state.code.numpy(), n, blocksize, **extra)
    error = np.abs(decoded - weight.reshape(-1).numpy())
    blocks = np.repeat(np.abs(weight.reshape(-1).numpy().reshape(-1)), 1)
    # within 17 % of the block's absmax (4-bit levels) plus the 8-bit error of nested statistics
    limit = 0.17 * weight.abs().max().item() * (1.1 if nested else 1.0)
    assert error.max() <= limit


def test_default_parameter_counts_match_the_reference_numbers():
    from causal_tuner_b200.modeling.config import ModelConfig
    assert ModelConfig().parameter_counts(256) == (9574004736, 796917760)
    seven_b = ModelConfig(hidden_size=4096, intermediate_size=14336, vocab_size=49152, num_hidden_layers=32)
    assert seven_b.parameter_counts(256)[1] == 656408576      # fp32 all-reduce payload of the 7B step: 2.63 GB
    with pytest.raises(ValueError):
        ModelConfig(num_key_value_heads=2)


def test_segments_positions_and_targets_never_cross_documents():
    from causal_tuner_b200 import segments as seg
    from oracle import model as oracle_model
    labels = torch.tensor([[1, 1, 1, 2, 2, 2, 2, 3, 3], [5, 5, 0, 0, 7, 7, 7, 7, 7]])
    mask = torch.tensor([[1] * 9, [1, 1, 0, 0, 1, 1, 1, 1, 1]])
    canonical = seg.canonical_segments(mask, labels)
    assert canonical.tolist() == [[1, 1, 1, 2, 2, 2, 2, 3, 3], [1, 1, 0, 0, 2, 2, 2, 2, 2]]
    assert torch.equal(canonical, oracle_model.segments_of(mask, labels))
    positions = seg.position_ids(canonical)
    assert positions.tolist() == [[0, 1, 2, 0, 1, 2, 3, 0, 1], [0, 1, 0, 0, 0, 1, 2, 3, 4]]
    assert torch.equal(positions, oracle_model.positions_of(canonical))
    assert seg.runs(canonical) == ((0, 0, 3), (0, 3, 7), (0, 7, 9), (1, 0, 2), (1, 4, 9))
    ids = torch.arange(18).reshape(2, 9)
    targets, weights = seg.prediction_targets({"input_ids": ids, "attention_mask": mask, "segment_ids": labels})
    assert weights.tolist() == [[1, 1, 0, 1, 1, 1, 0, 1, 0], [1, 0, 0, 0, 1, 1, 1, 1, 0]]
    assert targets[0, :2].tolist() == [1, 2] and targets[weights == 0].eq(0).all()


def test_segment_helpers_equal_the_installed_reference_on_random_packs():
    """Randomised packs (gaps, repeated raw labels, label 0, explicit weights, -100 targets) through the
    reference's own data/segments.py, installed in oracle/_ref, and through this package's functions."""
    from oracle import ref_bridge
    if not ref_bridge.available():
        pytest.skip("oracle/_ref is not installed")
    ref_bridge.load()
    from causal_tuner.data import segments as theirs
    from causal_tuner_b200 import segments as ours
    generator = torch.Generator().manual_seed(99)
    for trial in range(40):
        rows, width = int(torch.randint(1, 5, (), generator=generator)), int(torch.randint(1, 40, (), generator=generator))
        mask = (torch.rand(rows, width, generator=generator) > .2).long()
        labels = torch.randint(0, 3, (rows, width), generator=generator).sort(dim=1).values if trial % 2 else \
            torch.randint(0, 3, (rows, width), generator=generator)
        a, b = ours.canonical_segments(mask, labels), theirs.canonical_segments(mask, labels)
        assert a.dtype == b.dtype and torch.equal(a, b)
        assert torch.equal(ours.canonical_segments(mask), theirs.canonical_segments(mask))
        assert torch.equal(ours.position_ids(a), theirs.position_ids(b))
        assert ours.runs(a) == theirs.runs(b)
        ids = torch.randint(0, 50, (rows, width), generator=generator)
        batch = {"input_ids": ids, "attention_mask": mask, "segment_ids": labels}
        if trial % 3 == 0:
            batch["loss_weights"] = torch.rand(rows, width, generator=generator)
        if trial % 3 == 1:
            batch["assistant_masks"] = (torch.rand(rows, width, generator=generator) > .5).long()
        if trial % 4 == 0:
            batch["labels"] = torch.where(torch.rand(rows, width, generator=generator) > .8, -100, ids)
        if trial % 7 == 0:
            batch["prediction_targets"] = torch.randint(0, 50, (rows, width), generator=generator)
            batch["prediction_weights"] = torch.rand(rows, width, generator=generator)
        for mine, reference_value in zip(ours.prediction_targets(batch), theirs.prediction_targets(batch)):
            assert mine.dtype == reference_value.dtype and torch.equal(mine, reference_value)
    assert ours.runs(torch.zeros(2, 0, dtype=torch.int32)) == () and ours.runs(torch.zeros(2, 5, dtype=torch.int32)) == ()
    with pytest.raises(ValueError):
        ours.canonical_segments(torch.ones(3))
    with pytest.raises(ValueError):
        ours.canonical_segments(torch.ones(2, 3), torch.ones(2, 4))


def test_attention_layout_classification_equals_the_installed_reference():
    from oracle import ref_bridge
    if not ref_bridge.available():
        pytest.skip("oracle/_ref is not installed")
    ref_bridge.load()
    from causal_tuner.kernels.attention import prepare_dense_layout as theirs
    from causal_tuner_b200.kernels.attention import prepare_dense_layout as ours
    from causal_tuner_b200 import segments as seg
    generator = torch.Generator().manual_seed(5)
    seen = set()
    for trial in range(60):
        rows, width = int(torch.randint(1, 4, (), generator=generator)), int(torch.randint(1, 24, (), generator=generator))
        kind = trial % 4
        mask = torch.ones(rows, width, dtype=torch.long) if kind < 2 else (torch.rand(rows, width, generator=generator) > .3).long()
        labels = torch.zeros(rows, width, dtype=torch.long) if kind == 0 else \
            torch.randint(0, 3, (rows, width), generator=generator).sort(dim=1).values
        if kind == 3 and trial % 8 == 3:
            mask.zero_()
        spans = seg.runs(seg.canonical_segments(mask, labels))
        a, b = ours((rows, width), spans, "cpu"), theirs((rows, width), spans, "cpu")
        assert (a.spans, a.mode, a.maximum) == (b.spans, b.mode, b.maximum)
        assert (a.offsets is None) == (b.offsets is None) and (a.offsets is None or torch.equal(a.offsets, b.offsets))
        seen.add(a.mode)
    assert seen == {"empty", "full", "packed", "gaps"}
    with pytest.raises(NotImplementedError):
        ours((1, 2), ((0, 0, 2),), "cpu", torch.zeros(1, 2))


def test_active_rows_prefers_slices():
    from causal_tuner_b200.kernels.loss import active_rows, row_count
    assert active_rows(torch.tensor([0., 1, 2, 0])) == slice(1, 3)
    assert active_rows(torch.ones(4)) == slice(0, 4) and active_rows(torch.zeros(4)) == slice(0, 0)
    gaps = active_rows(torch.tensor([1., 0, 1, 1]))
    assert gaps.tolist() == [0, 2, 3] and row_count(gaps) == 3 and row_count(slice(2, 7)) == 5


def test_trainer_and_loss_surface():
    from causal_tuner_b200.kernels import loss, loss_cuda
    from causal_tuner_b200.training import Trainer, make_optimizer
    assert list(inspect.signature(loss.projection_loss).parameters) == [
        "hidden", "head", "targets", "weights", "token_budget", "compute_dtype", "implementation", "cut_chunk_size",
        "reuse_hidden", "rows"]
    assert list(inspect.signature(loss_cuda.weighted_ce).parameters) == ["logits", "targets", "weights", "gradient",
                                                                         "loss", "partials"]
    with pytest.raises(RuntimeError, match="no CPU path"):
        loss.projection_loss(torch.zeros(2, 4), torch.zeros(3, 4), torch.zeros(2, dtype=torch.long), torch.ones(2))
    with pytest.raises(ValueError):
        loss.projection_loss(torch.zeros(2, 4), torch.zeros(3, 4), torch.zeros(2), torch.ones(2), token_budget=0)
