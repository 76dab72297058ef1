"""tiled_lora_mlp / _TiledLoRAMLP on the GPU: recompute-in-backward against stored activations,
against the CPU oracle and the reference-generated fixtures, plus the checkpoint and ownership
rules the reference's tests pin (tests/test_mlp_cache.py, tests/test_recompute_and_layout.py,
tests/test_fast_training.py of the reference)."""

import copy

import pytest
import torch
from torch.utils.checkpoint import checkpoint, set_checkpoint_early_stop

from causal_tuner_b200 import _lib
from causal_tuner_b200.kernels import mlp_cuda
from causal_tuner_b200.modeling.lora import Projection
from causal_tuner_b200.modeling.model import MLP, Runtime
from oracle import ops

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("gpu_guard")]


class TinyConfig:
    hidden_size, intermediate_size = 32, 68


class WideConfig:
    hidden_size, intermediate_size = 4096, 14336


def relative(actual, expected):
    actual, expected = actual.float(), expected.float()
    return ((actual - expected).norm() / expected.norm().clamp_min(1e-20)).item()


def randomise_b(module, std):
    for name, parameter in module.named_parameters():
        if "lora_B" in name:
            torch.nn.init.normal_(parameter, std=std)


def trainable(module):
    return tuple(p for p in module.parameters() if p.requires_grad)


def oracle_mlp(module, x):
    triple = lambda p: (p.base_weight().detach(), p.lora_A, p.lora_B)
    return ops.mlp(x, triple(module.gate_proj), triple(module.up_proj), triple(module.down_proj),
                   module.gate_proj.compute_dtype)


@pytest.mark.parametrize("name", ["mlp_fp32.npz", "mlp_bf16.npz"])
@pytest.mark.parametrize("cache", [False, True])
def test_reference_fixture(golden, name, cache):
    g = golden(name)
    dtype = torch.bfloat16 if int(g["bf16"]) else torch.float32
    module = MLP(TinyConfig, Runtime(rank=4, base_dtype=dtype, compute_dtype=dtype, mlp_tile=5), "cuda")
    with torch.no_grad():
        for key, parameter in module.named_parameters():
            parameter.copy_(torch.from_numpy(g["p_" + key.replace(".", "_")]))
    x = torch.from_numpy(g["x"]).to(dtype).cuda().requires_grad_(True)
    y = module(x, cache=cache)
    names = [k for k, p in module.named_parameters() if p.requires_grad]
    grads = torch.autograd.grad(y, (x, *trainable(module)), torch.from_numpy(g["dy"]).to(dtype).cuda())
    tolerance = dict(rtol=.04, atol=.004) if dtype == torch.bfloat16 else dict(rtol=3e-5, atol=3e-6)
    torch.testing.assert_close(y.float().cpu(), torch.from_numpy(g["y"]), **tolerance)
    torch.testing.assert_close(grads[0].float().cpu(), torch.from_numpy(g["dx"]), **tolerance)
    for key, grad in zip(names, grads[1:]):
        assert grad.dtype == torch.float32
        torch.testing.assert_close(grad.cpu(), torch.from_numpy(g["g_" + key.replace(".", "_")]), **tolerance)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("train_input", [False, True])
@pytest.mark.parametrize("mixed_ranks", [False, True])
@pytest.mark.parametrize("cache", [False, True])
def test_independent_gradients(dtype, train_input, mixed_ranks, cache):
    module = MLP(TinyConfig, Runtime(rank=4, base_dtype=dtype, compute_dtype=dtype, mlp_tile=5), "cuda")
    module.cache_intermediates = cache
    if mixed_ranks:
        for name, rank in (("gate_proj", 3), ("up_proj", 5), ("down_proj", 7)):
            original = getattr(module, name)
            setattr(module, name, Projection(original.weight.shape[1], original.weight.shape[0], rank=rank,
                                             base_dtype=dtype, compute_dtype=dtype, device="cuda"))
    randomise_b(module, .1)
    reference = copy.deepcopy(module)
    x = torch.randn(2, 7, 32, device="cuda", dtype=dtype, requires_grad=train_input)
    y = x.detach().clone().requires_grad_(train_input)
    actual = module(x)
    expected = oracle_mlp(reference, y)
    tolerance = dict(rtol=.04, atol=.003) if dtype == torch.bfloat16 else dict(rtol=3e-5, atol=2e-6)
    torch.testing.assert_close(actual, expected, **tolerance)
    signal = torch.randn_like(actual)
    actual.backward(signal)
    expected.backward(signal)
    if train_input:
        torch.testing.assert_close(x.grad, y.grad, **tolerance)
    for (name, a), (_, b) in zip(module.named_parameters(), reference.named_parameters()):
        if a.requires_grad:
            assert a.grad.dtype == torch.float32, name
            torch.testing.assert_close(a.grad, b.grad, **tolerance)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tile", [0, 5])
def test_cached_matches_recompute_and_survives_repeated_backward(monkeypatch, dtype, tile):
    module = MLP(TinyConfig, Runtime(rank=4, base_dtype=dtype, compute_dtype=dtype, mlp_tile=tile), "cuda")
    randomise_b(module, .05)
    x = torch.randn(2, 7, 32, device="cuda", dtype=dtype, requires_grad=True)
    original = x.detach().clone()
    signal = torch.randn_like(x)
    params = (x, *trainable(module))
    expected = module(x, residual=x)
    reference = torch.autograd.grad(expected, params, signal)
    module.cache_intermediates = True
    saved = []
    with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(t) or t, lambda t: t):
        actual = module(x, residual=x)
    allowed = {x.data_ptr(), *(p.data_ptr() for p in module.parameters())}
    retained = [t for t in saved if t.data_ptr() not in allowed]
    assert sum(t.numel() * t.element_size() for t in retained) == module.cache_bytes(14)
    snapshots = [t.clone() for t in retained]

    def forbidden(*a, **kw):
        raise AssertionError("Cached backward must not recompute gate/up projections")
    monkeypatch.setattr(mlp_cuda, "forward_linear", forbidden)
    gradients = torch.autograd.grad(actual, params, signal, retain_graph=True)
    repeated = torch.autograd.grad(actual, params, signal)
    assert torch.equal(actual, expected)
    for value, expected_grad, repeat in zip(gradients, reference, repeated):
        assert torch.equal(value, expected_grad) and torch.equal(value, repeat)
    assert all(g.dtype == torch.float32 for g in gradients[1:])
    for value, snapshot in zip(retained, snapshots):
        assert torch.equal(value, snapshot)
    assert torch.equal(x, original)


def test_saves_only_boundary_and_weights(monkeypatch):
    module = MLP(TinyConfig, Runtime(rank=4, mlp_tile=5), "cuda")
    x = torch.randn(2, 13, 32, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    saved = []
    with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(t) or t, lambda t: t):
        output = module(x)
    allowed = {x.data_ptr(), *(parameter.data_ptr() for parameter in module.parameters())}
    assert all(tensor.data_ptr() in allowed for tensor in saved)

    def forbidden(*args, **kwargs):
        raise AssertionError("The fused MLP backward must not build per-tile autograd graphs")
    monkeypatch.setattr(torch.autograd, "grad", forbidden)
    output.sum().backward()


@pytest.mark.parametrize("downstream,early_stop,expected_calls", [(False, True, 1), (True, True, 2), (False, False, 2)])
def test_checkpoint_skips_only_unneeded_forward(monkeypatch, downstream, early_stop, expected_calls):
    module = MLP(TinyConfig, Runtime(rank=4, mlp_tile=5), "cuda")
    randomise_b(module, .1)
    reference = copy.deepcopy(module)
    x = torch.randn(2, 7, 32, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = x.detach().clone().requires_grad_(True)
    calls = 0
    original = mlp_cuda._forward_into

    def counted(*args):
        nonlocal calls
        calls += 1
        return original(*args)
    monkeypatch.setattr(mlp_cuda, "_forward_into", counted)

    def function(value):
        output = module(value, residual=value)
        return output.sin() if downstream else output
    with set_checkpoint_early_stop(early_stop):
        actual = checkpoint(function, x, use_reentrant=False, preserve_rng_state=False)
    signal = torch.randn_like(actual)
    actual.backward(signal)
    assert calls == expected_calls
    expected = reference(y) + y
    if downstream:
        expected = expected.sin()
    expected.backward(signal)
    assert torch.equal(actual, expected) and torch.equal(x.grad, y.grad)
    for left, right in zip(module.parameters(), reference.parameters()):
        if left.requires_grad:
            assert torch.equal(left.grad, right.grad)


@pytest.mark.parametrize("alias", [False, True])
def test_owned_residual(alias):
    module = MLP(TinyConfig, Runtime(rank=4, mlp_tile=5), "cuda")
    randomise_b(module, .1)
    x = torch.randn(2, 7, 32, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    residual = x if alias else torch.randn_like(x, requires_grad=True)
    saved_x, saved_residual = x.detach().clone(), residual.detach().clone()
    actual, expected = module(x, residual=residual), module(x) + residual
    assert torch.equal(actual, expected)
    signal = torch.randn_like(actual)
    original_signal = signal.clone()
    parameters = (x, *(() if alias else (residual,)), *trainable(module))
    first = torch.autograd.grad(actual, parameters, signal, retain_graph=True)
    second = torch.autograd.grad(actual, parameters, signal)
    oracle = torch.autograd.grad(expected, parameters, signal)
    for a, b, c in zip(first, second, oracle):
        assert torch.equal(a, b) and torch.equal(a, c)
    assert torch.equal(x, saved_x) and torch.equal(residual, saved_residual) and torch.equal(signal, original_signal)


def test_nf4_mlp_gradients():
    module = MLP(TinyConfig, Runtime(rank=4, mlp_tile=5), "cuda")
    for projection in (module.gate_proj, module.up_proj, module.down_proj):
        projection.install_nf4(projection.weight.detach().clone(), "cuda")
        torch.nn.init.normal_(projection.lora_B, std=.1)
    x = torch.randn(1, 13, 32, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    actual = module(x)
    expected = oracle_mlp(module, x)
    signal = torch.randn_like(actual)
    parameters = (x, *trainable(module))
    ag = torch.autograd.grad(actual, parameters, signal)
    eg = torch.autograd.grad(expected, parameters, signal)
    torch.testing.assert_close(actual, expected, rtol=.04, atol=.003)
    for a, e in zip(ag, eg):
        torch.testing.assert_close(a, e.to(a.dtype), rtol=.05, atol=.003)


def test_empty_input_returns_zero_parameter_gradients():
    module = MLP(TinyConfig, Runtime(rank=4, mlp_tile=5), "cuda")
    x = torch.empty(2, 0, 32, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    output = module(x)
    gradients = torch.autograd.grad(output.sum(), (x, *trainable(module)))
    assert gradients[0].shape == x.shape
    assert all(torch.count_nonzero(gradient) == 0 for gradient in gradients)


def test_untiled_store_activations_path_matches_recompute_path():
    module = MLP(TinyConfig, Runtime(rank=4), "cuda")
    randomise_b(module, .1)
    x = torch.randn(3, 11, 32, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    fused, stored = module(x), module.untiled(x)
    assert relative(fused, stored) < 2e-2
    signal = torch.randn_like(fused)
    for a, b in zip(torch.autograd.grad(fused, (x, *trainable(module)), signal),
                    torch.autograd.grad(stored, (x, *trainable(module)), signal)):
        assert relative(a, b) < 3e-2


def test_full_width_bf16_mlp_block_with_recompute():
    """Hidden 4096, intermediate 14336, NF4 base weights, rank-256 adapters, 2051 packed tokens:
    recompute and cached modes bit-identical, both within 2e-2 relative Frobenius error of a bf16
    PyTorch composition, and the recompute mode retains only x."""
    torch.manual_seed(3)
    module = MLP(WideConfig, Runtime(rank=256), "cuda")
    for projection in (module.gate_proj, module.up_proj, module.down_proj):
        projection.install_nf4(projection.weight.detach().clone(), "cuda", nested=False)
        torch.nn.init.normal_(projection.lora_B, std=.005)
    rows = 2051
    x = torch.randn(1, rows, 4096, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    signal = torch.randn_like(x)
    params = (x, *trainable(module))
    before = _lib.tcgen05_launch_count()
    saved = []
    with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(t) or t, lambda t: t):
        recomputed = module(x, residual=x, cache=False)
    allowed = {x.data_ptr(), *(p.data_ptr() for p in module.parameters())}
    assert all(t.data_ptr() in allowed for t in saved)
    g_recompute = torch.autograd.grad(recomputed, params, signal)
    assert _lib.tcgen05_launch_count() > before
    cached = module(x, residual=x, cache=True)
    g_cached = torch.autograd.grad(cached, params, signal)
    assert torch.equal(recomputed, cached)
    for a, b in zip(g_recompute, g_cached):
        assert torch.equal(a, b)
    z = x.detach().clone().requires_grad_(True)
    expected = oracle_mlp(module, z) + z
    reference = torch.autograd.grad(expected, (z, *trainable(module)), signal)
    for name, left, right in zip(["y", "dx"] + ["param"] * 6, (recomputed, *g_recompute), (expected, *reference)):
        assert torch.isfinite(left).all()
        assert relative(left, right) < 2e-2, name


def test_config3_recompute_versus_stored_activations(capsys):
    """One SwiGLU MLP block, hidden 4096, intermediate 14336, NF4 base weights, rank-256 adapters,
    8 packed rows of 4096 tokens (32768 tokens). Recompute-in-backward must retain only the block
    input between forward and backward; the cached mode retains exactly `cache_bytes` more; the
    three-node autograd path (`untiled`) retains the most. Times are printed for the record."""
    torch.manual_seed(9)
    module = MLP(WideConfig, Runtime(rank=256), "cuda")
    for projection in (module.gate_proj, module.up_proj, module.down_proj):
        projection.install_nf4(projection.weight.detach().clone(), "cuda", nested=False)
        torch.nn.init.normal_(projection.lora_B, std=.005)
    rows = 8 * 4096
    x = torch.randn(8, 4096, 4096, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    signal = torch.randn_like(x)
    params = (x, *trainable(module))
    report = {}
    outputs = {}
    for name, forward in (("recompute", lambda: module(x, cache=False)), ("cached", lambda: module(x, cache=True)),
                          ("stored", lambda: module.untiled(x))):
        for _ in range(2):   # warm-up, then the measured pass (nothing of the first pass stays alive)
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats()
            base = torch.cuda.memory_allocated()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            y = forward()
            torch.cuda.synchronize()
            retained = torch.cuda.memory_allocated() - base - y.numel() * 2
            grads = torch.autograd.grad(y, params, signal)
            stop.record()
            torch.cuda.synchronize()
            peak = torch.cuda.max_memory_allocated() - base
            report[name] = dict(retained_mb=retained / 2**20, peak_mb=peak / 2**20, ms=start.elapsed_time(stop))
            outputs[name] = (y.detach(), grads)
            del y, grads
            if _ == 0:
                del outputs[name]
    with capsys.disabled():
        print("\nconfig3 (32768 tokens):", {k: {a: round(b, 1) for a, b in v.items()} for k, v in report.items()})
    assert report["recompute"]["retained_mb"] < 1.0                       # nothing but x (already counted in base)
    expected_cache = module.cache_bytes(rows) / 2**20
    assert abs(report["cached"]["retained_mb"] - expected_cache) < 1.0
    assert report["stored"]["retained_mb"] > report["cached"]["retained_mb"]
    assert torch.equal(outputs["recompute"][0], outputs["cached"][0])
    for a, b in zip(outputs["recompute"][1], outputs["cached"][1]):
        assert torch.equal(a, b)
    for a, b in zip(outputs["recompute"][1], outputs["stored"][1]):
        assert relative(a, b) < 3e-2


def test_keeping_low_rank_inputs_changes_what_is_retained_not_a_value():
    module = MLP(TinyConfig, Runtime(rank=8, mlp_tile=5), "cuda")
    randomise_b(module, .05)
    module.cache_intermediates = True
    x = torch.randn(2, 7, 32, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    signal = torch.randn_like(x)
    params = (x, *trainable(module))
    results = []
    for keep in (False, True):
        for projection in (module.gate_proj, module.up_proj, module.down_proj):
            projection.keep_low_rank = keep
        saved = []
        with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(t) or t, lambda t: t):
            out = module(x, residual=x)
        allowed = {x.data_ptr(), *(p.data_ptr() for p in module.parameters())}
        retained = sum(t.numel() * t.element_size() for t in saved if t.data_ptr() not in allowed)
        first = torch.autograd.grad(out, params, signal, retain_graph=True)
        again = torch.autograd.grad(out, params, signal)
        assert all(torch.equal(a, b) for a, b in zip(first, again))
        results.append((out, first, retained))
    assert torch.equal(results[0][0], results[1][0])
    assert all(torch.equal(a, b) for a, b in zip(results[0][1], results[1][1]))
    assert results[0][2] == module.cache_bytes(14)
    # plus the down projection's [rows, rank] low-rank input and the six adapters in the compute dtype (bf16)
    adapters = sum(p.numel() for name, p in module.named_parameters() if "lora_" in name)
    assert results[1][2] == module.cache_bytes(14) + 14 * 8 * 2 + adapters * 2


# ---- gate / up projections with the SwiGLU in the GEMM's epilogue ---------------------------------

class MidConfig:
    hidden_size, intermediate_size = 512, 384


def _mid_module(nf4, nested=False, ranks=(16, 24, 8)):
    module = MLP(MidConfig, Runtime(rank=16), "cuda")
    for name, rank in zip(("gate_proj", "up_proj", "down_proj"), ranks):
        original = getattr(module, name)
        setattr(module, name, Projection(original.weight.shape[1], original.weight.shape[0], rank=rank, device="cuda"))
    for projection in (module.gate_proj, module.up_proj, module.down_proj):
        if nf4:
            projection.install_nf4(projection.weight.detach().clone(), "cuda", nested=nested)
        torch.nn.init.normal_(projection.lora_B, std=.05)
    return module


@pytest.mark.parametrize("nested", [False, True])
def test_interleaved_decode_places_both_weights_in_128_row_blocks(nested):
    from causal_tuner_b200.kernels.linear import materialize, materialize_into_pair
    module = _mid_module(True, nested)
    (gate_weight, *_), gate_state = mlp_cuda.projection_parameters(module.gate_proj)
    (up_weight, *_), up_state = mlp_cuda.projection_parameters(module.up_proj)
    pair = torch.full((2 * 384, 512), float("nan"), device="cuda", dtype=torch.bfloat16)
    materialize_into_pair(gate_weight, gate_state, pair, 0)
    materialize_into_pair(up_weight, up_state, pair, 1)
    blocks = pair.view(3, 2, 128, 512)
    assert torch.equal(blocks[:, 0].reshape(384, 512), materialize(gate_weight, gate_state, torch.bfloat16))
    assert torch.equal(blocks[:, 1].reshape(384, 512), materialize(up_weight, up_state, torch.bfloat16))
    dense = torch.randn(384, 512, device="cuda")
    materialize_into_pair(dense, None, pair, 1)
    assert torch.equal(blocks[:, 1].reshape(384, 512), dense.bfloat16())


@pytest.mark.parametrize("rows,inner,width", [(1000, 512, 384), (256, 512, 384), (77, 512, 384), (300, 520, 128),
                                              (513, 72, 256)])
def test_gated_launch_is_bit_identical_to_two_projections_and_the_activation(rows, inner, width):
    """ct_gated_forward / ct_gated_backward / ct_gated_input_gradient against ct_forward_linear x 2 + ct_swiglu
    and ct_input_gradient_group on the same operands: every output equal bit for bit, buffers the launch must
    not touch untouched, the in-place form (hidden over its own gradient) included."""
    from causal_tuner_b200.kernels import linear
    torch.manual_seed(rows)
    ranks = (16, 24)
    bf = dict(device="cuda", dtype=torch.bfloat16)
    x = torch.randn(rows, inner, **bf)
    weights = [torch.randn(width, inner, **bf) * .05 for _ in range(2)]
    a = [torch.randn(rank, inner, **bf) * .05 for rank in ranks]
    b = [torch.randn(width, rank, **bf) * .2 for rank in ranks]
    both = torch.empty(rows, sum(ranks), **bf)
    linear.matmul(x, torch.cat(a).T, out=both)
    xa = [both[:, :ranks[0]], both[:, ranks[0]:]]
    pair = torch.empty(2 * width, inner, **bf)
    for which in range(2):
        linear.materialize_into_pair(weights[which], None, pair, which)
    gate, up = torch.empty(rows, width, **bf), torch.empty(rows, width, **bf)
    for which, out in enumerate((gate, up)):
        linear.apply_projection(x, weights[which], b[which], xa[which], out=out)
    hidden = mlp_cuda.activation(gate, up)
    before = _lib.tcgen05_launch_count()
    fused = [torch.full((rows + 1, width), 7.0, **bf) for _ in range(3)]        # one guard row each
    linear.gated_projections(x, pair, xa[0], xa[1], b[0], b[1], hidden=fused[0][:rows], gate=fused[1][:rows],
                             up=fused[2][:rows])
    assert _lib.tcgen05_launch_count() == before + 1
    for actual, expected in zip(fused, (hidden, gate, up)):
        assert torch.equal(actual[:rows], expected)
        assert (actual[rows] == 7).all()
    alone = torch.empty(rows, width, **bf)
    linear.gated_projections(x, pair, xa[0], xa[1], b[0], b[1], hidden=alone)
    assert torch.equal(alone, hidden)
    # backward: (gate, up, d_hidden) -> (d_gate, d_up, hidden) in place, against recomputed accumulators
    upstream = torch.randn(rows, width, **bf)
    expected = [gate.clone(), up.clone(), upstream.clone()]
    mlp_cuda.activation(*expected)
    buffers = [torch.empty(rows, width, **bf) for _ in range(2)]
    in_place = upstream.clone()
    linear.gated_projections(x, pair, xa[0], xa[1], b[0], b[1], hidden=in_place, gate=buffers[0], up=buffers[1],
                             gradient=in_place)
    for actual, wanted in zip((*buffers, in_place), expected):
        assert torch.equal(actual, wanted)
    # input gradient through the interleaved weights
    lows = [torch.empty(rows, sum(ranks), **bf) for _ in range(2)]
    split = lambda t: [t[:, :ranks[0]], t[:, ranks[0]:]]
    dx = [torch.full((rows, inner), float("nan"), **bf) for _ in range(2)]
    linear.input_gradient_group(expected[:2], weights, a, b, dx[0], split(lows[0]))
    linear.gated_input_gradient(expected[0], expected[1], pair, a[0], a[1], b[0], b[1], dx[1], split(lows[1]))
    assert torch.equal(dx[0], dx[1]) and torch.equal(lows[0], lows[1])
    linear.input_gradient_group(expected[:2], weights, a, b, dx[0], split(lows[0]), add=True)
    linear.gated_input_gradient(expected[0], expected[1], pair, a[0], a[1], b[0], b[1], dx[1], split(lows[1]), add=True)
    assert torch.equal(dx[0], dx[1])


@pytest.mark.parametrize("nf4", [False, True])
@pytest.mark.parametrize("cache", [False, True])
@pytest.mark.parametrize("tile", [0, 300])
def test_mlp_with_the_gated_launch_equals_the_separate_kernels(monkeypatch, nf4, cache, tile):
    """The whole operator with and without the gated launch (forward pass and the recompute of the backward pass):
    output and every gradient equal bit for bit, with cached activations and with recompute, whole and in row
    tiles."""
    torch.manual_seed(5)
    module = _mid_module(nf4)
    module.tile = tile
    x = torch.randn(3, 333, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    signal = torch.randn_like(x)
    params = (x, *trainable(module))
    results = {}
    for fused in ("0", "1"):
        monkeypatch.setenv("CT_B200_MLP_FUSED", fused)              # the recompute of the backward pass
        monkeypatch.setenv("CT_B200_MLP_FUSED_FORWARD", fused)      # a forward pass that keeps gate and up (off by default)
        monkeypatch.setenv("CT_B200_MLP_FUSED_BACKWARD", fused)     # SwiGLU backward in the down projection's GEMM (off by default)
        monkeypatch.setenv("CT_B200_DECODE_TRANSPOSED", fused)      # weights of input-gradient products decoded transposed
        before = _lib.launch_count()
        y = module(x, residual=x, cache=cache)
        grads = torch.autograd.grad(y, params, signal)
        results[fused] = (y, *grads, _lib.launch_count() - before)
    assert results["1"][-1] < results["0"][-1]           # fewer launches: the path was taken
    for separate, gated in zip(results["0"][:-1], results["1"][:-1]):
        assert torch.isfinite(gated).all()
        assert torch.equal(separate, gated)


@pytest.mark.parametrize("rows", [1000, 256, 77])
@pytest.mark.parametrize("width", [384, 416])
def test_swiglu_backward_inside_the_down_projections_input_gradient(rows, width):
    """ct_input_gradient_swiglu against ct_input_gradient followed by ct_swiglu: (d_gate, d_up, hidden) equal bit for
    bit, the kept gate and up untouched, nothing written past the rows."""
    from causal_tuner_b200.kernels import linear
    torch.manual_seed(rows + width)
    hidden_size, rank = 512, 24
    bf = dict(device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(rows, hidden_size, **bf)
    weight = torch.randn(hidden_size, width, **bf) * .05
    a, b = torch.randn(rank, width, **bf) * .05, torch.randn(hidden_size, rank, **bf) * .2
    gate, up = torch.randn(rows, width, **bf), torch.randn(rows, width, **bf)
    kept = (gate.clone(), up.clone())
    low = torch.empty(rows, rank, **bf)
    linear.matmul(dy, b, out=low)
    dh = torch.empty(rows, width, **bf)
    linear.input_gradient_with(dy, weight, a, low, dh)
    expected = [gate.clone(), up.clone(), dh]
    mlp_cuda.activation(*expected)
    outputs = [torch.full((rows + 1, width), 7.0, **bf) for _ in range(3)]
    before = _lib.tcgen05_launch_count()
    linear.input_gradient_swiglu(dy, weight, a, low, gate, up, outputs[0][:rows], outputs[1][:rows], outputs[2][:rows])
    assert _lib.tcgen05_launch_count() == before + 1
    for actual, wanted in zip(outputs, expected):
        assert torch.equal(actual[:rows], wanted)
        assert (actual[rows] == 7).all()
    assert torch.equal(gate, kept[0]) and torch.equal(up, kept[1])
