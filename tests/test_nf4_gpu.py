"""ct_nf4_decode against the reference-generated fixtures and the CPU oracle: bit-exact."""

import glob
import os

import numpy as np
import pytest
import torch

from causal_tuner_b200.kernels.linear import materialize
from causal_tuner_b200.kernels.nf4_cuda import dequantize_nf4
from causal_tuner_b200.quant import NestedState, QuantState, quantize_nf4
from oracle import nf4 as oracle_nf4
from conftest import GOLDEN

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("gpu_guard")]

NF4_FILES = sorted(os.path.basename(p) for p in glob.glob(os.path.join(GOLDEN, "nf4_*.npz")))


def state_from_fixture(g, dtype):
    cuda = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    state = QuantState(shape=torch.Size((int(g["rows"]), int(g["cols"]))), dtype=dtype, blocksize=int(g["blocksize"]),
                       absmax=cuda(g["absmax"]), code=cuda(g["code"]))
    if int(g["nested"]):
        state.nested, state.offset = True, cuda(g["offset"])
        state.state2 = NestedState(code=cuda(g["code2"]), absmax=cuda(g["absmax2"]), blocksize=int(g["blocksize2"]))
    return cuda(g["packed"]).reshape(-1, 1), state


@pytest.mark.parametrize("name", NF4_FILES)
def test_decode_matches_reference_fixture_bit_for_bit(golden, name):
    g = golden(name)
    packed, state = state_from_fixture(g, torch.float32)
    out = dequantize_nf4(packed, state, torch.float32)
    assert out.shape == state.shape
    assert torch.equal(out.cpu().reshape(-1), torch.from_numpy(g["out"]))
    # 16-bit outputs: round-to-nearest-even of the same fp32 product
    for state_dtype in (torch.bfloat16, torch.float16, torch.float32):
        state.dtype = state_dtype
        for dtype in (torch.bfloat16, torch.float32):
            expected = torch.from_numpy(g["out"]).to(state_dtype).to(dtype)
            assert torch.equal(materialize(packed, state, dtype).cpu().reshape(-1), expected)


@pytest.mark.parametrize("nested", [False, True])
@pytest.mark.parametrize("source_dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("blocksize", [64, 128, 4096])
def test_decode_matches_oracle_over_the_reference_test_grid(nested, source_dtype, blocksize):
    values = torch.randn(71, 96, device="cuda", dtype=source_dtype)
    packed, state = quantize_nf4(values, blocksize=blocksize, nested=nested)
    extra = {}
    if nested:
        extra = dict(nested=True, code2=state.state2.code.cpu().numpy(), absmax2=state.state2.absmax.cpu().numpy(),
                     offset=float(state.offset), blocksize2=state.state2.blocksize)
    for dtype in (torch.bfloat16, torch.float32):
        expected = oracle_nf4.decode(packed.cpu().numpy(), state.absmax.cpu().numpy(), state.code.cpu().numpy(),
                                     values.numel(), blocksize, state_dtype=source_dtype, out_dtype=dtype, **extra)
        actual = materialize(packed, state, dtype)
        assert actual.dtype == dtype and actual.shape == values.shape
        assert np.array_equal(actual.float().cpu().numpy().reshape(-1), expected)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_odd_tail_groups(dtype):
    source = torch.randn(17, 19, device="cuda", dtype=dtype)
    packed, state = quantize_nf4(source, blocksize=64, nested=True)
    extra = dict(nested=True, code2=state.state2.code.cpu().numpy(), absmax2=state.state2.absmax.cpu().numpy(),
                 offset=float(state.offset), blocksize2=state.state2.blocksize)
    for compute in (torch.bfloat16, torch.float32):
        guard = torch.full((17 * 19 + 64,), 7.0, device="cuda", dtype=compute)
        expected = oracle_nf4.decode(packed.cpu().numpy(), state.absmax.cpu().numpy(), state.code.cpu().numpy(), 323,
                                     64, state_dtype=dtype, out_dtype=compute, **extra)
        actual = materialize(packed, state, compute)
        assert np.array_equal(actual.float().cpu().numpy().reshape(-1), expected)
        assert (guard == 7).all()


def test_unaligned_packed_view_takes_the_scalar_path():
    values = torch.randn(64, 64, device="cuda")
    packed, state = quantize_nf4(values, blocksize=64)
    shifted = torch.empty(packed.numel() + 1, dtype=torch.uint8, device="cuda")[1:]
    shifted.copy_(packed.reshape(-1))
    assert shifted.data_ptr() % 16 != 0
    assert torch.equal(dequantize_nf4(shifted, state, torch.bfloat16), dequantize_nf4(packed, state, torch.bfloat16))


def test_full_size_weight_properties():
    """gate/up projection of the 7B configuration: 14336 x 4096 (58.7 M elements, larger than L2 when decoded).
    Checked through size-independent properties: every block reproduces its absmax-scaled level
    exactly, decode is idempotent, and sampled blocks equal the oracle."""
    torch.manual_seed(2)
    rows, cols = 14336, 4096
    weight = (torch.randn(rows, cols, device="cuda") * 0.02).bfloat16()
    packed, state = quantize_nf4(weight, blocksize=64)
    first = dequantize_nf4(packed, state, torch.bfloat16)
    second = dequantize_nf4(packed, state, torch.bfloat16)
    assert torch.equal(first, second)
    codes = torch.stack((packed.reshape(-1) >> 4, packed.reshape(-1) & 15), dim=-1).reshape(-1).long()
    expected = (state.code[codes] * state.absmax.repeat_interleave(64)).bfloat16().reshape(rows, cols)
    assert torch.equal(first, expected)
    # the largest magnitude of every block decodes to +-absmax exactly
    assert torch.equal(first.float().reshape(-1, 64).abs().amax(1), state.absmax.bfloat16().float())
    sample = slice(1000 * 64, 1000 * 64 + 64 * 50)
    oracle = oracle_nf4.decode(packed.reshape(-1)[sample.start // 2:sample.stop // 2].cpu().numpy(),
                               state.absmax[1000:1050].cpu().numpy(), state.code.cpu().numpy(), 64 * 50, 64,
                               state_dtype=torch.bfloat16, out_dtype=torch.bfloat16)
    assert np.array_equal(first.reshape(-1)[sample].float().cpu().numpy(), oracle)
    assert (first.float() - weight.float()).abs().max() <= 0.17 * state.absmax.max()


@pytest.mark.parametrize("nested", [False, True])
@pytest.mark.parametrize("source_dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape,blocksize", [((128, 192), 64), ((64, 64), 16), ((256, 128), 128), ((4096, 14336), 64)])
def test_transposed_decode_holds_the_same_values(monkeypatch, nested, source_dtype, shape, blocksize):
    """ct_nf4_decode_transposed: the [N, K] view of its [K, N] output equals ct_nf4_decode bit for bit, nothing is
    written past the buffer, and `materialize_for_gradient` hands out that view (or the plain decode where the
    shape does not allow the transposed one)."""
    from causal_tuner_b200.kernels.linear import decodes_transposed, materialize_for_gradient
    from causal_tuner_b200.kernels.nf4_cuda import dequantize_nf4_transposed
    monkeypatch.setenv("CT_B200_DECODE_TRANSPOSED", "1")      # off by default: no gain inside a power-capped step
    values = torch.randn(*shape, device="cuda", dtype=source_dtype)
    packed, state = quantize_nf4(values, blocksize=blocksize, nested=nested)
    expected = dequantize_nf4(packed, state, torch.bfloat16)
    actual = dequantize_nf4_transposed(packed, state, torch.bfloat16)
    assert actual.shape == expected.shape and actual.stride() == (1, shape[0])
    assert torch.equal(actual, expected)
    assert decodes_transposed(packed, state, torch.bfloat16)
    view = materialize_for_gradient(packed, state, torch.bfloat16)
    assert view.stride(0) == 1 and torch.equal(view, expected)
    odd, odd_state = quantize_nf4(torch.randn(72, 96, device="cuda", dtype=source_dtype), blocksize=64, nested=nested)
    assert not decodes_transposed(odd, odd_state, torch.bfloat16)
    assert materialize_for_gradient(odd, odd_state, torch.bfloat16).is_contiguous()
    assert not decodes_transposed(packed, state, torch.float32)
    monkeypatch.setenv("CT_B200_DECODE_TRANSPOSED", "0")
    assert materialize_for_gradient(packed, state, torch.bfloat16).is_contiguous()
