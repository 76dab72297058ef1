"""ct_nf4_encode / ct_nf4_nest against the CPU oracle's encoder: bit-exact codes and statistics.

The encoding rule itself is not pinned by the reference (it calls bitsandbytes,
modeling/lora.py:41-56); what is pinned is that decoding inverts it (the decode fixtures) and that
the device encoder, the host rule and the oracle agree."""

import numpy as np
import pytest
import torch

from causal_tuner_b200 import _lib
from causal_tuner_b200.kernels.nf4_cuda import dequantize_nf4
from causal_tuner_b200.quant import quantize_nf4
from oracle import nf4 as oracle_nf4

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("gpu_guard")]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape,blocksize", [((71, 96), 64), ((1, 1), 64), ((3, 21), 64), ((64, 130), 128), ((5, 40), 8),
                                             ((300, 1000), 256), ((2048, 1024), 64)])
def test_codes_and_absmax_match_the_oracle(dtype, shape, blocksize):
    generator = torch.Generator().manual_seed(shape[0] * 7 + blocksize)
    weight = (torch.randn(shape, generator=generator) * 0.02).to(dtype)
    weight.view(-1)[::97] = 0                                   # exact zeros sit on a level
    before = _lib.launch_count()
    packed, state = quantize_nf4(weight.cuda(), blocksize=blocksize)
    assert _lib.launch_count() == before + 1                    # the kernel ran, not the tensor-op rule
    expected_packed, expected_absmax = oracle_nf4.encode(weight.float().numpy(), blocksize)
    assert packed.shape == ((weight.numel() + 1) // 2, 1) and packed.dtype == torch.uint8
    assert np.array_equal(packed.cpu().numpy().reshape(-1), expected_packed)
    assert np.array_equal(state.absmax.cpu().numpy(), expected_absmax)
    assert state.shape == weight.shape and state.dtype == dtype and state.blocksize == blocksize


@pytest.mark.parametrize("rows,blocksize2", [(917, 256), (256, 256), (5, 64), (3000, 300)])
def test_nested_statistics_match_the_oracle(rows, blocksize2):
    generator = torch.Generator().manual_seed(rows)
    weight = torch.randn(rows, 64, generator=generator) * torch.rand(rows, 1, generator=generator) * 0.05
    packed, state = quantize_nf4(weight.cuda(), blocksize=64, nested=True, blocksize2=blocksize2)
    host_packed, host_state = quantize_nf4(weight, blocksize=64, nested=True, blocksize2=blocksize2)
    _, absmax = oracle_nf4.encode(weight.numpy(), 64)
    indices, absmax2, offset = oracle_nf4.encode_statistics(absmax, blocksize2)
    assert np.array_equal(state.absmax.cpu().numpy(), indices)
    assert np.array_equal(state.state2.absmax.cpu().numpy(), absmax2)
    assert np.float32(state.offset.item()) == offset
    assert torch.equal(packed.cpu(), host_packed) and torch.equal(state.absmax.cpu(), host_state.absmax)
    assert state.nested and state.state2.blocksize == blocksize2 and state.absmax.dtype == torch.uint8


def test_unaligned_views_and_odd_lengths():
    base = (torch.randn(4099) * 0.1).bfloat16().cuda()
    for start, length in ((1, 4097), (3, 129), (0, 4099), (5, 1)):
        view = base[start:start + length]
        packed, state = quantize_nf4(view, blocksize=64)
        expected_packed, expected_absmax = oracle_nf4.encode(view.float().cpu().numpy(), 64)
        assert np.array_equal(packed.cpu().numpy().reshape(-1), expected_packed)
        assert np.array_equal(state.absmax.cpu().numpy(), expected_absmax)


def test_full_size_weight_is_a_fixed_point_of_decode_then_encode():
    # gate projection of the 7B-class decoder: 14336 x 4096. Decoding the codes and encoding the
    # result must reproduce codes and scales (every level times absmax maps back to its own level),
    # and the decode error is bounded by half the widest level gap per block.
    generator = torch.Generator(device="cuda").manual_seed(3)
    weight = (torch.randn(14336, 4096, device="cuda", generator=generator) * 0.02).bfloat16()
    packed, state = quantize_nf4(weight, blocksize=64)
    state.dtype = torch.float32
    decoded = dequantize_nf4(packed, state, torch.float32)
    again, state_again = quantize_nf4(decoded, blocksize=64)
    assert torch.equal(again, packed) and torch.equal(state_again.absmax, state.absmax)
    error = (decoded - weight.float()).abs().view(-1, 64)
    assert bool((error <= 0.16 * state.absmax[:, None] + 1e-8).all())
    assert int(packed.view(-1).sum(dtype=torch.int64)) == int(again.view(-1).sum(dtype=torch.int64))


def test_blocksizes_outside_the_kernel_use_the_tensor_rule_on_the_device():
    weight = torch.randn(8, 4096, device="cuda")
    packed, state = quantize_nf4(weight, blocksize=4096)
    expected_packed, expected_absmax = oracle_nf4.encode(weight.cpu().numpy(), 4096)
    assert np.array_equal(packed.cpu().numpy().reshape(-1), expected_packed)
    assert np.array_equal(state.absmax.cpu().numpy(), expected_absmax)
    with pytest.raises(NotImplementedError):
        code = torch.zeros(16, device="cuda")
        out, absmax = torch.empty(16384, dtype=torch.uint8, device="cuda"), torch.empty(8, device="cuda")
        _lib.check(_lib.load().ct_nf4_encode(weight.data_ptr(), weight.numel(), _lib.F32, 4096, code.data_ptr(),
                                             out.data_ptr(), absmax.data_ptr(), None))
