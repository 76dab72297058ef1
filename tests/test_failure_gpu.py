"""Failure detection on the device without a fault: a wait that nothing completes runs into its limit,
the kernel returns, the host reads the status, and the context stays usable."""

import time

import pytest
import torch

from causal_tuner_b200 import _lib
from causal_tuner_b200.kernels import linear

pytestmark = [pytest.mark.gpu]


def test_a_wait_that_nothing_completes_is_reported_and_the_context_survives():
    library = _lib.load()
    _lib.check_device()                                           # nothing pending
    stream = torch.cuda.current_stream().cuda_stream
    started = time.perf_counter()
    _lib.check(library.ct_selftest_bounded_wait(2000, stream))    # a 2 ms limit
    with pytest.raises(RuntimeError, match="bounded wait"):
        _lib.check_device()
    assert time.perf_counter() - started < 1.0                    # gave up at its limit, not at the GEMM's 2 s
    assert b"nothing completes" in library.ct_last_error()
    _lib.check_device()                                           # reported once, then clear
    # the context is intact: a tensor-core product still gives exact results
    left = torch.randint(-3, 4, (256, 128), device="cuda").bfloat16()
    right = torch.randint(-3, 4, (128, 512), device="cuda").bfloat16()
    out = torch.empty(256, 512, device="cuda")
    linear.matmul(left, right, out=out)
    assert torch.equal(out, left.float() @ right.float())
    _lib.check_device()


def test_the_self_test_refuses_limits_it_should_not_wait_for():
    library = _lib.load()
    assert library.ct_selftest_bounded_wait(0, None) == _lib.ERR_ARG
    assert library.ct_selftest_bounded_wait(100001, None) == _lib.ERR_ARG
    _lib.check_device()


def test_an_update_does_not_pass_when_a_kernel_gave_up(golden):
    # Trainer.update ends with the device check, so a kernel that ran into its wait limit during the step
    # surfaces as an error of that step.
    from test_step_gpu import batch_of, load_model
    from causal_tuner_b200.modeling.model import Runtime
    from causal_tuner_b200.training import Trainer, make_optimizer
    g = golden("step_tiny_b1.npz")
    runtime = Runtime(rank=16, base_dtype=torch.float32, train_dtype=torch.float32, compute_dtype=torch.float32,
                      attention="vanilla", checkpoint=False)
    model = load_model(g, runtime, nf4=False)
    trainer = Trainer(model, make_optimizer(model, learning_rate=1e-4), device="cuda", loss_token_budget=128)
    _lib.check(_lib.load().ct_selftest_bounded_wait(1000, torch.cuda.current_stream().cuda_stream))
    with pytest.raises(RuntimeError, match="bounded wait"):
        trainer.update([batch_of(g)])
    assert trainer.update([batch_of(g)])["loss"] > 0              # the next step runs normally
