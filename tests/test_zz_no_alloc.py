"""ct_parameter_gradients_noalloc: the LoRA-gradient entry point for hosts that must not allocate.

Some callers of this library cannot call cudaMalloc when the gradients are due: a runtime that
gave the whole GPU to its own pool at start-up, or a step loop that cannot take the device-wide
synchronisation an allocation implies. For them the slice scratch of the token-contracted dA/dB
products is a fixed 16 MiB array inside the library instead of a caller-provided workspace.
The test drives the entry point through the C ABI, twice in a row on the shared array, and
expects exactly what ct_parameter_gradients produces with a torch-allocated workspace.

This file sorts last on purpose, so that a run that stops at the first failure has already run
every other test.
"""

import pytest
import torch

from causal_tuner_b200 import _lib

pytestmark = pytest.mark.gpu


def operands(rows, inner, outer, rank, seed):
    generator = torch.Generator(device="cuda").manual_seed(seed)
    make = lambda *shape: torch.randn(*shape, device="cuda", generator=generator).bfloat16()
    return make(rows, inner), make(rows, outer), make(rows, rank), make(rows, rank)


def reference_gradients(x, dy, low, xa, add, seed_values):
    library = _lib.load()
    rows, inner = x.shape
    outer, rank = dy.shape[1], low.shape[1]
    da, db = seed_values[0].clone(), seed_values[1].clone()
    need = library.ct_parameter_gradients_workspace(rows, inner, outer, rank, _lib.BF16, _lib.PATH_AUTO)
    workspace = torch.empty(max(need, 1), device="cuda", dtype=torch.uint8)
    _lib.check(library.ct_parameter_gradients(
        x.data_ptr(), inner, dy.data_ptr(), outer, low.data_ptr(), rank, xa.data_ptr(), rank, da.data_ptr(),
        db.data_ptr(), rows, inner, outer, rank, int(add), _lib.BF16, workspace.data_ptr(), _lib.PATH_AUTO,
        torch.cuda.current_stream().cuda_stream))
    return da, db, need


def noalloc_gradients(x, dy, low, xa, add, da, db):
    """The call under test; `da` / `db` are made by the caller so that nothing is allocated in here."""
    library = _lib.load()
    rows, inner = x.shape
    outer, rank = dy.shape[1], low.shape[1]
    code = library.ct_parameter_gradients_noalloc(
        x.data_ptr(), inner, dy.data_ptr(), outer, low.data_ptr(), rank, xa.data_ptr(), rank, da.data_ptr(),
        db.data_ptr(), rows, inner, outer, rank, int(add), _lib.BF16, _lib.PATH_AUTO,
        torch.cuda.current_stream().cuda_stream)
    return code


def test_matches_the_workspace_entry_point_on_two_calls_in_a_row():
    library = _lib.load()
    assert library.ct_parameter_gradients_noalloc_capacity() == 16 << 20
    # Two different problems back to back: the second call finds the first call's partial sums
    # in the shared array and must not be affected by them. Both need slice scratch.
    for call, (rows, inner, outer, rank, add) in enumerate(((4096, 512, 768, 64, False), (2048, 1024, 256, 32, True))):
        x, dy, low, xa = operands(rows, inner, outer, rank, seed=call)
        start = (torch.randn(rank, inner, device="cuda"), torch.randn(outer, rank, device="cuda"))
        expected_da, expected_db, need = reference_gradients(x, dy, low, xa, add, start)
        assert 0 < need <= library.ct_parameter_gradients_noalloc_capacity()
        da, db = start[0].clone(), start[1].clone()
        torch.cuda.synchronize()
        free_before, allocated_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        _lib.check(noalloc_gradients(x, dy, low, xa, add, da, db))
        _lib.check_device()
        if call:
            # The property in the entry point's name. The first call on a device is the documented set-up
            # call (the driver places the library's image, scratch array included, on the device then);
            # from the second call on, neither the device's free memory nor torch's own count may move.
            assert torch.cuda.mem_get_info()[0] == free_before
            assert torch.cuda.memory_allocated() == allocated_before
        assert torch.equal(da, expected_da) and torch.equal(db, expected_db)
        # and both agree with a plain fp32 product of the same operands
        plain_da = low.float().T @ x.float() + (start[0] if add else 0)
        plain_db = dy.float().T @ xa.float() + (start[1] if add else 0)
        assert ((da - plain_da).norm() / plain_da.norm()).item() < 1e-5
        assert ((db - plain_db).norm() / plain_db.norm()).item() < 1e-5


def test_problems_beyond_the_built_in_capacity_are_refused_without_a_launch():
    library = _lib.load()
    rows, inner, outer, rank = 16384, 6144, 512, 256   # dA alone needs 3 slices of 6 MiB
    need = library.ct_parameter_gradients_workspace(rows, inner, outer, rank, _lib.BF16, _lib.PATH_AUTO)
    assert need > library.ct_parameter_gradients_noalloc_capacity()
    before = _lib.launch_count()
    code = library.ct_parameter_gradients_noalloc(1, inner, 1, outer, 1, rank, 1, rank, 1, 1, rows, inner, outer, rank, 0,
                                                  _lib.BF16, _lib.PATH_AUTO, None)
    assert code == _lib.ERR_UNSUPPORTED
    assert b"built-in" in library.ct_last_error()
    assert _lib.launch_count() == before
