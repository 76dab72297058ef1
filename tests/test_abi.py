"""The shared library loads, exports exactly the C ABI of include/ct_b200.h, and rejects bad
arguments without touching a GPU."""

import ctypes
import os
import re

import pytest
import torch

from causal_tuner_b200 import _lib
from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "ct_b200.h")


def declared_symbols():
    with open(HEADER) as f:
        text = f.read()
    return sorted(set(re.findall(r"CT_API\s+[\w\s\*]+?\b(ct_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_what_the_binding_expects():
    assert declared_symbols() == sorted(_lib.SIGNATURES)


def test_binding_passes_as_many_arguments_as_the_header_declares():
    with open(HEADER) as f:
        text = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
    for name, parameters in re.findall(r"CT_API\s+[\w\s\*]+?\b(ct_[a-z0-9_]+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        parameters = parameters.strip()
        count = 0 if parameters in ("", "void") else parameters.count(",") + 1
        assert count == len(_lib.SIGNATURES[name][1]), name
        # pointers are passed as void pointers, 64-bit sizes as int64, never as a narrower type
        for declared, bound in zip(parameters.split(","), _lib.SIGNATURES[name][1]):
            if "*" in declared:
                assert bound is ctypes.c_void_p, (name, declared)
            elif "int64_t" in declared:
                assert bound is ctypes.c_int64, (name, declared)
            elif "float" in declared:
                assert bound is ctypes.c_float, (name, declared)
            elif parameters not in ("", "void"):
                assert bound is ctypes.c_int, (name, declared)


def test_library_exports_every_declared_symbol():
    library = ctypes.CDLL(_lib.LIBRARY_PATH)
    for name in declared_symbols():
        assert getattr(library, name) is not None, name


def test_every_declaration_cites_the_reference_or_says_it_has_no_counterpart():
    with open(HEADER) as f:
        text = f.read()
    blocks = re.split(r"/\* ---- ", text)[2:]  # skip the preamble and the library-state block
    assert len(blocks) >= 8
    for block in blocks:
        assert re.search(r"(kernels|training|modeling|data)/\w+\.py:\d+", block) or "no counterpart in the reference" in block, block[:60]


def test_abi_version_and_counters():
    library = _lib.load()
    assert library.ct_abi_version() == 1
    assert library.ct_launch_count() >= 0 and library.ct_tcgen05_launch_count() >= 0


def test_argument_errors_are_reported_without_a_device():
    library = _lib.load()
    assert library.ct_nf4_decode(None, None, None, None, None, None, None, -1, 64, 0, 0, 0, 0, None) == _lib.ERR_ARG
    assert b"ct_nf4_decode" in library.ct_last_error()
    assert library.ct_nf4_decode(None, None, None, None, None, None, None, 10, 63, 0, 0, 0, 0, None) == _lib.ERR_ARG
    assert library.ct_nf4_decode(None, None, None, None, None, None, None, 0, 64, 0, 0, 0, 0, None) == _lib.OK
    assert library.ct_matmul(None, 1, 1, None, 1, 1, None, 1, 4, 4, 4, 0, 0, 0, 0, None) == _lib.ERR_ARG
    assert library.ct_matmul(None, 1, 1, None, 1, 1, None, 1, 0, 4, 4, 0, 0, 0, 0, None) == _lib.OK
    assert library.ct_swiglu(None, None, None, None, None, None, 8, 1, 1, None) == _lib.ERR_ARG
    assert library.ct_rope(None, None, None, None, 4, 2, 7, 2, 0, 1, None) == _lib.ERR_ARG  # odd head_dim
    assert library.ct_forward_linear(None, 0, None, 0, None, None, None, None, 0, None, 0, None, 0, 0, 8, 8, 4, 1, 0,
                                     None) == _lib.OK  # zero rows: nothing to do
    with pytest.raises(ValueError):
        _lib.check(library.ct_cast(None, 0, 0, None, 1, 0, -1, 4, None))


def test_workspace_query_is_pure_arithmetic():
    library = _lib.load()
    # rank-256 adapter on a 4096 -> 14336 projection over 16384 tokens: dA is split, dB is not
    need = library.ct_parameter_gradients_workspace(16384, 4096, 14336, 256, _lib.BF16, _lib.PATH_AUTO)
    assert need == 4 * 256 * 4096 * 4
    assert library.ct_parameter_gradients_workspace(16384, 4096, 14336, 256, _lib.F32, _lib.PATH_AUTO) == 0
    assert library.ct_parameter_gradients_workspace(16384, 4096, 14336, 256, _lib.BF16, _lib.PATH_SIMT) == 0


def test_operators_refuse_cpu_tensors():
    from causal_tuner_b200.kernels.linear import forward_linear
    from causal_tuner_b200.kernels.mlp_cuda import activation
    from causal_tuner_b200.modeling.lora import Projection
    x = torch.randn(4, 8)
    with pytest.raises(RuntimeError, match="no CPU path"):
        forward_linear(x, torch.randn(8, 8), torch.randn(2, 8), torch.randn(8, 2), out=torch.empty(4, 8), xa=torch.empty(4, 2))
    with pytest.raises(RuntimeError, match="no CPU path"):
        activation(x, x)
    with pytest.raises(RuntimeError, match="no CPU path"):
        Projection(8, 8, rank=2, device="cpu")(x)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_library", None)
    monkeypatch.setattr(_lib, "LIBRARY_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(_lib.LibraryMissing, match="no CPU or PyTorch fallback"):
        _lib.load()
