"""pytest plugin that runs the REFERENCE'S OWN test files against this library.

    python -m pytest -p reference_alias oracle/_ref/reference_tests/test_fused_core.py ...
    (with tests/ on PYTHONPATH; tests/test_reference_suite_gpu.py does exactly that in a child process)

Before any test module is imported it installs the drop-in the way INTEGRATION.md describes for a
maintainer: the reference package (oracle/_ref) is imported, and its operator modules
`causal_tuner.kernels.{linear, mlp_cuda, nf4_cuda, core_cuda, loss, loss_cuda}` are replaced by the
modules of the same names from `causal_tuner_b200.kernels`, both in `sys.modules` and as attributes of
the `causal_tuner.kernels` package. The reference's `modeling/`, `training/` and `data/` code then runs
unchanged on top of this library's operators. CT_ALIAS_MODULES (comma separated) narrows the list.
"""

import importlib
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEFAULT = ("linear", "mlp_cuda", "nf4_cuda", "core_cuda", "loss", "loss_cuda")


def install(names=None):
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    from oracle import ref_bridge
    ref_bridge.load()
    package = importlib.import_module("causal_tuner.kernels")
    chosen = names or tuple(n for n in os.environ.get("CT_ALIAS_MODULES", ",".join(DEFAULT)).split(",") if n)
    for name in chosen:
        module = importlib.import_module(f"causal_tuner_b200.kernels.{name}")
        sys.modules[f"causal_tuner.kernels.{name}"] = module
        setattr(package, name, module)
    return chosen


def pytest_configure(config):
    config._ct_aliased = install()


def pytest_terminal_summary(terminalreporter, exitstatus, config):
    terminalreporter.write_line(
        f"causal_tuner.kernels modules served by causal_tuner_b200: {', '.join(config._ct_aliased)}")
