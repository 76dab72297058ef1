"""Install the unmodified reference next to the oracle, as `oracle/_ref/`.

TEST INFRASTRUCTURE ONLY, like everything else under oracle/. The reference
(RealJosephus/causal-tuner) is a pure-Python package; this recipe installs it with pip from
its checkout into `oracle/_ref/` (offline, no dependencies, no build isolation) and places
its `tests/` directory beside it as `oracle/_ref/reference_tests/`. `oracle/_ref/` is not part
of the source history (it is listed in .gitignore); it exists so that

  * the GPU parity tests can call the reference's own CUDA path (Triton kernels + cuBLAS +
    FlashAttention-2) on the same seeded inputs as this library,
  * the reference's own operator tests can be run against this library's modules,
  * bench.py can time the reference's CPU branch and its GPU composition beside this library.

Nothing under causal_tuner_b200/ imports it.

    python oracle/make_ref.py [--source <reference checkout>] [--force]

The reference needs bitsandbytes only to *pack* NF4 weights (modeling/lora.py:41-56); the
decode and everything after it read a duck-typed quant state, so the tests pack with this
repository's quantiser and hand both sides the same bytes (see tests/reference_gpu.py).
"""

import argparse
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")
DEFAULT_SOURCE = "/root/reference"
MARKER = os.path.join(TARGET, "causal_tuner", "kernels", "linear.py")


def available():
    """True when the installed reference is present."""
    return os.path.exists(MARKER)


def install(source=DEFAULT_SOURCE, force=False, quiet=True):
    """pip-install `source` into oracle/_ref and copy its tests beside it. Returns the target
    directory, or None when there is no reference checkout to install from."""
    if available() and not force:
        return TARGET
    if not os.path.exists(os.path.join(source, "pyproject.toml")):
        return None
    if os.path.exists(TARGET):
        shutil.rmtree(TARGET)
    with tempfile.TemporaryDirectory(prefix="ct_ref_build_") as scratch:
        # The checkout is read-only and setuptools writes egg-info beside the sources: build from a copy.
        work = os.path.join(scratch, "reference")
        shutil.copytree(source, work, ignore=shutil.ignore_patterns(".git", "__pycache__", "*.pyc"))
        command = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                   "--no-compile", "--target", TARGET, work]
        subprocess.run(command, check=True, stdout=subprocess.DEVNULL if quiet else None,
                       stderr=subprocess.STDOUT if quiet else None)
        tests = os.path.join(work, "tests")
        if os.path.isdir(tests):
            shutil.copytree(tests, os.path.join(TARGET, "reference_tests"),
                            ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    if not available():
        raise RuntimeError("pip reported success but oracle/_ref/causal_tuner is missing")
    return TARGET


if __name__ == "__main__":
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--source", default=DEFAULT_SOURCE)
    parser.add_argument("--force", action="store_true")
    arguments = parser.parse_args()
    result = install(arguments.source, arguments.force, quiet=False)
    print(result if result else f"no reference checkout at {arguments.source}; nothing installed")
