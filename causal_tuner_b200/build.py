"""Compile causal_tuner_b200/csrc/*.cu into libct_b200.so for sm_100a.

The library is built in-tree with a plain ``nvcc -shared`` so that the binary
travels with the source tree; nothing is installed and no JIT cache is used.
``python -m causal_tuner_b200.build`` rebuilds it.
"""

import hashlib
import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(ROOT, "csrc")
LIBRARY = os.path.join(ROOT, "libct_b200.so")
STAMP = os.path.join(ROOT, "libct_b200.so.stamp")
SOURCES = ("api.cu", "nf4.cu", "nf4_encode.cu", "elementwise.cu", "norm_loss.cu", "optimizer.cu", "gemm_simt.cu", "gemm_tc.cu")
FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden")


def _nvcc():
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc was not found; libct_b200.so cannot be built")
    return path


def _digest():
    h = hashlib.sha256()
    for name in sorted(os.listdir(CSRC)):
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    with open(os.path.join(ROOT, "..", "include", "ct_b200.h"), "rb") as f:
        h.update(f.read())
    h.update(" ".join(FLAGS).encode())
    return h.hexdigest()


def up_to_date():
    if not (os.path.exists(LIBRARY) and os.path.exists(STAMP)):
        return False
    with open(STAMP) as f:
        return f.read().strip() == _digest()


def build(force=False, verbose=False):
    """Build the shared library unless the sources are unchanged since the last build."""
    if not force and up_to_date():
        return LIBRARY
    nvcc = _nvcc()
    objects = []
    build_dir = os.path.join(ROOT, "build")
    os.makedirs(build_dir, exist_ok=True)
    flags = list(FLAGS)
    processes = []
    for source in SOURCES:
        obj = os.path.join(build_dir, source.replace(".cu", ".o"))
        objects.append(obj)
        cmd = [nvcc, *flags, "-c", os.path.join(CSRC, source), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        processes.append((source, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for source, process in processes:
        output, _ = process.communicate()
        if verbose or process.returncode:
            sys.stderr.write(output)
        if process.returncode:
            raise RuntimeError(f"nvcc failed on {source}")
    subprocess.check_call([nvcc, "-shared", "-o", LIBRARY, *objects, "-lcudart"])
    with open(STAMP, "w") as f:
        f.write(_digest())
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
