"""Builds ``libparpy_b200.so`` in-tree with nvcc for sm_100a.

    python -m parpy_b200.csrc.build [--verbose]

The shared object lands next to the package's Python files so that it travels
with a source checkout; it is not installed anywhere else.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
OUT = os.path.join(PKG, "libparpy_b200.so")
SOURCES = ["runtime.cu", "hmm_forward.cu", "rowops.cu", "sparse.cu", "hmm_prepare.cu", "hmm_viterbi.cu"]
HEADERS = ["common.cuh", "cluster.cuh", os.path.join("..", "..", "include", "parpy_b200.h")]
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-shared", "-Xcompiler", "-fPIC",
]


def needs_build():
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(HERE, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compiles every .cu file of the package into one shared library."""
    if not force and not needs_build():
        return OUT
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libparpy_b200.so")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
    cmd += ["-o", OUT] + [os.path.join(HERE, s) for s in SOURCES]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{r.stdout}\n{r.stderr}")
    if verbose:
        sys.stderr.write(r.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force=True, verbose="--verbose" in sys.argv))
