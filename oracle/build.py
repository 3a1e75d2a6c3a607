"""Builds the CPU oracle library and, where the reference checkout is present,
the reference's own CUDA implementation of the HMM forward algorithm.

TEST INFRASTRUCTURE ONLY. Outputs:

  oracle/liboracle.so        gcc -O2 -fopenmp build of the C restatements
  oracle/libparpy_emitted.so nvcc build of parpy_emitted.cu: the CUDA program ParPy's compiler
                             emits for forward_kernel, written out by hand from its rules
  oracle/_ref/trellis_5mer.so, oracle/_ref/trellis_7mer.so
                             nvcc build of benchmarks/{5,7}mer/hmm.cu, compiled
                             from the reference sources where they lie (nothing
                             is copied); exports init/forward/viterbi with the
                             ctypes protocol of benchmarks/7mer/trellis.py:93-138

    python -m oracle.build [/path/to/ParPy]
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")
C_SOURCES = ["hmm_oracle.c", "kernels_oracle.c", "viterbi_oracle.c"]


def reference_root():
    """Where the reference checkout lies: ``$PARPY_REFERENCE_ROOT``, else a
    directory named ``reference`` beside this repository. None when absent."""
    env = os.environ.get("PARPY_REFERENCE_ROOT")
    if env:
        return env if os.path.isdir(env) else None
    sibling = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return sibling if os.path.isdir(os.path.join(sibling, "benchmarks")) else None


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"{' '.join(cmd)} failed:\n{r.stdout}\n{r.stderr}")


def build_oracle(force=False):
    srcs = [os.path.join(HERE, s) for s in C_SOURCES if os.path.exists(os.path.join(HERE, s))]
    if not force and os.path.exists(LIB) and all(os.path.getmtime(s) <= os.path.getmtime(LIB) for s in srcs):
        return LIB
    gcc = shutil.which("gcc")
    if gcc is None:
        raise RuntimeError("gcc not found: cannot build the CPU oracle")
    _run([gcc, "-O2", "-fopenmp", "-fPIC", "-shared", "-o", LIB] + srcs + ["-lm"])
    return LIB


EMITTED = os.path.join(HERE, "libparpy_emitted.so")


def build_emitted(force=False):
    """Compiles the hand transcription of ParPy's emitted forward program (needs
    nvcc; returns None without it)."""
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    src = os.path.join(HERE, "parpy_emitted.cu")
    if not os.path.exists(nvcc):
        return None
    if force or not os.path.exists(EMITTED) or os.path.getmtime(src) > os.path.getmtime(EMITTED):
        _run([nvcc, "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "--shared", src,
              "-o", EMITTED])
    return EMITTED


def build_reference(ref_root, force=False):
    """Compiles the reference-shipped CUDA (Trellis-generated) forward/Viterbi
    libraries. Returns the list of built files (empty if the checkout or nvcc is
    missing)."""
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    built = []
    if not ref_root or not os.path.isdir(ref_root) or not os.path.exists(nvcc):
        return built
    os.makedirs(REF_DIR, exist_ok=True)
    for k in ("5mer", "7mer"):
        src = os.path.join(ref_root, "benchmarks", k, "hmm.cu")
        out = os.path.join(REF_DIR, f"trellis_{k}.so")
        if not os.path.exists(src):
            continue
        if force or not os.path.exists(out) or os.path.getmtime(src) > os.path.getmtime(out):
            _run([nvcc, "-O3", "-gencode", "arch=compute_100,code=sm_100", "-Xcompiler", "-fPIC",
                  "--shared", src, "-o", out])
        built.append(out)
    return built


if __name__ == "__main__":
    print(build_oracle(force=True))
    print(build_emitted(force=True))
    for f in build_reference(sys.argv[1] if len(sys.argv) > 1 else reference_root(), force=True):
        print(f)
