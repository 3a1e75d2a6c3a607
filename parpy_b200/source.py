"""Source-level access to the prebuilt kernels: the reference's "inspect the
generated CUDA, tweak it, compile it yourself" workflow
(python/parpy/__init__.py:152-199, README "print_compiled / compile_string").

``kernel_source`` returns one self-contained CUDA translation unit for an
operator: the public header, the shared helpers, the runtime and the operator's
kernel file concatenated with their mutual includes removed. ``compile_source``
builds such a string with nvcc for sm_100a into a cached shared object, and
``wrapper`` calls an ``extern "C"`` entry of it with the reference's argument
flattening (python/parpy/compile.py:140-182).
"""
import ctypes
import hashlib
import os
import pathlib
import shutil
import subprocess

from .buffer import Buffer

_PKG = pathlib.Path(__file__).resolve().parent
_CSRC = _PKG / "csrc"
_HEADER = _PKG.parent / "include" / "parpy_b200.h"


def _cache_dir():
    """Where compiled strings are cached: $PARPY_B200_CACHE, else ~/.cache/parpy_b200
    (the reference uses ~/.cache/parpy, python/parpy/compile.py:4-12)."""
    return pathlib.Path(os.environ.get("PARPY_B200_CACHE", str(pathlib.Path.home() / ".cache" / "parpy_b200")))


# operator name -> kernel file
KERNEL_FILES = {
    "forward_kernel": "hmm_forward.cu",
    "softmax": "rowops.cu", "normalize_rows": "rowops.cu", "sum_exp_3d": "rowops.cu",
    "spmv_row": "sparse.cu", "spmm_cell": "sparse.cu",
    "parpy_sddmm_decompress_csr": "sparse.cu", "parpy_sddmm_csr_kernel": "sparse.cu",
    "parpy_sddmm_coo_kernel": "sparse.cu",
}
for _op in ("sum", "prod", "max", "min"):
    for _kind in ("rows", "axis", "2d"):
        KERNEL_FILES[f"{_op}_{_kind}"] = "rowops.cu"


def _strip_local_includes(text):
    keep = []
    for line in text.splitlines():
        s = line.strip()
        if s.startswith('#include "') or s == "#pragma once":
            continue
        keep.append(line)
    return "\n".join(keep) + "\n"


def kernel_source(op_name):
    """One compilable CUDA translation unit containing the kernel(s) behind
    ``op_name`` and everything they need."""
    if op_name not in KERNEL_FILES:
        raise RuntimeError(f"no kernel source registered for '{op_name}'")
    parts = [f"// parpy_b200: amalgamated source for '{op_name}' (sm_100a)\n"
             f"// build: nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -shared -Xcompiler -fPIC\n"]
    files = [_HEADER, _CSRC / "common.cuh"]
    if KERNEL_FILES[op_name].startswith("hmm_"):
        files.append(_CSRC / "cluster.cuh")
    files += [_CSRC / "runtime.cu", _CSRC / KERNEL_FILES[op_name]]
    for path in files:
        parts.append(f"\n// ======== {path.name} ========\n")
        parts.append(_strip_local_includes(path.read_text()))
    return "".join(parts)


def compile_source(code, extra_flags=()):
    """Builds CUDA source text into a shared object (cached by content hash)."""
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot compile CUDA source")
    key = hashlib.sha256((code + "\0" + " ".join(extra_flags)).encode()).hexdigest()[:32]
    cache = _cache_dir()
    cache.mkdir(parents=True, exist_ok=True)
    lib = cache / f"{key}-lib.so"
    if not lib.exists():
        src = cache / f"{key}.cu"
        src.write_text(code)
        cmd = [nvcc, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "--shared",
               "-Xcompiler", "-fPIC", *extra_flags, str(src), "-o", str(lib)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"Compilation of CUDA source failed.\nstdout:\n{r.stdout}\nstderr:\n{r.stderr}")
    return str(lib)


def clear_cache():
    cache = _cache_dir()
    if cache.exists():
        shutil.rmtree(cache)


class Scalar:
    """A 0-d array argument: passed by value in the C type of its dtype."""

    def __init__(self, ctype, value):
        self.ctype = ctype
        self.value = value


def wrapper(libpath, name):
    """A Python callable for ``extern "C" int32_t name(...)`` in ``libpath`` that
    flattens its arguments the way the reference does: dictionaries expanded in
    sorted-key order, 0-d buffers by value in their dtype, other buffers as
    pointers, Python int -> int64, float -> double; non-zero status raises with
    the library's error text."""
    lib = ctypes.CDLL(libpath)
    fn = getattr(lib, name)

    def expand(arg):
        return [v for _, v in sorted(arg.items())] if isinstance(arg, dict) else [arg]

    def ctype_and_value(arg):
        if isinstance(arg, bool) or isinstance(arg, int):
            return ctypes.c_int64, int(arg)
        if isinstance(arg, float):
            return ctypes.c_double, arg
        if isinstance(arg, Scalar):
            return arg.ctype, arg.value
        if isinstance(arg, Buffer):
            if len(arg.shape) == 0:
                return arg.dtype.to_ctype(), arg.numpy().item()
            return ctypes.c_void_p, arg._get_ptr()
        if arg is None:
            return ctypes.c_void_p, None
        raise RuntimeError(f"Argument {arg} has unsupported type {type(arg)}")

    def call(*args):
        flat = [x for a in args for x in expand(a)]
        pairs = [ctype_and_value(a) for a in flat]
        fn.argtypes = [t for t, _ in pairs]
        fn.restype = ctypes.c_int32
        status = fn(*[v for _, v in pairs])
        if status != 0:
            msg = "unknown error"
            if hasattr(lib, "parpy_get_error_message"):
                lib.parpy_get_error_message.restype = ctypes.c_char_p
                msg = lib.parpy_get_error_message().decode("ascii", "replace")
            raise RuntimeError(msg)
    call.__name__ = name
    return call
