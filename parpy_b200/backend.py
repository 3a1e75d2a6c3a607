"""Backend availability and resolution (python/parpy/backend.py). Only CUDA on
a compute-capability 10.x device exists here; ``Auto`` resolves to it and Metal
is always reported as unavailable."""
import os

from .options import CompileBackend

backends = [CompileBackend.Cuda]


def _assert_cuda_is_enabled():
    import torch
    from . import _native
    if not torch.cuda.is_available():
        raise RuntimeError("No CUDA device is visible to torch")
    if not os.path.exists(_native.LIB_PATH):
        raise RuntimeError(f"{_native.LIB_PATH} has not been built")
    major, minor = torch.cuda.get_device_capability()
    if major < 10:
        raise RuntimeError(f"parpy_b200 kernels need compute capability 10.x, found {major}.{minor}")


def is_enabled(backend, verbose=False):
    try:
        if backend == CompileBackend.Cuda:
            _assert_cuda_is_enabled()
        elif backend == CompileBackend.Metal:
            raise RuntimeError("The Metal backend does not exist in parpy_b200")
        else:
            raise RuntimeError(f"Unsupported backend {backend}")
        return True
    except RuntimeError as e:
        if verbose:
            print(f"Backend {backend} is not enabled: {e}")
        return False


def _resolve_backend(opts, strict):
    """Turns ``Auto`` into ``Cuda``; with ``strict`` the backend must be usable
    now (python/parpy/backend.py:49-77)."""
    if opts.verbose_backend_resolution:
        for b in backends:
            is_enabled(b, True)
    if opts.backend == CompileBackend.Auto:
        if strict and not is_enabled(CompileBackend.Cuda):
            raise RuntimeError("Found no enabled GPU backends. For detailed information on why "
                               "this is, enable the 'verbose_backend_resolution' flag in the "
                               "compiler options.")
        opts.backend = CompileBackend.Cuda
        return opts
    if opts.backend != CompileBackend.Cuda or (strict and not is_enabled(opts.backend)):
        raise RuntimeError(f"Specified backend {opts.backend} is not available. For more "
                           "information, enable the 'verbose_backend_resolution' flag in the "
                           "compiler options.")
    return opts
