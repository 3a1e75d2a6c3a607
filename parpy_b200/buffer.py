"""Device buffers and the host-array staging contract.

Mirrors the reference's ``parpy.buffer`` (python/parpy/buffer.py): an object
exposing ``__cuda_array_interface__`` is wrapped without a copy (:244-248); a
host array (``__array_interface__`` / ``__array__``) is copied to a fresh device
allocation and copied back into the caller's memory when the buffer is released
(:136-144, :237-260); read-only or non-contiguous memory is rejected with
``ValueError`` (:15-31). PyTorch owns the device allocations, exactly as in the
reference's CUDA buffer; the copies themselves go through torch on the current
stream.

One deliberate difference: buffers that the ``jit`` wrapper stages for the
duration of one call are written back explicitly when the call returns (and only
the arguments the operator declares as outputs), not from ``__del__``.
"""
import math

import numpy as np

from .options import CompileBackend, DataType, ElemSize


def _check_array_interface(intf):
    shape = tuple(intf["shape"])
    dtype = DataType(intf["typestr"])
    if "data" in intf and intf["data"] is not None:
        data, ro = intf["data"]
        if ro:
            raise ValueError("Cannot construct buffer from read-only memory")
    else:
        raise ValueError("Buffer protocol not supported")
    if intf.get("strides") is not None:
        raise ValueError("Buffers must only operate on contiguous memory")
    return shape, dtype, data


def _extract_array_interface(a, allow_cuda=False):
    if allow_cuda and hasattr(a, "__cuda_array_interface__"):
        return _check_array_interface(a.__cuda_array_interface__)
    if hasattr(a, "__array_interface__"):
        return _check_array_interface(a.__array_interface__)
    if hasattr(a, "__array__"):
        return _check_array_interface(a.__array__().__array_interface__)
    raise ValueError("Failed to extract array interface")


def _resolve_dtype(dtype):
    if isinstance(dtype, ElemSize):
        return DataType.from_elem_size(dtype)
    return dtype


def _require_cuda(backend):
    if backend not in (CompileBackend.Cuda, CompileBackend.Auto, None):
        raise RuntimeError(f"Backend {backend} is not available in parpy_b200 (CUDA sm_100a only)")


def sync(backend=None):
    """Waits until all queued device work has completed (python/parpy/buffer.py:72-78)."""
    _require_cuda(backend)
    from . import _native
    _native.check(_native.lib().parpy_sync(), "parpy_sync")


def _host_view(t):
    """A CPU torch tensor sharing memory with the host array ``t``."""
    import torch
    if isinstance(t, torch.Tensor):
        return t
    arr = t if isinstance(t, np.ndarray) else np.asarray(t)
    if arr.dtype in (np.uint16, np.uint32, np.uint64):
        arr = arr.view({2: np.int16, 4: np.int32, 8: np.int64}[arr.dtype.itemsize])
    return torch.from_numpy(arr)


class Buffer:
    def __init__(self, buf, shape, dtype, src=None, refcount=None):
        if type(self) is Buffer:
            raise RuntimeError("Cannot construct instance of base Buffer class")
        self.buf = buf
        self.shape = tuple(shape)
        self.dtype = _resolve_dtype(dtype)
        self.src = src
        # views made by reshape / same-width with_type share one count; the host array
        # is written back when the last of them goes (python/parpy/buffer.py:117-144)
        if refcount is None:
            self.refcount = [1]
        else:
            self.refcount = refcount
            self.refcount[0] += 1

    def __float__(self):
        if len(self.shape) == 0:
            return float(self.numpy().item())
        raise ValueError(f"Cannot convert buffer of shape {self.shape} to float")

    def __int__(self):
        if len(self.shape) == 0:
            return int(self.numpy().item())
        raise ValueError(f"Cannot convert buffer of shape {self.shape} to int")

    def __bool__(self):
        if len(self.shape) == 0:
            return bool(self.numpy().item())
        raise ValueError(f"Cannot convert buffer of shape {self.shape} to bool")

    def __index__(self):
        if len(self.shape) == 0 and self.dtype.is_integer():
            return self.__int__()
        raise ValueError(f"Cannot use buffer of shape {self.shape} and type {self.dtype} as index")

    def size(self):
        return self.dtype.size() * math.prod(self.shape)


class CudaBuffer(Buffer):
    """A contiguous device array. ``buf`` is a CUDA torch tensor (owned, or the
    caller's when wrapped zero-copy); ``src`` is the host array to copy back to."""

    backend = CompileBackend.Cuda

    def __init__(self, buf, shape, dtype, src=None, refcount=None):
        super().__init__(buf, shape, dtype, src, refcount)
        self.__cuda_array_interface__ = buf.__cuda_array_interface__

    def __del__(self):
        try:
            self.refcount[0] -= 1
            if self.refcount[0] == 0:
                self.release()
        except Exception:
            pass

    def release(self):
        """Copies the device data back into the host array this buffer was
        staged from (if any) and synchronises, once."""
        if self.src is not None:
            src, self.src = self.src, None
            _host_view(src).reshape(self.buf.shape).copy_(self.buf)
            self.sync()

    def forget_source(self):
        """Drops the host array without copying back (inputs, ignored scratch)."""
        self.src = None

    @staticmethod
    def _from_array(t):
        import torch
        try:
            shape, dtype, _ = _extract_array_interface(t, allow_cuda=True)
        except ValueError as e:
            raise ValueError(f"Cannot convert argument to a CUDA buffer: {e}")
        if hasattr(t, "__cuda_array_interface__"):
            dev = t if isinstance(t, torch.Tensor) else torch.as_tensor(t, device="cuda")
            return CudaBuffer(dev, shape, dtype)
        host = _host_view(t)
        dev = torch.empty(host.shape, dtype=host.dtype, device="cuda")
        dev.copy_(host, non_blocking=True)
        return CudaBuffer(dev, shape, dtype, src=t)

    def _get_ptr(self):
        return self.buf.data_ptr()

    def sync(self):
        sync(self.backend)

    def numpy(self):
        return np.asarray(self.buf.cpu())

    def torch(self):
        return self.buf

    def copy(self):
        return CudaBuffer(self.buf.detach().clone(), self.shape, self.dtype)

    def reshape(self, *dims):
        new_shape = tuple(dims)
        if math.prod(self.shape) != math.prod(new_shape):
            raise ValueError(f"Cannot reshape buffer of shape {self.shape} to {new_shape}")
        return CudaBuffer(self.buf.reshape(new_shape), new_shape, self.dtype, self.src, self.refcount)

    def with_type(self, new_dtype):
        new_dtype = _resolve_dtype(new_dtype)
        if not isinstance(new_dtype, DataType):
            raise ValueError(f"Found unsupported data type: {type(new_dtype)}")
        if self.dtype.size() == new_dtype.size():
            return CudaBuffer(self.buf.view(new_dtype.to_torch()), self.shape, new_dtype, self.src, self.refcount)
        t = self.buf.detach().clone().to(new_dtype.to_torch())
        return CudaBuffer(t, self.shape, new_dtype)


class DummyBuffer(Buffer):
    """Describes a host array without touching a device: what `from_array(t, None)`
    returns, used to inspect arguments where no GPU is available
    (python/parpy/buffer.py:206-228)."""

    backend = None

    def __init__(self, buf, shape, dtype, src=None, refcount=None):
        super().__init__(buf, shape, dtype, src, refcount)
        self.__array_interface__ = {"data": (buf, False), "strides": None, "typestr": str(self.dtype),
                                    "shape": self.shape, "version": 3}

    @staticmethod
    def _from_array(t):
        try:
            shape, dtype, ptr = _extract_array_interface(t, allow_cuda=True)
        except ValueError:
            raise RuntimeError(f"Cannot convert argument {t} to CPU buffer")
        return DummyBuffer(ptr, shape, dtype)

    def _get_ptr(self):
        return self.buf

    def numpy(self):
        return np.asarray(self)


def empty(shape, dtype, backend=CompileBackend.Cuda):
    import torch
    _require_cuda(backend)
    dtype = _resolve_dtype(dtype)
    return CudaBuffer(torch.empty(tuple(shape), dtype=dtype.to_torch(), device="cuda"), shape, dtype)


def zeros(shape, dtype, backend=CompileBackend.Cuda):
    import torch
    _require_cuda(backend)
    dtype = _resolve_dtype(dtype)
    return CudaBuffer(torch.zeros(tuple(shape), dtype=dtype.to_torch(), device="cuda"), shape, dtype)


def empty_like(b):
    return empty(b.shape, b.dtype, b.backend)


def zeros_like(b):
    return zeros(b.shape, b.dtype, b.backend)


def from_array(t, backend=CompileBackend.Cuda):
    """Wraps (CUDA array) or stages (host array) ``t`` as a device buffer."""
    if backend is None:
        return DummyBuffer._from_array(t)
    if backend in (CompileBackend.Cuda, CompileBackend.Auto):
        return CudaBuffer._from_array(t)
    if backend == CompileBackend.Metal:
        raise RuntimeError("The Metal backend is not available in parpy_b200")
    raise ValueError(f"Cannot convert to buffer of unknown backend {backend}")
