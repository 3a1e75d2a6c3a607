"""parpy_b200 — the reference's Python call surface over prebuilt sm_100a kernels.

Usage is the reference's (python/parpy/__init__.py): decorate the function with
``@parpy_b200.jit`` and call it with ``opts=parpy_b200.par({...})``; outputs are
written in place and the call returns ``None``. Instead of compiling the
function, ``jit`` binds it to the hand-written native kernel registered for its
name and parameter list (:mod:`parpy_b200.ops`) and raises for anything else.
Arrays exposing ``__cuda_array_interface__`` are used in place; host arrays are
staged to the device and the outputs copied back before the call returns.
"""
from . import backend
from . import buffer
from . import operators
from . import types
from .buffer import sync
from .operators import gpu, label
from .options import (CompileBackend, CompileOptions, DataType, ElemSize, LoopPar, Target, par)

__version__ = "0.1.0"

_bound = {}  # wrapper -> OpSpec


def threads(n):
    """A LoopPar over ``n`` parallel threads (python/parpy/__init__.py:138-143)."""
    return LoopPar().threads(n)


def reduce():
    """A LoopPar marking a parallelisable reduction (python/parpy/__init__.py:145-150)."""
    return LoopPar().reduce()


def clear_cache():
    """Drops cached scalar read-backs and the shared objects built by
    :func:`compile_string` (the reference removes ~/.cache/parpy here)."""
    from . import ops, source
    ops._scalar_cache.clear()
    source.clear_cache()


def _check_kwargs(kwargs, fun_name):
    # python/parpy/__init__.py:59-67,89-99
    if "opts" not in kwargs or kwargs["opts"] is None:
        raise RuntimeError(f"Missing required keyword argument opts in call to {fun_name}")
    opts = kwargs.pop("opts")
    if not isinstance(opts, CompileOptions):
        raise RuntimeError("The keyword argument opts should be of type CompileOptions")
    if len(kwargs) > 0:
        raise RuntimeError(f"Received unsupported keyword arguments: {kwargs}")
    return opts


def _role_of(spec, opts, name, key=None):
    r = spec.roles.get(name, "in")
    if key is not None:
        r = r.get(key, "in") if isinstance(r, dict) else r
    if callable(r):
        r = r(opts)
    return r


def _stage_one(arg, role, where, staged):
    """Validates one argument (python/parpy/validate.py:16-35) and moves it to
    the device according to its role."""
    from .buffer import Buffer, CudaBuffer
    if isinstance(arg, (int, float)) or arg is None:
        return arg
    if isinstance(arg, Buffer):
        return arg
    if hasattr(arg, "__cuda_array_interface__"):
        return CudaBuffer._from_array(arg)
    if hasattr(arg, "__array_interface__") or hasattr(arg, "__array__"):
        import torch
        from .buffer import _extract_array_interface, _host_view
        shape, dtype, _ = _extract_array_interface(arg)
        if role == "skip":
            return None
        host = _host_view(arg)
        if len(shape) == 0:
            # 0-d host values are passed by value; no device copy is needed
            return host.reshape(()).item()
        dev = torch.empty(host.shape, dtype=host.dtype, device="cuda")
        if role in ("in", "inout"):
            dev.copy_(host, non_blocking=True)
        b = CudaBuffer(dev, shape, dtype, src=arg if role in ("out", "inout") else None)
        if b.src is not None:
            staged.append(b)
        return b
    raise RuntimeError(f"Argument {where} has unsupported type {type(arg)}")


def _stage_arguments(spec, args, opts):
    staged = []
    out = []
    if len(args) != len(spec.params):
        raise TypeError(f"{spec.name}() takes {len(spec.params)} positional arguments "
                        f"({', '.join(spec.params)}) but {len(args)} were given")
    for i, (name, arg) in enumerate(zip(spec.params, args)):
        if isinstance(arg, dict):
            d = {}
            for k, v in arg.items():
                if not isinstance(k, str):
                    raise RuntimeError(f"Dictionary argument #{i+1} contains non-string key {k}")
                if isinstance(v, dict):
                    raise RuntimeError(f"Dictionary argument #{i+1} contains nested dictionary")
                d[k] = _stage_one(v, _role_of(spec, opts, name, k), f"#{i+1}[\"{k}\"]", staged)
            out.append(d)
        else:
            out.append(_stage_one(arg, _role_of(spec, opts, name), f"#{i+1}", staged))
    return out, staged


def jit(fun):
    """Binds ``fun`` to its native kernel. The function body is never executed
    or compiled; its name and parameter names select the kernel. Functions that
    the reference's benchmarks only use as inlined callees of a registered
    kernel are accepted and raise if called on their own."""
    import functools
    import inspect
    from . import ops
    name = fun.__name__
    params = tuple(inspect.signature(fun).parameters)
    if name in ops.HELPERS and not any(s.params == params for s in ops.REGISTRY.get(name, [])):
        @functools.wraps(fun)
        def helper(*args, **kwargs):
            raise RuntimeError(f"'{name}' is only available inlined into its native kernel")
        return helper
    spec = ops.resolve(name, params)

    @functools.wraps(fun)
    def inner(*args, **kwargs):
        opts = backend._resolve_backend(_check_kwargs(kwargs, name), True)
        dev_args, staged = _stage_arguments(spec, args, opts)
        try:
            spec.adapter(opts, *dev_args)
        except Exception:
            for b in staged:
                b.forget_source()
            raise
        for b in staged:
            b.release()
    _bound[inner] = spec
    return inner


def print_compiled(fun, args, opts=None):
    """Returns CUDA C++ source for ``fun`` (python/parpy/__init__.py:177-199). The
    reference prints what its compiler generates for the given arguments; here the
    kernels are hand-written, so this is the amalgamated source of the kernel
    file that serves ``fun`` — a complete translation unit that
    :func:`compile_string` accepts back, edited or not."""
    import inspect
    from . import ops, source
    spec = _bound.get(fun) or ops.resolve(fun.__name__, tuple(inspect.signature(fun).parameters))
    return source.kernel_source(spec.name)


def compile_string(fun_name, code, opts=None):
    """Compiles CUDA source given as a string and returns a callable for its
    ``extern "C"`` entry ``fun_name`` (python/parpy/__init__.py:161-175). The
    callable takes the arguments positionally (no ``opts``), stages host arrays
    to the device and copies every one of them back afterwards, as the
    reference's wrapper does."""
    import functools
    from . import source
    extra = tuple(getattr(opts, "extra_flags", ()) or ()) if opts is not None else ()
    fn = source.wrapper(source.compile_source(code, extra), fun_name)

    def stage(arg, where, staged):
        # 0-d host arrays travel by value in their own dtype (python/parpy/compile.py:157-170)
        if not isinstance(arg, (int, float, dict)) and not hasattr(arg, "__cuda_array_interface__") and \
                (hasattr(arg, "__array_interface__") or hasattr(arg, "__array__")):
            from .buffer import _extract_array_interface, _host_view
            shape, dtype, _ = _extract_array_interface(arg)
            if len(shape) == 0:
                return source.Scalar(dtype.to_ctype(), _host_view(arg).reshape(()).item())
        return _stage_one(arg, "inout", where, staged)

    @functools.wraps(fn)
    def inner(*args):
        staged = []
        dev_args = []
        for i, arg in enumerate(args):
            if isinstance(arg, dict):
                dev_args.append({k: stage(v, f"#{i+1}[\"{k}\"]", staged) for k, v in arg.items()})
            else:
                dev_args.append(stage(arg, f"#{i+1}", staged))
        try:
            fn(*dev_args)
        except Exception:
            for b in staged:
                b.forget_source()
            raise
        for b in staged:
            b.release()
    return inner


def external(ext_name, backend, target, header=None, parallelize=None):
    raise RuntimeError("parpy_b200 ships prebuilt kernels; external device functions are not supported")
