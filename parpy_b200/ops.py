"""Registry that maps the reference's jit-decorated Python functions to the
prebuilt native kernels.

The reference compiles whatever function it is given; this package ships
hand-written kernels for a fixed set of functions and resolves a decorated
function by its name and parameter names. Each entry lists, per parameter (and
per dictionary key), how the argument is staged when the caller passes host
memory:

  in      copied to the device, never copied back
  out     device allocation only, copied back after the call
  inout   copied both ways
  skip    not staged at all (scratch the native kernel ignores)

and an adapter that flattens the arguments the way the reference's ctypes
wrapper does (python/parpy/compile.py:140-178) and calls the C ABI on torch's
current stream.
"""
import ctypes

from . import _native
from .buffer import Buffer


class OpSpec:
    def __init__(self, name, params, roles, adapter, doc=""):
        self.name = name
        self.params = tuple(params)
        self.roles = roles          # param -> role, or param -> {key -> role} for dict args
        self.adapter = adapter
        self.doc = doc


REGISTRY = {}   # name -> [OpSpec]
HELPERS = set()  # jit-decorated callees that only exist inlined into a registered kernel


def register(spec):
    REGISTRY.setdefault(spec.name, []).append(spec)


def resolve(name, params):
    """Finds the native operator for a decorated function, or raises: there is
    no interpreter or CPU fallback behind this package."""
    for spec in REGISTRY.get(name, []):
        if spec.params == tuple(params):
            return spec
    known = ", ".join(sorted(f"{n}({', '.join(s.params)})" for n, v in REGISTRY.items() for s in v))
    raise RuntimeError(
        f"parpy_b200 has no native kernel for function '{name}({', '.join(params)})'. "
        f"This package does not compile Python; it provides: {known}")


# ---- argument helpers -------------------------------------------------------
_scalar_cache = {}


def scalar(v, what):
    """Python value of an int/float argument or of a 0-d buffer. Device-resident
    0-d tensors cost one D2H read, cached per (pointer, version)."""
    if isinstance(v, (bool, int, float)):
        return v
    if isinstance(v, Buffer):
        if len(v.shape) != 0:
            raise TypeError(f"{what}: expected a scalar, got a buffer of shape {v.shape}")
        t = v.buf
        key = (t.data_ptr(), getattr(t, "_version", None), t.dtype)
        if key[1] is not None and key in _scalar_cache:
            return _scalar_cache[key]
        val = t.item()
        if key[1] is not None:
            if len(_scalar_cache) > 4096:
                _scalar_cache.clear()
            _scalar_cache[key] = val
        return val
    raise TypeError(f"{what}: expected an int, float or 0-d array, got {type(v)}")


def tensor(v, what, dtype=None, ndim=None, allow_none=False):
    """The CUDA torch tensor behind a buffer argument, with dtype/rank checks."""
    if v is None:
        if allow_none:
            return None
        raise TypeError(f"{what}: missing array argument")
    if not isinstance(v, Buffer):
        raise TypeError(f"{what}: expected an array, got {type(v)}")
    t = v.buf
    if dtype is not None:
        dts = dtype if isinstance(dtype, (tuple, list)) else (dtype,)
        if t.dtype not in dts:
            raise TypeError(f"{what}: expected dtype {' or '.join(map(str, dts))}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise TypeError(f"{what}: expected a {ndim}-d array, got shape {tuple(t.shape)}")
    return t


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def current_stream():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# ---- HMM forward ---------------------------------------------------------------
def _forward_flags(opts):
    b = getattr(opts, "b200", None) or {}
    flags = _native.FWD_AUTO
    mode = b.get("forward", "auto")
    if mode == "streaming":
        flags |= _native.FWD_STREAMING
    elif mode == "five_term":
        flags |= _native.FWD_FIVE_TERM
    elif mode != "auto":
        raise RuntimeError(f"opts.b200['forward'] must be 'auto', 'five_term' or 'streaming', got {mode!r}")
    if b.get("write_alpha", False):
        flags |= _native.FWD_WRITE_ALPHA
    return flags


def forward_wants_alpha(opts):
    return _forward_flags(opts) & (_native.FWD_STREAMING | _native.FWD_WRITE_ALPHA) != 0


def _forward_call(opts, hmm, seqs, result, alpha1, alpha2):
    import torch
    n = int(scalar(hmm["num_states"], "hmm['num_states']"))
    maxlen = int(scalar(seqs["maxlen"], "seqs['maxlen']"))
    batch = int(scalar(seqs["num_instances"], "seqs['num_instances']"))
    gamma = float(scalar(hmm["gamma"], "hmm['gamma']"))
    synth = float(scalar(hmm["synthetic_248"], "hmm['synthetic_248']"))
    f32 = torch.float32
    init = tensor(hmm["initial_prob"], "hmm['initial_prob']", f32, 1)
    outp = tensor(hmm["output_prob"], "hmm['output_prob']", f32, 2)
    t1 = tensor(hmm["trans1"], "hmm['trans1']", f32, 2)
    t2 = tensor(hmm["trans2"], "hmm['trans2']", f32, 1)
    data = tensor(seqs["data"], "seqs['data']", (torch.int8, torch.uint8), 2)
    lens = tensor(seqs["lens"], "seqs['lens']", (torch.int64, torch.int32), 1)
    res = tensor(result, "result", f32, 1)
    a1 = tensor(alpha1, "alpha1", f32, 2, allow_none=True)
    a2 = tensor(alpha2, "alpha2", f32, 2, allow_none=True)
    if n < 64 or n % 64 != 0:
        raise RuntimeError(f"forward_kernel: num_states={n} must be a positive multiple of 64")
    k = n // 16
    if init.shape[0] != n or tuple(t1.shape) != (k, 4) or t2.shape[0] != 16 or outp.shape[1] != k:
        raise RuntimeError(
            f"forward_kernel: table shapes {tuple(init.shape)}, {tuple(t1.shape)}, {tuple(t2.shape)}, "
            f"{tuple(outp.shape)} do not match num_states={n}")
    if tuple(data.shape) != (batch, maxlen) or lens.shape[0] != batch or res.shape[0] != batch:
        raise RuntimeError(
            f"forward_kernel: data {tuple(data.shape)}, lens {tuple(lens.shape)}, result "
            f"{tuple(res.shape)} do not match num_instances={batch}, maxlen={maxlen}")
    for a, nm in ((a1, "alpha1"), (a2, "alpha2")):
        if a is not None and tuple(a.shape) != (batch, n):
            raise RuntimeError(f"forward_kernel: {nm} has shape {tuple(a.shape)}, expected {(batch, n)}")
    if lens.dtype != torch.int64:
        lens = lens.to(torch.int64)
    flags = _forward_flags(opts)
    rc = _native.lib().parpy_b200_forward(
        gamma, ptr(init), n, ptr(outp), synth, ptr(t1), ptr(t2), ptr(data), ptr(lens), maxlen,
        batch, ptr(res), ptr(a1), ptr(a2), flags, current_stream())
    _native.check(rc, "forward_kernel")


_HMM_ROLES = {k: "in" for k in ("gamma", "initial_prob", "num_states", "output_prob",
                                "synthetic_248", "trans1", "trans2")}
_SEQ_ROLES = {k: "in" for k in ("data", "lens", "maxlen", "num_instances")}


def _alpha_role(opts):
    return "out" if forward_wants_alpha(opts) else "skip"


register(OpSpec(
    "forward_kernel", ("hmm", "seqs", "result", "alpha1", "alpha2"),
    {"hmm": _HMM_ROLES, "seqs": _SEQ_ROLES, "result": "out", "alpha1": _alpha_role, "alpha2": _alpha_role},
    lambda opts, hmm, seqs, result, alpha1, alpha2: _forward_call(opts, hmm, seqs, result, alpha1, alpha2),
    doc="benchmarks/forward.py:175-187"))

register(OpSpec(
    "forward_kernel", ("hmm", "seqs", "alpha1", "alpha2", "result"),
    {"hmm": _HMM_ROLES, "seqs": _SEQ_ROLES, "result": "out", "alpha1": _alpha_role, "alpha2": _alpha_role},
    lambda opts, hmm, seqs, alpha1, alpha2, result: _forward_call(opts, hmm, seqs, result, alpha1, alpha2),
    doc="test/test_forward.py:83-160"))

# Callees of forward_kernel in the benchmark; the native kernel contains them.
HELPERS.update({"forward_init_inst", "forward_step_inst", "forward_lse_inst"})
