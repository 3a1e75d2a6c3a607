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
_scalar_cache = {}   # id(tensor) -> (weakref, version, value)


def scalar(v, what):
    """Python value of an int/float argument or of a 0-d buffer. A device-resident
    0-d tensor costs one D2H read, remembered for as long as that tensor object
    lives and is not written to (its version counter is unchanged)."""
    import weakref
    if isinstance(v, (bool, int, float)):
        return v
    if isinstance(v, Buffer):
        if len(v.shape) != 0:
            raise TypeError(f"{what}: expected a scalar, got a buffer of shape {v.shape}")
        t = v.buf
        version = getattr(t, "_version", None)
        hit = _scalar_cache.get(id(t))
        if hit is not None and hit[0]() is t and hit[1] == version and version is not None:
            return hit[2]
        val = t.item()
        if version is not None:
            if len(_scalar_cache) > 4096:
                _scalar_cache.clear()
            try:
                _scalar_cache[id(t)] = (weakref.ref(t), version, val)
            except TypeError:
                pass
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
    if t.is_cuda:
        import torch
        if t.device.index != torch.cuda.current_device():
            raise RuntimeError(f"{what}: array lives on cuda:{t.device.index} but the current device is "
                               f"cuda:{torch.cuda.current_device()}")
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
    elif mode == "scaled":
        flags |= _native.FWD_SCALED
    elif mode == "log_space":
        flags |= _native.FWD_LOG_SPACE
    elif mode != "auto":
        raise RuntimeError("opts.b200['forward'] must be 'auto', 'five_term', 'log_space', 'scaled' or "
                           f"'streaming', got {mode!r}")
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
    n_obs = int(outp.shape[0])
    rc = _native.lib().parpy_b200_forward_ex(
        gamma, ptr(init), n, ptr(outp), n_obs if n_obs <= 256 else 0, synth, ptr(t1), ptr(t2), ptr(data),
        ptr(lens), maxlen, batch, ptr(res), ptr(a1), ptr(a2), flags, current_stream())
    _native.check(rc, "forward_kernel")


_HMM_ROLES = {k: "in" for k in ("gamma", "initial_prob", "num_states", "output_prob",
                                "synthetic_248", "trans1", "trans2")}
_SEQ_ROLES = {k: "in" for k in ("data", "lens", "maxlen", "num_instances")}


def _alpha_role(opts):
    # Copied both ways when the kernel writes them: only one of alpha1 / alpha2 receives a
    # given sequence's final vector, the other keeps the caller's contents.
    return "inout" if forward_wants_alpha(opts) else "skip"


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


# ---- softmax (test/test_softmax.py:11-26) ---------------------------------------------
def _softmax_call(opts, x, N, M, out):
    import torch
    xt = tensor(x, "x", torch.float32, 2)
    ot = tensor(out, "out", torch.float32, 2)
    n, m = int(scalar(N, "N")), int(scalar(M, "M"))
    if tuple(xt.shape) != (n, m) or tuple(ot.shape) != (n, m):
        raise RuntimeError(f"softmax: x {tuple(xt.shape)} / out {tuple(ot.shape)} do not match N={n}, M={m}")
    _native.check(_native.lib().parpy_b200_softmax(ptr(xt), n, m, ptr(ot), current_stream()), "softmax")


register(OpSpec("softmax", ("x", "N", "M", "out"), {"x": "in", "out": "out"}, _softmax_call,
                doc="test/test_softmax.py:11-26"))


# ---- reductions (test/test_reduce.py:12-70) --------------------------------------------
def _reduce_call(op, full):
    def call(opts, x, out, N):
        import torch
        xt = tensor(x, "x", torch.float32, 2)
        ot = tensor(out, "out", torch.float32, 1)
        n = int(scalar(N, "N"))
        # row / axis reductions write all of `out` (a host `out` is staged without its old
        # contents and copied back whole), so its length must be N exactly
        if xt.shape[0] != n or (ot.shape[0] < 1 if full else ot.shape[0] != n):
            raise RuntimeError(f"reduce: x {tuple(xt.shape)} / out {tuple(ot.shape)} do not match N={n}")
        rows, width = (1, xt.numel()) if full else (n, xt.shape[1])
        _native.check(_native.lib().parpy_b200_reduce_rows(op, ptr(xt), ptr(ot), rows, width,
                                                           current_stream()), "reduce")
    return call


for _i, _op in enumerate(("sum", "prod", "max", "min")):
    for _suffix in ("rows", "axis"):
        register(OpSpec(f"{_op}_{_suffix}", ("x", "out", "N"), {"x": "in", "out": "out"},
                        _reduce_call(_i, False), doc="test/test_reduce.py:12-54"))
    # the full reductions write out[0] only; the rest of `out` keeps the caller's values
    register(OpSpec(f"{_op}_2d", ("x", "out", "N"), {"x": "in", "out": "inout"},
                    _reduce_call(_i, True), doc="test/test_reduce.py:56-70"))


# ---- CSR SpMV (test/test_spmv.py:12-18) ---------------------------------------------------
def _spmv_call(opts, A, x, y):
    import torch
    i64 = torch.int64
    values = tensor(A["values"], "A['values']", torch.float32, 1)
    rows = tensor(A["rows"], "A['rows']", i64, 1)
    cols = tensor(A["cols"], "A['cols']", i64, 1)
    nrows = int(scalar(A["nrows"], "A['nrows']"))
    xt = tensor(x, "x", torch.float32, 1)
    yt = tensor(y, "y", torch.float32, 1)
    if rows.shape[0] != nrows + 1 or yt.shape[0] != nrows or cols.shape[0] != values.shape[0]:
        raise RuntimeError(f"spmv_row: rows {tuple(rows.shape)}, cols {tuple(cols.shape)}, values "
                           f"{tuple(values.shape)}, y {tuple(yt.shape)} do not match nrows={nrows}")
    _native.check(_native.lib().parpy_b200_spmv(ptr(values), ptr(rows), ptr(cols), nrows,
                                                values.shape[0], ptr(xt), ptr(yt), current_stream()),
                  "spmv_row")


register(OpSpec("spmv_row", ("A", "x", "y"),
                {"A": {"values": "in", "rows": "in", "cols": "in", "nrows": "in"}, "x": "in", "y": "inout"},
                _spmv_call, doc="test/test_spmv.py:12-18"))


# ---- SDDMM (benchmarks/sddmm.py:21-41,63-70) -------------------------------------------------
def _sddmm_decompress_call(opts, C_crows, C_rows, N):
    import torch
    crows = tensor(C_crows, "C_crows", torch.int64, 1)
    rows = tensor(C_rows, "C_rows", torch.int64, 1)
    n = int(scalar(N, "N"))
    if crows.shape[0] != n + 1:
        raise RuntimeError(f"parpy_sddmm_decompress_csr: crows {tuple(crows.shape)} does not match N={n}")
    _native.check(_native.lib().parpy_b200_sddmm_decompress_csr(ptr(crows), ptr(rows), n, current_stream()),
                  "parpy_sddmm_decompress_csr")


def _sddmm_operands(A, B, C, D):
    import torch
    At = tensor(A, "A", torch.float32, 2)
    Bt = tensor(B, "B", torch.float32, 2)
    cols = tensor(C["cols"], "C['cols']", torch.int64, 1)
    vals = tensor(C["values"], "C['values']", torch.float32, 1)
    Dt = tensor(D, "D", torch.float32, 1)
    nnz = int(scalar(C["nnz"], "C['nnz']"))
    if At.shape[1] != Bt.shape[0] or cols.shape[0] != nnz or vals.shape[0] != nnz or Dt.shape[0] != nnz:
        raise RuntimeError(f"sddmm: A {tuple(At.shape)}, B {tuple(Bt.shape)}, cols {tuple(cols.shape)}, "
                           f"values {tuple(vals.shape)}, D {tuple(Dt.shape)} do not match nnz={nnz}")
    return At, Bt, cols, vals, Dt, nnz


def _sddmm_csr_call(opts, A, B, C, D, N, alpha, beta):
    import torch
    At, Bt, cols, vals, Dt, nnz = _sddmm_operands(A, B, C, D)
    crows = tensor(C["crows"], "C['crows']", torch.int64, 1)
    rows = tensor(C["rows"], "C['rows']", torch.int64, 1)
    n = int(scalar(N, "N"))
    if crows.shape[0] != n + 1 or rows.shape[0] != nnz or At.shape[0] != n:
        raise RuntimeError(f"parpy_sddmm_csr_kernel: crows {tuple(crows.shape)} / rows {tuple(rows.shape)} "
                           f"do not match N={n}, nnz={nnz}")
    _native.check(_native.lib().parpy_b200_sddmm_csr(
        ptr(At), ptr(Bt), ptr(crows), ptr(rows), ptr(cols), ptr(vals), ptr(Dt), n, At.shape[1],
        Bt.shape[1], nnz, float(scalar(alpha, "alpha")), float(scalar(beta, "beta")), current_stream()),
        "parpy_sddmm_csr_kernel")


def _sddmm_coo_call(opts, A, B, C, D, alpha, beta):
    import torch
    At, Bt, cols, vals, Dt, nnz = _sddmm_operands(A, B, C, D)
    rows = tensor(C["rows"], "C['rows']", torch.int64, 1)
    if rows.shape[0] != nnz:
        raise RuntimeError(f"parpy_sddmm_coo_kernel: rows {tuple(rows.shape)} does not match nnz={nnz}")
    _native.check(_native.lib().parpy_b200_sddmm_coo(
        ptr(At), ptr(Bt), ptr(rows), ptr(cols), ptr(vals), ptr(Dt), At.shape[1], Bt.shape[1], nnz,
        float(scalar(alpha, "alpha")), float(scalar(beta, "beta")), current_stream()),
        "parpy_sddmm_coo_kernel")


register(OpSpec("parpy_sddmm_decompress_csr", ("C_crows", "C_rows", "N"),
                {"C_crows": "in", "C_rows": "out"}, _sddmm_decompress_call,
                doc="benchmarks/sddmm.py:21-26"))
register(OpSpec("parpy_sddmm_csr_kernel", ("A", "B", "C", "D", "N", "alpha", "beta"),
                {"A": "in", "B": "in", "D": "out",
                 "C": {"crows": "in", "rows": "out", "cols": "in", "values": "in", "nnz": "in"}},
                _sddmm_csr_call, doc="benchmarks/sddmm.py:28-41"))
register(OpSpec("parpy_sddmm_coo_kernel", ("A", "B", "C", "D", "alpha", "beta"),
                {"A": "in", "B": "in", "D": "out",
                 "C": {"rows": "in", "cols": "in", "values": "in", "nnz": "in"}},
                _sddmm_coo_call, doc="benchmarks/sddmm.py:63-70"))


# ---- row normalisation, exp + row sum, SpMM (test_normalize.py, test_sync.py, test_spmm.py) ----
def _normalize_call(opts, t, nrows, ncols):
    import torch
    tt = tensor(t, "t", torch.float32, 2)
    n, m = int(scalar(nrows, "nrows")), int(scalar(ncols, "ncols"))
    if tuple(tt.shape) != (n, m):
        raise RuntimeError(f"normalize_rows: t {tuple(tt.shape)} does not match nrows={n}, ncols={m}")
    _native.check(_native.lib().parpy_b200_normalize_rows(ptr(tt), n, m, current_stream()), "normalize_rows")


def _sum_exp_3d_call(opts, x, N, M, out):
    import torch
    xt = tensor(x, "x", torch.float32, 3)
    ot = tensor(out, "out", torch.float32, 2)
    n, m = int(scalar(N, "N")), int(scalar(M, "M"))
    if tuple(xt.shape[:2]) != (n, m) or tuple(ot.shape) != (n, m):
        raise RuntimeError(f"sum_exp_3d: x {tuple(xt.shape)} / out {tuple(ot.shape)} do not match N={n}, M={m}")
    _native.check(_native.lib().parpy_b200_sum_exp_rows(ptr(xt), n * m, xt.shape[2], ptr(ot), current_stream()),
                  "sum_exp_3d")


def _spmm_call(opts, A, B, C):
    import torch
    values = tensor(A["values"], "A['values']", torch.float32, 1)
    rows = tensor(A["rows"], "A['rows']", torch.int64, 1)
    cols = tensor(A["cols"], "A['cols']", torch.int64, 1)
    nrows = int(scalar(A["nrows"], "A['nrows']"))
    Bv = tensor(B["values"], "B['values']", torch.float32, 2)
    ncols = int(scalar(B["ncols"], "B['ncols']"))
    Ct = tensor(C, "C", torch.float32, 2)
    if rows.shape[0] != nrows + 1 or Bv.shape[1] != ncols or tuple(Ct.shape) != (nrows, ncols):
        raise RuntimeError(f"spmm_cell: rows {tuple(rows.shape)}, B {tuple(Bv.shape)}, C {tuple(Ct.shape)} "
                           f"do not match nrows={nrows}, ncols={ncols}")
    _native.check(_native.lib().parpy_b200_spmm(ptr(values), ptr(rows), ptr(cols), nrows, ptr(Bv), ncols,
                                                ptr(Ct), current_stream()), "spmm_cell")


register(OpSpec("normalize_rows", ("t", "nrows", "ncols"), {"t": "inout"}, _normalize_call,
                doc="test/test_normalize.py:7-15"))
register(OpSpec("sum_exp_3d", ("x", "N", "M", "out"), {"x": "inout", "out": "out"}, _sum_exp_3d_call,
                doc="test/test_sync.py:59-69"))
register(OpSpec("spmm_cell", ("A", "B", "C"),
                {"A": {"values": "in", "rows": "in", "cols": "in", "nrows": "in"},
                 "B": {"values": "in", "ncols": "in"}, "C": "inout"},
                _spmm_call, doc="test/test_spmm.py:16-24"))
