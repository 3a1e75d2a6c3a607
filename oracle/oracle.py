"""Python face of the CPU oracle.

TEST INFRASTRUCTURE ONLY: the checker the CUDA kernels are compared against.
Only the tests, the smoke check and the CPU-baseline leg of the benchmark may
import this module; the shipped package never does.

Parity pin: :func:`forward` (the C restatement in ``hmm_oracle.c``) and
:func:`forward_numpy` reproduce the reference's golden vectors
test/data/3mer-expected.txt and test/data/5mer-expected.txt; the CPU test suite
asserts it.
"""
import ctypes
import os

import numpy as np

from . import build as _build

_lib = None
_P = ctypes.c_void_p


def lib():
    global _lib
    if _lib is None:
        path = _build.build_oracle()
        _lib = ctypes.CDLL(path)
        _lib.oracle_forward.restype = ctypes.c_int
        _lib.oracle_forward.argtypes = [ctypes.c_float, _P, ctypes.c_int64, _P, ctypes.c_float, _P,
                                        _P, _P, _P, ctypes.c_int64, ctypes.c_int64, _P, _P,
                                        ctypes.c_int32]
        _lib.oracle_max_threads.restype = ctypes.c_int32
    return _lib


def max_threads():
    return int(lib().oracle_max_threads())


def _np(x, dtype):
    if hasattr(x, "detach"):
        x = x.detach().cpu().numpy()
    return np.ascontiguousarray(np.asarray(x), dtype=dtype)


def forward(hmm, seqs, want_alpha=False, num_threads=0):
    """C restatement of benchmarks/forward.py:94-187 on host arrays. ``hmm`` and
    ``seqs`` are the reference's dictionaries (torch or numpy values). Returns
    float32 log-likelihoods [B] (and the final alpha [B, N] when asked)."""
    n = int(hmm["num_states"])
    init = _np(hmm["initial_prob"], np.float32)
    outp = _np(hmm["output_prob"], np.float32)
    t1 = _np(hmm["trans1"], np.float32)
    t2 = _np(hmm["trans2"], np.float32)
    data = _np(seqs["data"], None)
    if data.dtype not in (np.int8, np.uint8):
        raise TypeError("observations must be int8 or uint8")
    lens = _np(seqs["lens"], np.int64)
    batch, maxlen = data.shape
    res = np.zeros(batch, dtype=np.float32)
    alpha = np.zeros((batch, n), dtype=np.float32) if want_alpha else None
    rc = lib().oracle_forward(
        float(hmm["gamma"]), init.ctypes.data, n, outp.ctypes.data, float(hmm["synthetic_248"]),
        t1.ctypes.data, t2.ctypes.data, data.ctypes.data, lens.ctypes.data, maxlen, batch,
        res.ctypes.data, alpha.ctypes.data if want_alpha else None, int(num_threads))
    if rc != 0:
        raise RuntimeError("oracle_forward rejected its arguments")
    return (res, alpha) if want_alpha else res


def forward_numpy(hmm, seqs):
    """Vectorised float32 NumPy restatement of the same algorithm
    (benchmarks/forward.py:94-187), independent of the C code: alpha is kept as
    [B, 16, K]; the five terms are summed in the order p1..p5 (:149-155); a NaN
    log-sum-exp becomes -inf through fmax (:156); sequences stop at their own
    length (:113). Small inputs only (pure NumPy)."""
    n = int(hmm["num_states"])
    K = n // 16
    f = np.float32
    t1 = _np(hmm["trans1"], f)
    t2 = _np(hmm["trans2"], f)
    outp = _np(hmm["output_prob"], f)
    init = _np(hmm["initial_prob"], f).reshape(16, K)
    gamma = f(float(hmm["gamma"]))
    syn = f(float(hmm["synthetic_248"]))
    data = _np(seqs["data"], None).view(np.uint8)
    lens = _np(seqs["lens"], np.int64)
    B = data.shape[0]
    s = np.arange(K)
    pred = (np.arange(4)[:, None] * (K // 4) + s[None, :] // 4)          # [4, K]  (:117-120)
    tr = t1[pred, s[None, :] % 4]                                          # [4, K]  (:121-124)
    c = np.zeros(16, dtype=f)
    c[14] = syn
    c[15] = gamma
    alpha = init[None, :, :] + outp[data[:, 0]][:, None, :]               # (:96-101)
    alpha = alpha.astype(f)
    with np.errstate(invalid="ignore", divide="ignore", over="ignore"):
        for t in range(1, int(lens.max())):
            live = t < lens
            if not live.any():
                break
            a = alpha[live]
            a0 = a[:, 0, :][:, pred]                                       # [b, 4, K]
            p14 = (tr[None, :, None, :] + t2[None, None, :, None]) + a0[:, :, None, :]   # (:126-129)
            nxt = np.concatenate([a[:, 1:, :], a[:, 15:, :]], axis=1)      # (:131-141)
            p5 = c[None, :, None] + nxt                                    # (:142)
            m = np.maximum(np.maximum(np.maximum(np.maximum(p14[:, 0], p14[:, 1]), p14[:, 2]),
                                      p14[:, 3]), p5)                      # (:145-148)
            ssum = (np.exp(p14[:, 0] - m) + np.exp(p14[:, 1] - m) + np.exp(p14[:, 2] - m) +
                    np.exp(p14[:, 3] - m) + np.exp(p5 - m))
            lse = np.fmax(m + np.log(ssum), f(-np.inf))                    # (:149-156)
            new = lse + outp[data[live, t]][:, None, :]                    # (:158)
            alpha[live] = new.astype(f)
        flat = alpha.reshape(B, n)
        m = flat.max(axis=1)
        res = m + np.log(np.exp(flat - m[:, None]).sum(axis=1, dtype=f))   # (:168-173)
    return res.astype(f)


# ---- reference-shipped CUDA (needs a GPU; built by oracle/build.py) -------------
def trellis_available(k):
    return os.path.exists(os.path.join(_build.REF_DIR, f"trellis_{k}mer.so"))


def trellis_forward(k, hmm, seqs):
    """Runs the reference's own CUDA implementation (benchmarks/{5,7}mer/hmm.cu,
    compiled unmodified into oracle/_ref) through the ctypes protocol of
    benchmarks/7mer/trellis.py:7-23,93-138. Host arrays in, host result out;
    needs a GPU. Its `init` uploads the tables into __device__ globals."""
    path = os.path.join(_build.REF_DIR, f"trellis_{k}mer.so")
    t = ctypes.CDLL(path)
    t1 = _np(hmm["trans1"], np.float32)
    t2 = _np(hmm["trans2"], np.float32)
    outp = _np(hmm["output_prob"], np.float32)
    init = _np(hmm["initial_prob"], np.float32)
    t.init.argtypes = [ctypes.c_float, _P, _P, _P, _P, ctypes.c_float]
    t.init.restype = None
    t.init(float(hmm["gamma"]), t1.ctypes.data, t2.ctypes.data, outp.ctypes.data, init.ctypes.data,
           float(hmm["synthetic_248"]))
    data = _np(seqs["data"], None).view(np.uint8)
    lens = _np(seqs["lens"], np.int32)
    batch, maxlen = data.shape
    t.forward.argtypes = [_P, _P, ctypes.c_int, ctypes.c_int]
    t.forward.restype = ctypes.POINTER(ctypes.c_float)
    res_ptr = t.forward(data.ctypes.data, lens.ctypes.data, maxlen, batch)
    res = np.ctypeslib.as_array(res_ptr, shape=(batch,)).copy()
    ctypes.CDLL(None).free(res_ptr)
    return res


def parpy_emitted_available():
    return os.path.exists(_build.EMITTED)


def parpy_emitted_forward(hmm, seqs, nthreads, zero_fill=True, alpha=None):
    """The CUDA program ParPy's compiler emits for benchmarks/forward.py
    ``forward_kernel`` with ``state: threads(nthreads)``, nthreads > 1024 (hand
    transcription in parpy_emitted.cu), on CUDA tensors, the way
    ``forward_parpy`` (benchmarks/forward.py:189-198) calls it: result and the two
    alpha matrices are allocated here and zero-filled by the call. Asynchronous;
    returns the result tensor. ``alpha`` may pass preallocated matrices."""
    import torch
    lib = ctypes.CDLL(_build.EMITTED)
    fn = lib.parpy_emitted_forward_kernel
    fn.restype = ctypes.c_int32
    fn.argtypes = [ctypes.c_float, _P, ctypes.c_int64, _P, ctypes.c_float, _P, _P, _P, _P, ctypes.c_int64,
                   ctypes.c_int64, _P, _P, _P, ctypes.c_int64, ctypes.c_int32]
    n = int(hmm["num_states"])
    batch, maxlen = seqs["data"].shape
    dev = lambda t: t if t.is_cuda else t.cuda()
    tables = {k: dev(hmm[k]) for k in ("initial_prob", "output_prob", "trans1", "trans2")}
    data, lens = dev(seqs["data"]).contiguous(), dev(seqs["lens"]).to(torch.int64).contiguous()
    result = torch.empty(batch, dtype=torch.float32, device="cuda")
    a1, a2 = alpha if alpha is not None else (torch.empty((batch, n), dtype=torch.float32, device="cuda"),
                                              torch.empty((batch, n), dtype=torch.float32, device="cuda"))
    # the generated code runs on the legacy default stream: order it after torch's current stream
    torch.cuda.current_stream().synchronize()
    rc = fn(float(hmm["gamma"]), tables["initial_prob"].data_ptr(), n, tables["output_prob"].data_ptr(),
            float(hmm["synthetic_248"]), tables["trans1"].data_ptr(), tables["trans2"].data_ptr(), data.data_ptr(),
            lens.data_ptr(), maxlen, batch, result.data_ptr(), a1.data_ptr(), a2.data_ptr(), int(nthreads),
            1 if zero_fill else 0)
    if rc != 0:
        raise RuntimeError(f"parpy_emitted_forward_kernel failed (code={rc})")
    torch.cuda.synchronize()
    return result


# ---- surrounding kernels ------------------------------------------------------------
def _f32(a):
    return _np(a, np.float32)


def softmax(x):
    """test/test_softmax.py:11-26 on a host array [N, M]."""
    x = _f32(x)
    out = np.empty_like(x)
    fn = lib().oracle_softmax
    fn.restype = None
    fn.argtypes = [_P, ctypes.c_int64, ctypes.c_int64, _P]
    fn(x.ctypes.data, x.shape[0], x.shape[1], out.ctypes.data)
    return out


def reduce_rows(op, x):
    """test/test_reduce.py:12-54; op in {'sum','prod','max','min'}."""
    x = _f32(x)
    out = np.empty(x.shape[0], dtype=np.float32)
    fn = lib().oracle_reduce_rows
    fn.restype = None
    fn.argtypes = [ctypes.c_int32, _P, _P, ctypes.c_int64, ctypes.c_int64]
    fn({"sum": 0, "prod": 1, "max": 2, "min": 3}[op], x.ctypes.data, out.ctypes.data, x.shape[0], x.shape[1])
    return out


def spmv(A, x, y):
    """test/test_spmv.py:12-18; returns y + A @ x for the CSR dict A."""
    values, rows, cols = _f32(A["values"]), _np(A["rows"], np.int64), _np(A["cols"], np.int64)
    x, y = _f32(x), _f32(y).copy()
    fn = lib().oracle_spmv
    fn.restype = None
    fn.argtypes = [_P, _P, _P, ctypes.c_int64, _P, _P]
    fn(values.ctypes.data, rows.ctypes.data, cols.ctypes.data, len(rows) - 1, x.ctypes.data, y.ctypes.data)
    return y


def sddmm_decompress(crows):
    crows = _np(crows, np.int64)
    rows = np.empty(int(crows[-1]), dtype=np.int64)
    fn = lib().oracle_sddmm_decompress
    fn.restype = None
    fn.argtypes = [_P, _P, ctypes.c_int64]
    fn(crows.ctypes.data, rows.ctypes.data, len(crows) - 1)
    return rows


def sddmm(A, B, rows, cols, cvalues, alpha, beta):
    """benchmarks/sddmm.py:33-41: D[i] = alpha * A[rows[i],:] . B[:,cols[i]] + beta * C[i]."""
    A, B, cvalues = _f32(A), _f32(B), _f32(cvalues)
    rows, cols = _np(rows, np.int64), _np(cols, np.int64)
    D = np.empty(len(cols), dtype=np.float32)
    fn = lib().oracle_sddmm
    fn.restype = None
    fn.argtypes = [_P, _P, _P, _P, _P, _P, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                   ctypes.c_double, ctypes.c_double]
    fn(A.ctypes.data, B.ctypes.data, rows.ctypes.data, cols.ctypes.data, cvalues.ctypes.data,
       D.ctypes.data, A.shape[1], B.shape[1], len(cols), float(alpha), float(beta))
    return D


def normalize_rows(t):
    """test/test_normalize.py:7-15; returns the normalised copy."""
    t = _f32(t).copy()
    fn = lib().oracle_normalize_rows
    fn.restype = None
    fn.argtypes = [_P, ctypes.c_int64, ctypes.c_int64]
    fn(t.ctypes.data, t.shape[0], t.shape[1])
    return t


def sum_exp_rows(x):
    """test/test_sync.py:59-69 on [rows, K]; returns (exp(x), row sums)."""
    x = _f32(x).copy()
    out = np.empty(x.shape[0], dtype=np.float32)
    fn = lib().oracle_sum_exp_rows
    fn.restype = None
    fn.argtypes = [_P, ctypes.c_int64, ctypes.c_int64, _P]
    fn(x.ctypes.data, x.shape[0], x.shape[1], out.ctypes.data)
    return x, out


def spmm(A, B, C):
    """test/test_spmm.py:16-24; returns C + A @ B for the CSR dict A and dense B."""
    values, rows, cols = _f32(A["values"]), _np(A["rows"], np.int64), _np(A["cols"], np.int64)
    B, C = _f32(B), _f32(C).copy()
    fn = lib().oracle_spmm
    fn.restype = None
    fn.argtypes = [_P, _P, _P, ctypes.c_int64, _P, ctypes.c_int64, _P]
    fn(values.ctypes.data, rows.ctypes.data, cols.ctypes.data, len(rows) - 1, B.ctypes.data, B.shape[1],
       C.ctypes.data)
    return C


# ---- Viterbi -----------------------------------------------------------------------------
def viterbi(hmm, seqs, batch_size=1024, batch_overlap=128):
    """Windowed Viterbi decoding as the reference's CUDA does it
    (benchmarks/7mer/hmm.cu:116-176,352-508,569-657). Returns a list of uint32
    state arrays, one per sequence, trimmed to the sequence's length."""
    n = int(hmm["num_states"])
    init, outp = _np(hmm["initial_prob"], np.float32), _np(hmm["output_prob"], np.float32)
    t1, t2 = _np(hmm["trans1"], np.float32), _np(hmm["trans2"], np.float32)
    data = _np(seqs["data"], None).view(np.uint8)
    lens = _np(seqs["lens"], np.int64)
    batch, maxlen = data.shape
    out = np.zeros((batch, maxlen), dtype=np.uint32)
    fn = lib().oracle_viterbi
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_float, _P, ctypes.c_int64, _P, ctypes.c_float, _P, _P, _P, _P, ctypes.c_int64,
                   ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, _P, ctypes.c_int64]
    rc = fn(float(hmm["gamma"]), init.ctypes.data, n, outp.ctypes.data, float(hmm["synthetic_248"]),
            t1.ctypes.data, t2.ctypes.data, data.ctypes.data, lens.ctypes.data, maxlen, batch,
            batch_size, batch_overlap, out.ctypes.data, maxlen)
    if rc != 0:
        raise RuntimeError("oracle_viterbi rejected its arguments")
    return [out[i, :int(lens[i])].copy() for i in range(batch)]


def trellis_viterbi(k, hmm, seqs, num_parallel=1):
    """The reference's own CUDA Viterbi (oracle/_ref), driven as
    benchmarks/7mer/trellis.py:25-83 does: observations padded to a whole number of
    windows plus the overlap, true lengths passed separately. Needs a GPU."""
    path = os.path.join(_build.REF_DIR, f"trellis_{k}mer.so")
    t = ctypes.CDLL(path)
    t1 = _np(hmm["trans1"], np.float32)
    t2 = _np(hmm["trans2"], np.float32)
    outp = _np(hmm["output_prob"], np.float32)
    init = _np(hmm["initial_prob"], np.float32)
    t.init.argtypes = [ctypes.c_float, _P, _P, _P, _P, ctypes.c_float]
    t.init.restype = None
    t.init(float(hmm["gamma"]), t1.ctypes.data, t2.ctypes.data, outp.ctypes.data, init.ctypes.data,
           float(hmm["synthetic_248"]))
    data = _np(seqs["data"], None).view(np.uint8)
    lens = _np(seqs["lens"], np.int32)
    bos, overlap = 1024 - 128, 128
    plens = (lens + bos - 1) // bos * bos + overlap
    maxlen = int(plens.max())
    padded = np.zeros((len(lens), maxlen), dtype=np.uint8)
    for i, n in enumerate(lens):
        padded[i, :n] = data[i, :n]
    padded = np.ascontiguousarray(padded.reshape(-1))
    lens = np.ascontiguousarray(lens)
    # state_t is uint16 in the 5-mer build and uint32 in the 7-mer build (hmm.cu:4)
    ctype = ctypes.c_uint16 if k == 5 else ctypes.c_uint32
    t.viterbi.argtypes = [_P, _P, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    t.viterbi.restype = ctypes.POINTER(ctype)
    ptr = t.viterbi(padded.ctypes.data, lens.ctypes.data, maxlen, int(num_parallel), len(lens))
    res = np.ctypeslib.as_array(ptr, shape=(len(lens), maxlen)).astype(np.uint32)
    ctypes.CDLL(None).free(ptr)
    return [res[i, :int(lens[i])].copy() for i in range(len(lens))]
