"""The HMM forward call surface of the reference's benchmark
(benchmarks/forward.py:175-198), bound to the native kernels.

``forward_kernel`` keeps the reference's signature and in-place semantics;
``forward_parpy`` is the benchmark's convenience wrapper. The native resident
kernel keeps alpha on chip, so the two [B, num_states] scratch matrices the
reference allocates and zero-fills on every call are optional here.
"""
from . import jit, par, threads
from .options import CompileOptions


@jit
def forward_kernel(hmm, seqs, result, alpha1, alpha2):
    """result[i] = log-likelihood of sequence i under the k-mer/duration HMM.
    Bound to the native kernel; this body is never run."""


def forward_parpy(hmm, seqs, nthreads=None, opts=None, alpha=None):
    """benchmarks/forward.py:189-198: allocates ``result`` on the device, runs
    the forward algorithm and returns it. ``nthreads`` is the reference's tuning
    knob for the 'state' label; the native kernel chooses its own mapping, so it
    is recorded in the options and otherwise ignored. ``alpha`` may be a pair of
    [B, num_states] float32 device tensors when the final alpha vectors are
    wanted (``opts.b200['write_alpha']``) or the streaming kernel is forced."""
    import torch
    batch = seqs["num_instances"]
    batch = int(batch.item()) if hasattr(batch, "item") else int(batch)
    result = torch.zeros(batch, dtype=torch.float32, device="cuda")
    if opts is None:
        p = {"inst": threads(batch)}
        if nthreads:
            p["state"] = threads(int(nthreads))
        opts = par(p)
    elif not isinstance(opts, CompileOptions):
        raise RuntimeError("opts must be a CompileOptions")
    a1, a2 = alpha if alpha is not None else (None, None)
    forward_kernel(hmm, seqs, result, a1, a2, opts=opts)
    return result


def to_device(tables, device="cuda", pin=False):
    """Moves every array of an ``hmm`` / ``seqs`` dictionary to ``device``; 0-d
    entries stay on the host (they are read by value anyway)."""
    import torch
    out = {}
    for k, v in tables.items():
        if isinstance(v, torch.Tensor) and v.dim() > 0:
            out[k] = v.pin_memory() if pin else v.to(device)
        else:
            out[k] = v
    return out


def _hdf5_access():
    """(open, read-dataset) functions: h5py when installed, else the package's reader."""
    try:
        import h5py
        return (lambda p: h5py.File(p, "r")), (lambda ds: ds[:])
    except ImportError:
        from .hdf5_min import H5File
        return H5File, (lambda ds: ds.read())


def read_model(model_path):
    """Model half of the reference's loader (benchmarks/forward.py:43-72) with the
    table work on the device: uploads the raw probability tables once and builds
    the log tables, the base-reversal permuted emission matrix, the transposed
    transition table and the initial distribution with one kernel. Returns the
    ``hmm`` dictionary with CUDA tensors (0-d entries included)."""
    import ctypes
    import numpy as np
    import torch
    from . import _native
    opener, read = _hdf5_access()
    f = opener(model_path)
    tables = f["Tables"]
    obs = np.ascontiguousarray(read(tables["ObservationProbabilities"]))
    trans = np.ascontiguousarray(read(tables["TransitionProbabilities"]))
    dur = np.ascontiguousarray(read(tables["DurationProbabilities"]))
    tail = np.log(tables["DurationProbabilities"].attrs["TailFactor"])       # forward.py:48
    k = int(f["Parameters"].attrs["KMerLength"])
    K = 4 ** k
    is_f64 = obs.dtype == np.float64
    want = np.float64 if is_f64 else np.float32
    d_obs, d_trans, d_dur = (torch.from_numpy(a.astype(want, copy=False)).cuda() for a in (obs, trans, dur))
    n_obs = obs.shape[0]
    out_prob = torch.empty((n_obs, K), dtype=torch.float32, device="cuda")
    trans1 = torch.empty((K, 4), dtype=torch.float32, device="cuda")
    trans2 = torch.empty(16, dtype=torch.float32, device="cuda")
    init = torch.empty(16 * K, dtype=torch.float32, device="cuda")
    P = ctypes.c_void_p
    _native.check(_native.lib().parpy_b200_hmm_prepare_tables(
        P(d_obs.data_ptr()), P(d_trans.data_ptr()), P(d_dur.data_ptr()), int(is_f64), k, n_obs,
        P(out_prob.data_ptr()), P(trans1.data_ptr()), P(trans2.data_ptr()), P(init.data_ptr()),
        P(torch.cuda.current_stream().cuda_stream)), "hmm_prepare_tables")
    synthetic_248 = np.log(np.exp(0.0) - np.exp(tail))                      # forward.py:56
    return {
        "gamma": torch.tensor(tail, dtype=torch.float32, device="cuda"),
        "trans1": trans1, "trans2": trans2, "output_prob": out_prob, "initial_prob": init,
        "synthetic_248": torch.tensor(synthetic_248, dtype=torch.float32, device="cuda"),
        "num_states": torch.tensor(16 * K, dtype=torch.int64, device="cuda"),
    }


def read_signals(signals_path):
    """Signal half of the reference's loader (benchmarks/forward.py:53-55,74-86):
    one upload of the concatenated int16 signals, padded int8 matrix and lengths
    built on the device. Returns the ``seqs`` dictionary with CUDA tensors."""
    import ctypes
    import numpy as np
    import torch
    from . import _native
    opener, read = _hdf5_access()
    s = opener(signals_path)
    keys = sorted(s.keys())
    signals = [np.asarray(read(s[key]["Raw"]["Signal"]), dtype=np.int16) for key in keys]
    offsets = np.zeros(len(signals) + 1, dtype=np.int64)
    np.cumsum([len(x) for x in signals], out=offsets[1:])
    maxlen = int(max(len(x) for x in signals))
    flat = torch.from_numpy(np.concatenate(signals)).cuda()
    d_off = torch.from_numpy(offsets).cuda()
    data = torch.empty((len(signals), maxlen), dtype=torch.int8, device="cuda")
    lens = torch.empty(len(signals), dtype=torch.int64, device="cuda")
    P = ctypes.c_void_p
    _native.check(_native.lib().parpy_b200_hmm_pad_signals(
        P(flat.data_ptr()), P(d_off.data_ptr()), len(signals), maxlen, P(data.data_ptr()),
        P(lens.data_ptr()), P(torch.cuda.current_stream().cuda_stream)), "hmm_pad_signals")
    return {
        "data": data, "lens": lens,
        "maxlen": torch.tensor(maxlen, dtype=torch.int64, device="cuda"),
        "num_instances": torch.tensor(len(signals), dtype=torch.int64, device="cuda"),
    }


def read_trellis_inputs(model_path, signals_path):
    """benchmarks/forward.py:40-87: ``(hmm, seqs)`` for a model file and a signal file."""
    return read_model(model_path), read_signals(signals_path)


def viterbi(hmm, seqs, batch_size=1024, batch_overlap=128):
    """Most likely state path of every sequence (windowed Viterbi with the
    semantics of benchmarks/7mer/trellis.py:25-83 and benchmarks/7mer/hmm.cu).
    ``hmm`` and ``seqs`` are the dictionaries ``forward_kernel`` takes, on the
    device. Returns a uint32-valued int64 CUDA tensor [B, maxlen] whose row i holds
    ``lens[i]`` decoded states, and the lengths; use ``viterbi_paths`` for a list
    of per-sequence NumPy arrays."""
    import ctypes
    import torch
    from . import _native
    from .buffer import from_array
    from .ops import scalar
    n = int(scalar(from_array(hmm["num_states"]), "num_states")) if hasattr(hmm["num_states"], "shape") else int(hmm["num_states"])
    data, lens = seqs["data"], seqs["lens"]
    if lens.dtype != torch.int64:
        lens = lens.to(torch.int64)
    batch, maxlen = data.shape
    out = torch.zeros((batch, maxlen), dtype=torch.int32, device=data.device)
    P = ctypes.c_void_p
    rc = _native.lib().parpy_b200_viterbi(
        float(hmm["gamma"]), P(hmm["initial_prob"].data_ptr()), n, P(hmm["output_prob"].data_ptr()),
        float(hmm["synthetic_248"]), P(hmm["trans1"].data_ptr()), P(hmm["trans2"].data_ptr()),
        P(data.data_ptr()), P(lens.data_ptr()), maxlen, batch, batch_size, batch_overlap,
        P(out.data_ptr()), maxlen, P(torch.cuda.current_stream().cuda_stream))
    _native.check(rc, "viterbi")
    return out, lens


def viterbi_paths(hmm, seqs, batch_size=1024, batch_overlap=128):
    """``viterbi`` with the result trimmed per sequence, as the reference's wrapper
    returns it (benchmarks/7mer/trellis.py:64-66): a list of uint32 NumPy arrays."""
    import numpy as np
    out, lens = viterbi(hmm, seqs, batch_size, batch_overlap)
    host, hl = out.cpu().numpy().view(np.uint32), lens.cpu().numpy()
    return [host[i, :int(hl[i])].copy() for i in range(host.shape[0])]
