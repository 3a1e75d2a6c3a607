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
    Bound to the native kernel; this body is never run.

    ``opts.b200 = {"forward": mode}`` chooses the arithmetic: ``"auto"``
    (default: the scaled kernel for 4096 k-mers and more, the log-space kernel
    below that and whenever alpha is requested), ``"log_space"``, ``"scaled"``,
    ``"five_term"`` (the reference's literal operand order) or ``"streaming"``
    (one launch per time step, alpha in the caller's scratch);
    ``{"write_alpha": True}`` stores every sequence's final alpha vector in
    ``alpha1`` / ``alpha2`` as the reference leaves it."""


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


def forward_schedule(lens, clusters):
    """The static schedule the forward kernels build for a batch (at most 4096
    sequences): a NumPy int32 array giving, for every sequence, the resident
    cluster that scores it. ``lens`` are the sequence lengths (any integer array
    or tensor), ``clusters`` the number of resident clusters (see
    ``parpy_b200_forward_plan``). A launch lasts as long as its busiest cluster,
    i.e. as the largest per-cluster sum of lengths."""
    import ctypes
    import torch
    from . import _native
    t = torch.as_tensor(lens).to(torch.int64).cuda().contiguous()
    out = torch.empty(t.numel(), dtype=torch.int32, device="cuda")
    P = ctypes.c_void_p
    _native.check(_native.lib().parpy_b200_forward_schedule(
        P(t.data_ptr()), t.numel(), int(clusters), P(out.data_ptr()),
        P(torch.cuda.current_stream().cuda_stream)), "forward_schedule")
    return out.cpu().numpy()


def forward_status():
    """Reads and clears the forward kernels' device status word (synchronises the
    device). Returns ``{"length_clamped": bool, "observation_clamped": bool,
    "wait_timed_out": bool}``: a sequence length outside [1, maxlen], or an
    observation byte that is not a row of ``output_prob``, was met (and clamped)
    by a call since the last read; or a bounded wait for another CTA's values ran
    out inside a kernel, in which case the results of those calls are not valid."""
    import ctypes
    from . import _native
    st = ctypes.c_uint32(0)
    _native.check(_native.lib().parpy_b200_forward_status(ctypes.byref(st)), "forward_status")
    return {"length_clamped": bool(st.value & 1), "observation_clamped": bool(st.value & 2),
            "wait_timed_out": bool(st.value & 4)}


def viterbi_status():
    """Reads and clears the Viterbi kernel's device status word (synchronises the
    device). Returns ``{"wait_timed_out": bool, "observation_clamped": bool}``."""
    import ctypes
    from . import _native
    st = ctypes.c_uint32(0)
    _native.check(_native.lib().parpy_b200_viterbi_status(ctypes.byref(st)), "viterbi_status")
    return {"wait_timed_out": bool(st.value & 1), "observation_clamped": bool(st.value & 2)}


def viterbi(hmm, seqs, batch_size=1024, batch_overlap=128, check=True):
    """Most likely state path of every sequence (windowed Viterbi with the
    semantics of benchmarks/7mer/trellis.py:25-83 and benchmarks/7mer/hmm.cu).
    ``hmm`` and ``seqs`` are the dictionaries ``forward_kernel`` takes, as
    contiguous CUDA tensors on the current device (float32 tables, int8/uint8
    observations). Returns an int32 CUDA tensor [B, maxlen] whose row i holds
    ``lens[i]`` decoded states (read it as uint32: state = layer * K + kmer), and
    the int64 lengths; use ``viterbi_paths`` for a list of per-sequence NumPy
    arrays. With ``check`` (default) the call waits for the kernel and raises
    ``RuntimeError`` if one of its bounded waits ran out, in which case the paths
    are not valid; ``check=False`` leaves the call asynchronous and the status to
    :func:`viterbi_status`. Back-pointer scratch of up to 6 GiB per (device,
    stream) is kept by the library between calls."""
    import torch
    from . import _native
    from .buffer import from_array
    from .ops import current_stream, ptr, scalar, tensor
    as_scalar = lambda v, what: scalar(from_array(v), what) if hasattr(v, "shape") else v
    n = int(as_scalar(hmm["num_states"], "hmm['num_states']"))
    gamma = float(as_scalar(hmm["gamma"], "hmm['gamma']"))
    synth = float(as_scalar(hmm["synthetic_248"], "hmm['synthetic_248']"))
    f32 = torch.float32

    def dev(v, what, dtype, ndim):
        if not (isinstance(v, torch.Tensor) and v.is_cuda):
            raise TypeError(f"viterbi: {what} must be a CUDA tensor")
        if not v.is_contiguous():
            raise ValueError(f"viterbi: {what} must be contiguous")
        return tensor(from_array(v), what, dtype, ndim)
    init = dev(hmm["initial_prob"], "hmm['initial_prob']", f32, 1)
    outp = dev(hmm["output_prob"], "hmm['output_prob']", f32, 2)
    t1 = dev(hmm["trans1"], "hmm['trans1']", f32, 2)
    t2 = dev(hmm["trans2"], "hmm['trans2']", f32, 1)
    data = dev(seqs["data"], "seqs['data']", (torch.int8, torch.uint8), 2)
    lens = dev(seqs["lens"], "seqs['lens']", (torch.int64, torch.int32), 1)
    if n < 64 or n % 64 != 0:
        raise RuntimeError(f"viterbi: num_states={n} must be a positive multiple of 64")
    k = n // 16
    if init.shape[0] != n or tuple(t1.shape) != (k, 4) or t2.shape[0] != 16 or outp.shape[1] != k:
        raise RuntimeError(f"viterbi: table shapes {tuple(init.shape)}, {tuple(t1.shape)}, {tuple(t2.shape)}, "
                           f"{tuple(outp.shape)} do not match num_states={n}")
    batch, maxlen = data.shape
    if lens.shape[0] != batch:
        raise RuntimeError(f"viterbi: lens {tuple(lens.shape)} does not match data {tuple(data.shape)}")
    if lens.dtype != torch.int64:
        lens = lens.to(torch.int64)
    out = torch.zeros((batch, maxlen), dtype=torch.int32, device=data.device)
    n_obs = int(outp.shape[0])
    rc = _native.lib().parpy_b200_viterbi_ex(
        gamma, ptr(init), n, ptr(outp), n_obs if n_obs <= 256 else 0, synth, ptr(t1), ptr(t2), ptr(data), ptr(lens),
        maxlen, batch, batch_size, batch_overlap, ptr(out), maxlen, current_stream())
    _native.check(rc, "viterbi")
    if check:
        st = viterbi_status()
        if st["wait_timed_out"]:
            raise RuntimeError("viterbi: a wait inside the kernel ran out; the decoded paths are not valid")
    return out, lens


def viterbi_paths(hmm, seqs, batch_size=1024, batch_overlap=128):
    """``viterbi`` with the result trimmed per sequence, as the reference's wrapper
    returns it (benchmarks/7mer/trellis.py:64-66): a list of uint32 NumPy arrays."""
    import numpy as np
    out, lens = viterbi(hmm, seqs, batch_size, batch_overlap)
    host, hl = out.cpu().numpy().view(np.uint32), lens.cpu().numpy()
    return [host[i, :int(hl[i])].copy() for i in range(host.shape[0])]
