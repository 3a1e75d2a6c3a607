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
