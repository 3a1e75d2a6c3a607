"""Helpers for the GPU parity tests: calling the C ABI directly with torch
device memory."""
import ctypes

import torch


def to_dev(d):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) and v.dim() > 0 else v) for k, v in d.items()}


def cabi_forward(native, hmm, seqs, flags=0, alpha=False, entry="parpy_b200_forward"):
    """Calls the forward entry point through ctypes. `hmm` / `seqs` hold CUDA tensors.
    Returns (result, alpha1, alpha2) as CUDA tensors."""
    lib = native.lib()
    B = int(seqs["num_instances"])
    N = int(hmm["num_states"])
    res = torch.full((B,), float("nan"), dtype=torch.float32, device="cuda")
    a1 = a2 = None
    if alpha:
        a1 = torch.zeros(B, N, dtype=torch.float32, device="cuda")
        a2 = torch.zeros_like(a1)
    P = ctypes.c_void_p
    common = [float(hmm["gamma"]), P(hmm["initial_prob"].data_ptr()), N, P(hmm["output_prob"].data_ptr()),
              float(hmm["synthetic_248"]), P(hmm["trans1"].data_ptr()), P(hmm["trans2"].data_ptr()),
              P(seqs["data"].data_ptr()), P(seqs["lens"].data_ptr()), int(seqs["maxlen"]), B]
    pa1 = P(a1.data_ptr()) if alpha else None
    pa2 = P(a2.data_ptr()) if alpha else None
    if entry == "parpy_b200_forward":
        rc = lib.parpy_b200_forward(*common, P(res.data_ptr()), pa1, pa2, flags,
                                    P(torch.cuda.current_stream().cuda_stream))
    elif entry == "parpy_b200_forward_ex":      # the same with the table height given (n_obs after output_prob)
        rc = lib.parpy_b200_forward_ex(*common[:4], int(hmm["output_prob"].shape[0]), *common[4:],
                                       P(res.data_ptr()), pa1, pa2, flags,
                                       P(torch.cuda.current_stream().cuda_stream))
    elif entry == "forward_kernel":
        rc = lib.forward_kernel(*common, P(res.data_ptr()), pa1, pa2)
    elif entry == "forward_kernel_scratch_first":
        rc = lib.forward_kernel_scratch_first(*common, pa1, pa2, P(res.data_ptr()))
    else:
        raise ValueError(entry)
    return rc, res, a1, a2
