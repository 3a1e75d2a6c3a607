"""Seeded synthetic inputs with the shapes, dtypes and value ranges of the
reference's benchmark data. They stand in for the nanopore fixture
(test/data/*.hdf5) and the SuiteSparse collection, neither of which travels
with this package. Everything is generated on the CPU from an explicit seed so
that every rank of a multi-GPU job builds identical tables.
"""
import math

import numpy as np
import torch

N_OBS = 101      # observation levels (rows of output_prob), benchmarks/forward.py:36
LAYERS = 16      # explicit-duration layers


def hmm_model(k, seed=1234, tail_factor=0.605):
    """Model tables in the reference's layout (benchmarks/forward.py:64-72):
    ``trans1`` [K,4] and ``trans2`` [16] are log-softmaxed normal logits,
    ``output_prob`` [101,K] is a log-softmax over the 101 levels per k-mer,
    ``initial_prob`` is log(1/K) in layer 0 and -inf elsewhere (:20-27),
    ``gamma`` = log(tail), ``synthetic_248`` = log(1 - tail) (:48,:56)."""
    K = 4 ** k
    g = torch.Generator().manual_seed(seed)
    trans1 = torch.log_softmax(torch.randn(K, 4, generator=g, dtype=torch.float32), dim=1)
    trans2 = torch.log_softmax(torch.randn(LAYERS, generator=g, dtype=torch.float32), dim=0)
    output_prob = torch.log_softmax(torch.randn(N_OBS, K, generator=g, dtype=torch.float32), dim=0)
    init = torch.full((LAYERS, K), -math.inf, dtype=torch.float32)
    init[0, :] = math.log(1.0 / K)
    return {
        "gamma": torch.tensor(math.log(tail_factor), dtype=torch.float32),
        "trans1": trans1.contiguous(),
        "trans2": trans2.contiguous(),
        "output_prob": output_prob.contiguous(),
        "initial_prob": init.reshape(-1).contiguous(),
        "synthetic_248": torch.tensor(math.log1p(-tail_factor), dtype=torch.float32),
        "num_states": torch.tensor(LAYERS * K, dtype=torch.int64),
    }


def hmm_sequences(batch, min_len, max_len, seed=1234, pad_value=None, data_seed=None):
    """Observation batch in the reference's layout (benchmarks/forward.py:74-86):
    ``data`` int8 [B, maxlen] with levels in [0, 101), ``lens`` int64 [B] uniform
    in [min_len, max_len]. Entries past a sequence's length are padding; with
    ``pad_value=None`` they hold out-of-range garbage (the benchmark pads with
    uninitialised memory), which a correct kernel must never use. ``data_seed``
    redraws the observations only, keeping the lengths that ``seed`` gives."""
    g = torch.Generator().manual_seed(seed + 1)
    if min_len == max_len:
        lens = torch.full((batch,), max_len, dtype=torch.int64)
    else:
        lens = torch.randint(min_len, max_len + 1, (batch,), generator=g, dtype=torch.int64)
    maxlen = int(lens.max())
    if data_seed is not None:
        # same lengths for every data_seed (e.g. one per rank), different observations
        g = torch.Generator().manual_seed(data_seed)
    data = torch.randint(0, N_OBS, (batch, maxlen), generator=g, dtype=torch.int64).to(torch.int8)
    pad = -7 if pad_value is None else pad_value
    mask = torch.arange(maxlen).unsqueeze(0) >= lens.unsqueeze(1)
    data[mask] = pad
    return {
        "data": data.contiguous(),
        "lens": lens,
        "maxlen": torch.tensor(maxlen, dtype=torch.int64),
        "num_instances": torch.tensor(batch, dtype=torch.int64),
    }


def state_steps(hmm, seqs):
    """Work measure of one forward pass: num_states * sum of lengths."""
    return int(hmm["num_states"]) * int(seqs["lens"].sum())


def forward_algorithmic_bytes(hmm, seqs):
    """Bytes a streaming implementation must move: read + write alpha once per
    state-step, one emission row and one observation byte per sequence-step,
    one result per sequence."""
    n = int(hmm["num_states"])
    k = n // LAYERS
    steps = int(seqs["lens"].sum())
    return n * steps * 8 + steps * (4 * k + 1) + 4 * int(seqs["num_instances"])


def zipf_csr(nrows, ncols, mean_nnz=32, cap=4096, s=1.5, seed=1234):
    """CSR matrix with power-law row lengths (Zipf exponent ``s``, rescaled to
    the requested mean, capped), uniform columns, values U(-1,1); int64 indices
    as torch's CSR tensors carry them (test/test_spmv.py:20-27)."""
    rng = np.random.default_rng(seed)
    raw = rng.zipf(s, nrows).astype(np.float64)
    raw = np.minimum(raw, cap)
    scale = mean_nnz / raw.mean()
    lens = np.minimum(np.maximum(np.rint(raw * scale), 0), cap).astype(np.int64)
    rows = np.zeros(nrows + 1, dtype=np.int64)
    np.cumsum(lens, out=rows[1:])
    nnz = int(rows[-1])
    cols = rng.integers(0, ncols, nnz, dtype=np.int64)
    values = rng.uniform(-1.0, 1.0, nnz).astype(np.float32)
    return {
        "values": torch.from_numpy(values),
        "rows": torch.from_numpy(rows),
        "cols": torch.from_numpy(cols),
        "nrows": nrows,
    }


def uniform_csr(nrows, ncols, density, seed=1234):
    """CSR mask with ``round(ncols*density)`` distinct sorted columns per row."""
    rng = np.random.default_rng(seed)
    per_row = max(1, int(round(ncols * density)))
    cols = np.empty((nrows, per_row), dtype=np.int64)
    for i in range(nrows):
        cols[i] = np.sort(rng.choice(ncols, per_row, replace=False))
    crows = np.arange(nrows + 1, dtype=np.int64) * per_row
    values = rng.standard_normal(nrows * per_row).astype(np.float32)
    return {
        "crows": torch.from_numpy(crows),
        "cols": torch.from_numpy(cols.reshape(-1)),
        "values": torch.from_numpy(values),
        "nnz": nrows * per_row,
    }
