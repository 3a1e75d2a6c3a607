"""Regenerates the committed HMM fixtures from the reference's test data.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/ParPy

It reads test/data/{3mer,5mer}-model.hdf5, test/data/signals.hdf5 and the
{3mer,5mer,7mer}-expected.txt golden log-likelihoods, builds the model tables
exactly the way the reference does (benchmarks/forward.py:20-87,
test/test_forward.py:11-78: logs taken in the file's dtype, transition table
reshaped [4,K] -> [K,4], emission columns permuted by base reversal, padded
int8 signal matrix) and writes compressed .npz files next to this script.
The 7mer model file is not distributed with the reference, so only its
expected values are stored (unused by the parity tests).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from parpy_b200.hdf5_min import H5File  # noqa: E402


def reverse_index(i, k):
    # benchmarks/forward.py:29-30
    return sum(((i // 4 ** x) % 4) * 4 ** (k - x - 1) for x in range(k))


def build_model(path):
    f = H5File(path)
    tables = f["Tables"]
    with np.errstate(divide="ignore"):
        obs = np.log(tables["ObservationProbabilities"].read())
    trans1 = np.log(tables["TransitionProbabilities"].read())
    dur_ds = tables["DurationProbabilities"]
    duration = np.log(dur_ds.read())
    tail_factor = np.log(dur_ds.attrs["TailFactor"])
    k = int(f["Parameters"].attrs["KMerLength"])
    K = 4 ** k
    init = np.full((16, K), -np.inf, dtype=np.float32)
    init[0, :] = np.log(1.0 / float(K))
    trans1 = trans1.reshape(4, K).transpose(1, 0)
    perm = np.array([reverse_index(i, k) for i in range(K)])
    out_prob = obs[:, perm].astype(np.float32)  # [101, K]
    synthetic_248 = np.log(np.exp(0.0) - np.exp(tail_factor))
    return {
        "gamma": np.float32(tail_factor),
        "trans1": np.ascontiguousarray(trans1, dtype=np.float32),
        "trans2": duration.astype(np.float32),
        "output_prob": np.ascontiguousarray(out_prob),
        "initial_prob": init.reshape(-1),
        "synthetic_248": np.float32(synthetic_248),
        "num_states": np.int64(16 * K),
    }


def build_signals(path):
    f = H5File(path)
    keys = f.keys()  # sorted, the order h5py iterates in
    sigs = [f[k]["Raw"]["Signal"].read() for k in keys]
    lens = np.array([len(s) for s in sigs], dtype=np.int64)
    data = np.zeros((len(sigs), int(lens.max())), dtype=np.int8)
    for i, s in enumerate(sigs):
        data[i, :len(s)] = s.astype(np.int8)
    return {"data": data, "lens": lens}


def main(ref_root):
    d = os.path.join(ref_root, "test", "data")
    for name in ("3mer", "5mer"):
        m = build_model(os.path.join(d, f"{name}-model.hdf5"))
        np.savez_compressed(os.path.join(HERE, f"hmm_{name}.npz"), **m)
    np.savez_compressed(os.path.join(HERE, "signals.npz"),
                        **build_signals(os.path.join(d, "signals.hdf5")))
    exp = {}
    for name in ("3mer", "5mer", "7mer"):
        with open(os.path.join(d, f"{name}-expected.txt")) as fh:
            exp["expected_" + name] = np.array([float(l) for l in fh], dtype=np.float32)
    np.savez_compressed(os.path.join(HERE, "expected.npz"), **exp)


if __name__ == "__main__":
    main(sys.argv[1])
