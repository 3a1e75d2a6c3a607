"""The allocation-free forward entry point, checked against the regular one.

Some callers of the library cannot tolerate a device allocation inside the call
(fully budgeted device memory, latency-critical stream pipelines, hosts that
forbid allocation in their execute callback). For them the library offers
parpy_b200_forward_noalloc, whose scheduling scratch is a fixed array compiled
into the library. This file calls it through the C ABI twice in a row — the
second time with a smaller batch, so that the array still holds entries of the
first call — and compares with parpy_b200_forward on the same inputs.

Collected last on purpose (file name), so that a run that stops at the first
failure has already run every other test; it must also pass on its own in a
fresh process.
"""
import ctypes

import numpy as np
import pytest
import torch

from conftest import max_rel
from gpu_util import cabi_forward, to_dev

pytestmark = pytest.mark.gpu
P = ctypes.c_void_p
REL = 1e-5   # the tolerance the other kernel-vs-kernel and kernel-vs-oracle tests use


def call_noalloc(native, hmm, seqs):
    B = int(seqs["num_instances"])
    res = torch.full((B,), float("nan"), dtype=torch.float32, device="cuda")
    rc = native.lib().parpy_b200_forward_noalloc(
        float(hmm["gamma"]), P(hmm["initial_prob"].data_ptr()), int(hmm["num_states"]),
        P(hmm["output_prob"].data_ptr()), float(hmm["synthetic_248"]), P(hmm["trans1"].data_ptr()),
        P(hmm["trans2"].data_ptr()), P(seqs["data"].data_ptr()), P(seqs["lens"].data_ptr()),
        int(seqs["maxlen"]), B, P(res.data_ptr()), P(torch.cuda.current_stream().cuda_stream))
    return rc, res


def test_noalloc_forward_matches_regular_entry_twice_in_a_row(native):
    from parpy_b200 import synthetic
    hmm = to_dev(synthetic.hmm_model(5, seed=31))
    first = to_dev(synthetic.hmm_sequences(300, 20, 400, seed=32))
    second = to_dev(synthetic.hmm_sequences(37, 1, 150, seed=33))     # smaller: stale entries remain
    for seqs in (first, second):
        rc, got = call_noalloc(native, hmm, seqs)
        assert rc == 0, native.error_message()
        rc2, ref, _, _ = cabi_forward(native, hmm, seqs)
        assert rc2 == 0, native.error_message()
        torch.cuda.synchronize()
        g, r = got.cpu().numpy(), ref.cpu().numpy()
        assert np.isfinite(g).all()
        assert max_rel(g, r) <= REL
        assert np.array_equal(g, r)          # same kernel, same arithmetic: bit-identical in fact


def test_noalloc_forward_7mer_cluster_path(native):
    from parpy_b200 import synthetic
    hmm = to_dev(synthetic.hmm_model(7, seed=34))
    seqs = to_dev(synthetic.hmm_sequences(20, 5, 60, seed=35))
    rc, got = call_noalloc(native, hmm, seqs)
    assert rc == 0, native.error_message()
    rc2, ref, _, _ = cabi_forward(native, hmm, seqs)
    assert rc2 == 0
    assert max_rel(got.cpu().numpy(), ref.cpu().numpy()) <= REL
    rc3, ref_log, _, _ = cabi_forward(native, hmm, seqs, 16)      # PARPY_B200_FWD_LOG_SPACE: the same kernel
    assert rc3 == 0 and np.array_equal(got.cpu().numpy(), ref_log.cpu().numpy())


def test_noalloc_forward_rejects_what_it_cannot_hold(native):
    from parpy_b200 import synthetic
    hmm = to_dev(synthetic.hmm_model(3, seed=36))
    seqs = to_dev(synthetic.hmm_sequences(4, 3, 9, seed=37))
    too_many = dict(seqs)
    too_many["num_instances"] = torch.tensor(native.NOALLOC_MAX_SEQUENCES + 1)
    rc, _ = call_noalloc(native, hmm, seqs)
    assert rc == 0, native.error_message()
    B = native.NOALLOC_MAX_SEQUENCES + 1
    res = torch.zeros(4, device="cuda")
    rc = native.lib().parpy_b200_forward_noalloc(
        float(hmm["gamma"]), P(hmm["initial_prob"].data_ptr()), int(hmm["num_states"]),
        P(hmm["output_prob"].data_ptr()), float(hmm["synthetic_248"]), P(hmm["trans1"].data_ptr()),
        P(hmm["trans2"].data_ptr()), P(seqs["data"].data_ptr()), P(seqs["lens"].data_ptr()),
        int(seqs["maxlen"]), B, P(res.data_ptr()), None)
    assert rc != 0
    msg = native.error_message()
    assert "exceeds the fixed scratch capacity" in msg and str(native.NOALLOC_MAX_SEQUENCES) in msg
    tiny = to_dev(synthetic.hmm_model(2, seed=38))       # 256 states: streaming kernel only
    rc, _ = call_noalloc(native, tiny, seqs)
    assert rc != 0 and "no resident mapping" in native.error_message()
    torch.cuda.synchronize()
