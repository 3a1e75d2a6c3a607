"""Pins the CPU oracle to the reference's golden vectors (no GPU needed)."""
import numpy as np
import pytest

from conftest import load_expected, load_model, load_signals, max_rel, shortest_reads
from oracle import oracle


def test_c_oracle_reproduces_3mer_golden_all_reads():
    # test/data/3mer-expected.txt, all 100 reads; the reference's own tolerance is
    # torch.allclose(atol=1e-5) (test/test_forward.py:176-178). The restatement is exact.
    hmm, seqs, exp = load_model("3mer"), load_signals(), load_expected("3mer")
    got = oracle.forward(hmm, seqs)
    assert np.array_equal(got, exp)


def test_c_oracle_reproduces_5mer_golden_subset():
    idx = shortest_reads(8)
    hmm, seqs, exp = load_model("5mer"), load_signals(idx), load_expected("5mer")[idx]
    got = oracle.forward(hmm, seqs)
    assert np.allclose(got, exp, rtol=1e-7, atol=0.0), max_rel(got, exp)


def test_numpy_restatement_matches_golden_and_c_oracle():
    idx = shortest_reads(4)
    hmm, seqs, exp = load_model("3mer"), load_signals(idx), load_expected("3mer")[idx]
    got_np = oracle.forward_numpy(hmm, seqs)
    got_c = oracle.forward(hmm, seqs)
    assert np.allclose(got_np, exp, rtol=2e-7, atol=0.0), max_rel(got_np, exp)
    assert np.allclose(got_np, got_c, rtol=2e-7, atol=0.0)


def test_oracle_final_alpha_is_consistent_with_result():
    idx = shortest_reads(2)
    hmm, seqs = load_model("3mer"), load_signals(idx)
    res, alpha = oracle.forward(hmm, seqs, want_alpha=True)
    with np.errstate(divide="ignore"):
        m = alpha.max(axis=1)
        lse = m + np.log(np.exp(alpha - m[:, None]).sum(axis=1, dtype=np.float32))
    assert np.allclose(lse, res, rtol=1e-6)


def test_oracle_ignores_padding_and_handles_length_one():
    import torch
    from parpy_b200 import synthetic
    hmm = synthetic.hmm_model(3, seed=7)
    seqs = synthetic.hmm_sequences(6, 1, 40, seed=3)
    seqs["lens"][0] = 1
    a = oracle.forward(hmm, seqs)
    seqs2 = dict(seqs)
    d = seqs["data"].clone()
    mask = torch.arange(d.shape[1])[None, :] >= seqs["lens"][:, None]
    d[mask] = 100
    seqs2["data"] = d
    b = oracle.forward(hmm, seqs2)
    assert np.array_equal(a, b)
    # length 1: log-sum-exp of initial + emission
    K = 64
    e = hmm["output_prob"][int(seqs["data"][0, 0].item()) & 0xFF].numpy()
    expect = np.log(np.sum(np.exp((np.log(1.0 / K) + e).astype(np.float64))))
    assert abs(a[0] - expect) < 1e-5


def test_oracle_zero_probability_emissions_give_minus_inf_states_not_nan():
    # the 3mer model has zero-probability emissions (log -> -inf); forward.py:156
    hmm = load_model("3mer")
    assert np.isinf(hmm["output_prob"].numpy()).any()
    idx = shortest_reads(1)
    seqs = load_signals(idx)
    res, alpha = oracle.forward(hmm, seqs, want_alpha=True)
    assert np.isfinite(res).all()
    assert not np.isnan(alpha).any()
    # force a dead k-mer at the last observation: its 16 states must be -inf, never NaN
    last = int(seqs["data"][0, int(seqs["lens"][0]) - 1].item())
    hmm["output_prob"] = hmm["output_prob"].clone()
    hmm["output_prob"][last, 5] = -np.inf
    res2, alpha2 = oracle.forward(hmm, seqs, want_alpha=True)
    a = alpha2.reshape(16, 64)
    assert np.isneginf(a[:, 5]).all() and not np.isnan(alpha2).any()
    assert np.isfinite(res2).all() and res2[0] <= res[0]
