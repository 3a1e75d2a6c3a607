"""Parity of the CUDA HMM forward kernels with the reference's golden vectors and
the CPU oracle, through the C ABI and through the Python call surface.

Tolerances: the reference's own test accepts torch.allclose(atol=1e-5) with the
default rtol=1e-5 (test/test_forward.py:176-178); the target for this library is
max relative error <= 1e-4 on fp32 log-likelihoods. Both are asserted against
the golden vectors; comparisons with the oracle use 1e-5.
"""
import ctypes

import numpy as np
import pytest
import torch

from conftest import load_expected, load_model, load_signals, max_rel, shortest_reads
from gpu_util import cabi_forward, to_dev

pytestmark = pytest.mark.gpu

REL_TARGET = 1e-4        # library target vs the reference
REL_ORACLE = 1e-5        # kernel vs fp32 CPU oracle on identical inputs
FLAGS = {"factored": 0, "five_term": 4, "streaming": 1, "scaled": 8, "log_space": 16}


@pytest.fixture(scope="module")
def oracle_mod():
    from oracle import oracle
    return oracle


@pytest.mark.parametrize("model", ["3mer", "5mer"])
@pytest.mark.parametrize("variant", ["factored", "five_term", "streaming"])
def test_golden_vectors_all_reads(native, model, variant):
    hmm, seqs, exp = to_dev(load_model(model)), to_dev(load_signals()), load_expected(model)
    rc, res, _, _ = cabi_forward(native, hmm, seqs, FLAGS[variant], alpha=(variant == "streaming"))
    assert rc == 0, native.error_message()
    got = res.cpu().numpy()
    assert max_rel(got, exp) <= REL_TARGET
    assert np.allclose(got, exp, atol=1e-5, rtol=1e-5), max_rel(got, exp)
    if variant != "factored":
        # same operand order as the reference: agreement to a few ulp
        assert max_rel(got, exp) <= 1e-6


@pytest.mark.parametrize("entry", ["forward_kernel", "forward_kernel_scratch_first"])
def test_reference_shaped_entries_on_default_stream(native, entry):
    hmm, seqs, exp = to_dev(load_model("3mer")), to_dev(load_signals()), load_expected("3mer")
    rc, res, _, _ = cabi_forward(native, hmm, seqs, entry=entry)
    assert rc == 0, native.error_message()
    torch.cuda.synchronize()
    assert np.allclose(res.cpu().numpy(), exp, atol=1e-5, rtol=1e-5)


def test_5mer_config_against_oracle(native, oracle_mod):
    # 5mer benchmark workload: 100 sequences of T=2000 (oracle on a subset to keep CPU time bounded)
    from parpy_b200 import synthetic
    hmm = synthetic.hmm_model(5)
    seqs = synthetic.hmm_sequences(100, 2000, 2000)
    rc, res, _, _ = cabi_forward(native, to_dev(hmm), to_dev(seqs))
    assert rc == 0, native.error_message()
    got = res.cpu().numpy()
    assert np.isfinite(got).all()
    idx = np.arange(0, 100, 9)
    sub = {"data": seqs["data"][idx], "lens": seqs["lens"][idx]}
    exp = oracle_mod.forward(hmm, sub)
    assert max_rel(got[idx], exp) <= REL_ORACLE


def test_7mer_against_oracle_with_final_alpha(native, oracle_mod):
    # 7mer state space (262144 states), ragged short sequences so the oracle finishes in seconds;
    # checks every state of the final alpha vector, not just the scalar.
    from parpy_b200 import synthetic
    hmm = synthetic.hmm_model(7)
    seqs = synthetic.hmm_sequences(5, 2, 120, seed=99)     # lengths are only ever shortened below
    seqs["lens"][0] = 1
    seqs["lens"][1] = 2
    exp, exp_alpha = oracle_mod.forward(hmm, seqs, want_alpha=True)
    for variant in ("factored", "five_term"):
        rc, res, a1, a2 = cabi_forward(native, to_dev(hmm), to_dev(seqs), FLAGS[variant] | 2, alpha=True)
        assert rc == 0, native.error_message()
        assert max_rel(res.cpu().numpy(), exp) <= REL_ORACLE
        for i in range(5):
            # the reference leaves the final alpha in alpha1 for odd lengths (forward.py:163-165)
            a = (a1 if int(seqs["lens"][i]) & 1 else a2)[i].cpu().numpy()
            other = (a2 if int(seqs["lens"][i]) & 1 else a1)[i].cpu().numpy()
            assert max_rel(a, exp_alpha[i]) <= REL_ORACLE
            assert not other.any()


@pytest.mark.parametrize("arith", ["default", "log_space"])
def test_7mer_full_config_properties(native, arith):
    # 7mer benchmark workload: 500 sequences, lengths uniform in [1000, 4000]; size-independent checks,
    # for the default (scaled arithmetic on this state space) and for the log-space kernel.
    from parpy_b200 import synthetic
    hmm = synthetic.hmm_model(7)
    seqs = synthetic.hmm_sequences(500, 1000, 4000)
    dh, ds = to_dev(hmm), to_dev(seqs)
    fl = FLAGS["log_space"] if arith == "log_space" else 0
    rc, res, _, _ = cabi_forward(native, dh, ds, fl)
    assert rc == 0, native.error_message()
    full = res.cpu().numpy()
    assert np.isfinite(full).all() and (full < 0).all()
    # determinism: a second run is bit-identical
    rc, res2, _, _ = cabi_forward(native, dh, ds, fl)
    assert np.array_equal(full, res2.cpu().numpy())
    # permutation / batch-composition invariance: every sequence is scored independently
    perm = torch.randperm(500, generator=torch.Generator().manual_seed(5))[:97]
    sub = {"data": seqs["data"][perm].contiguous(), "lens": seqs["lens"][perm].contiguous(),
           "maxlen": seqs["maxlen"], "num_instances": torch.tensor(97)}
    rc, res3, _, _ = cabi_forward(native, dh, to_dev(sub), fl)
    assert rc == 0
    assert np.array_equal(res3.cpu().numpy(), full[perm.numpy()])
    # a prefix is at least as likely as the whole sequence (all emissions are log-probabilities)
    half = dict(sub)
    half["lens"] = (sub["lens"] // 2).contiguous()
    rc, res4, _, _ = cabi_forward(native, dh, to_dev(half), fl)
    assert (res4.cpu().numpy() >= res3.cpu().numpy()).all()
    # the five-term form agrees with this arithmetic far inside the tolerance
    rc, res5, _, _ = cabi_forward(native, dh, to_dev(sub), FLAGS["five_term"])
    assert max_rel(res3.cpu().numpy(), res5.cpu().numpy()) <= REL_ORACLE


def test_7mer_benchmark_batch_full_length_against_oracle(native, oracle_mod, capsys):
    # The benchmark's own batch (500 sequences, lengths uniform in [1000, 4000], seed 1234) through
    # the default kernel (the scaled one on this state space); the longest, the shortest and six more sequences are scored at full length
    # by the CPU oracle (benchmarks/forward.py:103-158 restated). fp32 log-space rounding drifts with
    # length, so this is the check at the lengths the throughput figure is quoted on. Tolerance of
    # the reference's own test: test/test_forward.py:176-178 (rtol 1e-5).
    from parpy_b200 import synthetic
    hmm = synthetic.hmm_model(7)
    seqs = synthetic.hmm_sequences(500, 1000, 4000)
    lens = seqs["lens"].numpy()
    rest = np.random.default_rng(7).permutation(500)
    pick = [int(np.argmax(lens)), int(np.argmin(lens))]
    pick += [int(i) for i in rest if int(i) not in pick][:6]
    pick = np.array(sorted(pick))
    sub = {"data": seqs["data"][pick].contiguous(), "lens": seqs["lens"][pick].contiguous(),
           "maxlen": seqs["maxlen"], "num_instances": torch.tensor(len(pick))}
    exp = oracle_mod.forward(hmm, sub)
    dh = to_dev(hmm)
    rc, res, _, _ = cabi_forward(native, dh, to_dev(seqs))
    assert rc == 0, native.error_message()
    got = res.cpu().numpy()
    assert np.isfinite(got).all()
    err = {"default": max_rel(got[pick], exp)}
    ds = to_dev(sub)
    for name in ("log_space", "five_term", "scaled"):
        rc, r, _, _ = cabi_forward(native, dh, ds, FLAGS[name])
        assert rc == 0, native.error_message()
        err[name] = max_rel(r.cpu().numpy(), exp)
        if name == "scaled":     # what a call without flags runs on this state space
            assert np.array_equal(r.cpu().numpy(), got[pick])
    with capsys.disabled():
        print("\n7mer full-length parity (max rel vs oracle, lengths %d..%d): %s"
              % (lens[pick].min(), lens[pick].max(), ", ".join(f"{k} {v:.2e}" for k, v in err.items())))
    assert err["default"] <= REL_ORACLE
    assert err["log_space"] <= REL_ORACLE
    assert err["five_term"] <= REL_ORACLE
    # the scaled kernel follows exact arithmetic; its distance from the fp32 oracle is the
    # oracle's own accumulated rounding, which the library target bounds
    assert err["scaled"] <= REL_TARGET


def test_padding_is_never_used_and_uint8_is_accepted(native):
    from parpy_b200 import synthetic
    hmm = synthetic.hmm_model(5, seed=3)
    seqs = synthetic.hmm_sequences(40, 3, 300, seed=8)          # padding = -7 (out of range)
    dh = to_dev(hmm)
    rc, a, _, _ = cabi_forward(native, dh, to_dev(seqs))
    clean = dict(seqs)
    d = seqs["data"].clone()
    d[d < 0] = 0
    clean["data"] = d.to(torch.uint8)
    rc2, b, _, _ = cabi_forward(native, dh, to_dev(clean))
    assert rc == 0 and rc2 == 0
    assert np.array_equal(a.cpu().numpy(), b.cpu().numpy())
    # extra slack columns (maxlen larger than any length) change nothing
    wide = dict(clean)
    wide["data"] = torch.cat([clean["data"], torch.full((40, 17), 100, dtype=torch.uint8)], dim=1).contiguous()
    wide["maxlen"] = torch.tensor(wide["data"].shape[1])
    rc3, c, _, _ = cabi_forward(native, dh, to_dev(wide))
    assert rc3 == 0 and np.array_equal(a.cpu().numpy(), c.cpu().numpy())


@pytest.mark.parametrize("k", [2, 3, 4, 6])
def test_other_state_spaces_against_oracle(native, oracle_mod, k):
    # k=2 (256 states) has no resident mapping and runs the streaming kernel
    from parpy_b200 import synthetic
    hmm = synthetic.hmm_model(k, seed=k)
    seqs = synthetic.hmm_sequences(7, 1, 90 if k < 6 else 40, seed=k + 1)
    exp = oracle_mod.forward(hmm, seqs)
    rc, res, _, _ = cabi_forward(native, to_dev(hmm), to_dev(seqs), alpha=True)
    assert rc == 0, native.error_message()
    assert max_rel(res.cpu().numpy(), exp) <= REL_ORACLE


def test_kernel_layout_variants_agree_with_oracle(native, oracle_mod, monkeypatch):
    # 7mer: the packed base-2 split kernel (default) and the scalar natural-log split kernel, each
    # with several sets of layers on the polynomial exponential, and the all-register 8-CTA layout;
    # every variant against the CPU oracle on the same inputs.
    from parpy_b200 import synthetic
    hmm = synthetic.hmm_model(7, seed=5)
    seqs = synthetic.hmm_sequences(6, 2, 90, seed=6)
    exp, exp_alpha = oracle_mod.forward(hmm, seqs, want_alpha=True)
    dh, ds = to_dev(hmm), to_dev(seqs)
    settings = ([{"PARPY_B200_FWD_SPLIT": "0"}]
                + [{"PARPY_B200_FWD_PACKED": "0", "PARPY_B200_FWD_POLY": str(n)} for n in (0, 4, 5, 6, 8)]
                + [{"PARPY_B200_FWD_POLY": str(n)} for n in (0, 5, 8, 9, 10, 11, 12)]
                # default layout (upper layers and transition columns in tensor memory, finite arithmetic,
                # logarithm of 13 layers as degree-5 polynomial); the degree-6 polynomial on 11 layers; the
                # kernels that compute on -inf itself with 4, 6 and 8 layers in registers; other masks; the
                # same kernels with shared memory in place of tensor memory
                + [{}, {"PARPY_B200_FWD_LG6": "0"}, {"PARPY_B200_FWD_LG6": "1", "PARPY_B200_FWD_MASKS": "0:FFFE"},
                   {"PARPY_B200_FWD_FINITE": "0"}, {"PARPY_B200_FWD_MASKS": "0:AAAA"}, {"PARPY_B200_FWD_REGLAYERS": "6"}, {"PARPY_B200_FWD_REGLAYERS": "8"},
                   {"PARPY_B200_FWD_MASKS": "0:EEEE"}, {"PARPY_B200_FWD_MASKS": "5554:0", "PARPY_B200_FWD_REGLAYERS": "4"},
                   {"PARPY_B200_FWD_TMEM": "0"}, {"PARPY_B200_FWD_TMEM": "0", "PARPY_B200_FWD_MASKS": "0:FFFF"},
                   {"PARPY_B200_FWD_TMEM": "0", "PARPY_B200_FWD_MASKS": "5554:AAAA"}])
    knobs = ("PARPY_B200_FWD_SPLIT", "PARPY_B200_FWD_POLY", "PARPY_B200_FWD_PACKED", "PARPY_B200_FWD_TMEM",
             "PARPY_B200_FWD_MASKS", "PARPY_B200_FWD_REGLAYERS", "PARPY_B200_FWD_LG6", "PARPY_B200_FWD_FINITE")
    for env in settings:
        for k in knobs:
            monkeypatch.delenv(k, raising=False)
        for k, v in env.items():
            monkeypatch.setenv(k, v)
        rc, res, a1, a2 = cabi_forward(native, dh, ds, 2, alpha=True)
        assert rc == 0, native.error_message()
        assert max_rel(res.cpu().numpy(), exp) <= REL_ORACLE, env
        for i in range(6):
            a = (a1 if int(seqs["lens"][i]) & 1 else a2)[i].cpu().numpy()
            assert max_rel(a, exp_alpha[i]) <= REL_ORACLE, env
    # 5mer: one CTA per sequence with packed arithmetic (default) against the 4-CTA cluster layout
    hmm = synthetic.hmm_model(5, seed=7)
    seqs = synthetic.hmm_sequences(9, 2, 120, seed=8)
    exp, exp_alpha = oracle_mod.forward(hmm, seqs, want_alpha=True)
    dh, ds = to_dev(hmm), to_dev(seqs)
    for env in ([{}, {"PARPY_B200_FWD_LG6": "0"}, {"PARPY_B200_FWD_LG6": "2"}, {"PARPY_B200_FWD_FINITE": "0"},
                 {"PARPY_B200_FWD_PACKED": "0"}] + [{"PARPY_B200_FWD_POLY": str(n)} for n in (0, 5, 8, 10, 12, 14, 16)]
                + [{"PARPY_B200_FWD_MASKS": m} for m in ("0:EEEC", "0:FFFE", "AAAA:5554", "AAAA:5555", "0:AAAA", "8888:7776")]):
        for k in knobs:
            monkeypatch.delenv(k, raising=False)
        for k, v in env.items():
            monkeypatch.setenv(k, v)
        rc, res, a1, a2 = cabi_forward(native, dh, ds, 2, alpha=True)
        assert rc == 0, native.error_message()
        assert max_rel(res.cpu().numpy(), exp) <= REL_ORACLE, env
        for i in range(9):
            a = (a1 if int(seqs["lens"][i]) & 1 else a2)[i].cpu().numpy()
            assert max_rel(a, exp_alpha[i]) <= REL_ORACLE, env


def test_packed_arithmetic_is_bit_identical_to_scalar(native, monkeypatch):
    # The packed kernel issues the scalar kernel's additions and multiply-adds two at a time
    # (add/sub/mul/fma.f32x2); every half rounds like the scalar instruction, so with the same
    # set of polynomial layers the two must agree bit for bit, final alpha included.
    from parpy_b200 import synthetic
    hmm = synthetic.hmm_model(7, seed=11)
    seqs = synthetic.hmm_sequences(5, 40, 300, seed=12)
    dh, ds = to_dev(hmm), to_dev(seqs)
    for n in (0, 5, 8):
        out = {}
        for packed in ("0", "1"):
            monkeypatch.setenv("PARPY_B200_FWD_POLY", str(n))
            monkeypatch.setenv("PARPY_B200_FWD_PACKED", packed)
            rc, res, a1, a2 = cabi_forward(native, dh, ds, 2, alpha=True)
            assert rc == 0, native.error_message()
            out[packed] = (res.cpu().numpy().copy(), a1.cpu().numpy().copy(), a2.cpu().numpy().copy())
        assert np.array_equal(out["0"][0], out["1"][0]), n
        for i in range(5):
            which = 1 if int(seqs["lens"][i]) & 1 else 2
            assert np.array_equal(out["0"][which][i], out["1"][which][i]), (n, i)


def test_scaled_variant_against_golden_oracle_and_log_space(native, oracle_mod):
    # Extended-range linear arithmetic (PARPY_B200_FWD_SCALED). It tracks a float64
    # evaluation to ~1e-8, so its distance from the reference's fp32 golden vectors is the
    # golden vectors' own rounding: 1.5e-5 at worst on the 5mer fixture (read 79), which is inside
    # the library target of 1e-4 but outside the reference test's rtol of 1e-5; that is why it is
    # the default only for state spaces larger than the ones the reference ships golden vectors
    # for (4096 k-mers and more), and opt-in here.
    hmm, seqs, exp = to_dev(load_model("5mer")), to_dev(load_signals()), load_expected("5mer")
    rc, res, _, _ = cabi_forward(native, hmm, seqs, FLAGS["scaled"])
    assert rc == 0, native.error_message()
    got = res.cpu().numpy()
    assert max_rel(got, exp) <= REL_TARGET
    assert max_rel(got, exp) <= 2e-5
    # 7mer, per-state check of the final alpha against the CPU oracle
    from parpy_b200 import synthetic
    hmm7 = synthetic.hmm_model(7, seed=5)
    seqs7 = synthetic.hmm_sequences(6, 1, 90, seed=6)
    seqs7["lens"][0] = 1
    exp7, exp_alpha = oracle_mod.forward(hmm7, seqs7, want_alpha=True)
    rc, res, a1, a2 = cabi_forward(native, to_dev(hmm7), to_dev(seqs7), FLAGS["scaled"] | 2, alpha=True)
    assert rc == 0, native.error_message()
    assert max_rel(res.cpu().numpy(), exp7) <= REL_ORACLE
    for i in range(6):
        a = (a1 if int(seqs7["lens"][i]) & 1 else a2)[i].cpu().numpy()
        assert max_rel(a, exp_alpha[i]) <= REL_ORACLE
    # zero-probability emissions: an impossible sequence scores NaN, as it does in the reference's
    # final reduction ((-inf) - (-inf), benchmarks/forward.py:168-173) and in the oracle
    dead = dict(hmm7)
    dead_tbl = hmm7["output_prob"].clone()
    last = int(seqs7["data"][2, int(seqs7["lens"][2]) - 1].item()) & 0xFF
    dead_tbl[last, :] = -np.inf
    dead["output_prob"] = dead_tbl
    rc, res, _, _ = cabi_forward(native, to_dev(dead), to_dev(seqs7), FLAGS["scaled"])
    exp_dead = oracle_mod.forward(dead, seqs7)
    got_dead = res.cpu().numpy()
    assert rc == 0 and np.isnan(got_dead[2]) and np.array_equal(np.isnan(got_dead), np.isnan(exp_dead))
    assert max_rel(got_dead[~np.isnan(exp_dead)], exp_dead[~np.isnan(exp_dead)]) <= REL_ORACLE
    # small state spaces are refused rather than silently run in log space
    rc, _, _, _ = cabi_forward(native, to_dev(load_model("3mer")), to_dev(load_signals(shortest_reads(2))),
                               FLAGS["scaled"])
    assert rc != 0 and "scaled kernel needs" in native.error_message()


def test_default_arithmetic_by_state_space(native, monkeypatch):
    # Without flags: scaled arithmetic for 4096 k-mers and more, log space below that and whenever
    # alpha is asked for; PARPY_B200_FWD_DEFAULT=log and the LOG_SPACE flag give log space everywhere.
    from parpy_b200 import synthetic
    monkeypatch.delenv("PARPY_B200_FWD_DEFAULT", raising=False)
    for k, scaled_default in ((5, False), (6, True), (7, True)):
        hmm, seqs = to_dev(synthetic.hmm_model(k, seed=40 + k)), to_dev(synthetic.hmm_sequences(7, 2, 70, seed=50 + k))
        out = {}
        for name, flags in (("none", 0), ("log", FLAGS["log_space"]), ("scaled", FLAGS["scaled"])):
            rc, res, _, _ = cabi_forward(native, hmm, seqs, flags)
            assert rc == 0, native.error_message()
            out[name] = res.cpu().numpy()
        assert not np.array_equal(out["log"], out["scaled"])          # different rounding somewhere
        assert np.array_equal(out["none"], out["scaled" if scaled_default else "log"])
        assert max_rel(out["scaled"], out["log"]) <= REL_ORACLE
        rc, res, a1, a2 = cabi_forward(native, hmm, seqs, 2, alpha=True)     # alpha requested: log space
        assert rc == 0 and np.array_equal(res.cpu().numpy(), out["log"])
        monkeypatch.setenv("PARPY_B200_FWD_DEFAULT", "log")
        rc, res, _, _ = cabi_forward(native, hmm, seqs)
        assert rc == 0 and np.array_equal(res.cpu().numpy(), out["log"])
        monkeypatch.delenv("PARPY_B200_FWD_DEFAULT")
    rc, _, _, _ = cabi_forward(native, hmm, seqs, FLAGS["log_space"] | FLAGS["scaled"])
    assert rc != 0 and "exclude each other" in native.error_message()


@pytest.mark.parametrize("k,scale,nseq,lo,hi", [(6, 8.0, 6, 50, 400), (6, 16.0, 6, 50, 400), (7, 8.0, 4, 30, 200),
                                                (6, 8.0, 2, 8000, 12000)])
def test_peaky_tables_and_long_sequences(native, oracle_mod, k, scale, nseq, lo, hi):
    # Tables with a wide dynamic range (emission log-probabilities down to -60 / -120, transition
    # rows dominated by one successor) and sequences of 10^4 steps, on the state spaces whose
    # default is the scaled kernel: neighbouring k-mers of a thread then differ by many orders of
    # magnitude, which is what its per-thread exponent has to absorb. Same bar as everywhere.
    from parpy_b200 import synthetic
    hmm = synthetic.hmm_model(k, seed=70 + k)
    g = torch.Generator().manual_seed(99)
    hmm["output_prob"] = torch.log_softmax(scale * torch.randn(101, 4 ** k, generator=g), dim=0).contiguous()
    hmm["trans1"] = torch.log_softmax(4.0 * torch.randn(4 ** k, 4, generator=g), dim=1).contiguous()
    assert float(hmm["output_prob"].min()) < -7.0 * scale
    seqs = synthetic.hmm_sequences(nseq, lo, hi, seed=80 + k)
    exp = oracle_mod.forward(hmm, seqs)
    for flags in (0, FLAGS["scaled"], FLAGS["log_space"]):
        rc, res, _, _ = cabi_forward(native, to_dev(hmm), to_dev(seqs), flags)
        assert rc == 0, native.error_message()
        assert max_rel(res.cpu().numpy(), exp) <= REL_ORACLE, flags
    rc = ctypes.c_uint32(0)
    assert native.lib().parpy_b200_forward_status(ctypes.byref(rc)) == 0 and rc.value == 0


@pytest.mark.parametrize("k,nseq,lo,hi", [(7, 40, 30, 400), (6, 50, 1, 300)])
def test_scaled_layouts_agree_bit_for_bit(native, monkeypatch, k, nseq, lo, hi):
    # The scaled kernel in its layouts: clusters of 512-thread CTAs with all 16 layers in
    # registers (PARPY_B200_SCALED_SPLIT=0); 1024-thread CTAs with layers 8..15 and the transition
    # columns in shared memory and one exponent per sending thread in the exchange
    # (PARPY_B200_SCALED_TMEM=0); the same with those values in tensor memory (default from 4096
    # k-mers). Every scaling is by a power of two and the operations are the same in the same order,
    # so all three must produce the same bits, final alpha included.
    from parpy_b200 import synthetic
    hmm = synthetic.hmm_model(k, seed=20 + k)
    seqs = synthetic.hmm_sequences(nseq, lo, hi, seed=30 + k)
    dh, ds = to_dev(hmm), to_dev(seqs)
    out = []
    for split, tmem, async_x, rl in (("0", "0", "0", "8"), ("1", "0", "0", "8"), ("1", "1", "0", "8"), ("1", "1", "1", "8"),
                                     ("1", "1", "1", "6"), ("1", "1", "1", "4"), ("1", "1", "0", "4")):
        monkeypatch.setenv("PARPY_B200_SCALED_SPLIT", split)
        monkeypatch.setenv("PARPY_B200_SCALED_TMEM", tmem)
        monkeypatch.setenv("PARPY_B200_SCALED_ASYNC", async_x)     # layer 0 by st.async + mbarriers
        monkeypatch.setenv("PARPY_B200_FWD_REGLAYERS", rl)         # layers kept in registers
        rc, res, a1, a2 = cabi_forward(native, dh, ds, FLAGS["scaled"] | 2, alpha=True)
        assert rc == 0, native.error_message()
        out.append((res.cpu().numpy().copy(), a1.cpu().numpy().copy(), a2.cpu().numpy().copy()))
        # twice in a row: tensor memory is released and taken again
        rc, res2, _, _ = cabi_forward(native, dh, ds, FLAGS["scaled"])
        assert rc == 0 and np.array_equal(res2.cpu().numpy(), out[-1][0])
    assert np.isfinite(out[0][0]).all()
    for n, other in enumerate(out[1:]):
        assert np.array_equal(out[0][0], other[0]), (n + 1, int((out[0][0] != other[0]).sum()))
        for q in (1, 2):
            diff = out[0][q] != other[q]
            assert not diff.any(), (n + 1, q, int(diff.sum()), out[0][q][diff][:4], other[q][diff][:4])


def test_8mer_runs_on_a_16_cta_cluster(native, oracle_mod):
    # 4^8 k-mers x 16 layers = 1,048,576 states: non-portable cluster of 16 CTAs, log-space and
    # scaled kernels (the scaled one only exists in the 1024-thread layout at this size)
    from parpy_b200 import synthetic
    hmm = synthetic.hmm_model(8, seed=8)
    seqs = synthetic.hmm_sequences(3, 1, 16, seed=9)
    exp = oracle_mod.forward(hmm, seqs)
    for flags in (0, FLAGS["log_space"], FLAGS["scaled"]):
        rc, res, _, _ = cabi_forward(native, to_dev(hmm), to_dev(seqs), flags)
        assert rc == 0, native.error_message()
        assert max_rel(res.cpu().numpy(), exp) <= REL_ORACLE


def test_empty_batch_and_single_step(native):
    from parpy_b200 import synthetic
    hmm = to_dev(synthetic.hmm_model(5, seed=2))
    seqs = to_dev(synthetic.hmm_sequences(3, 1, 1, seed=3))          # maxlen = 1: no time steps at all
    rc, res, _, _ = cabi_forward(native, hmm, seqs)
    assert rc == 0 and np.isfinite(res.cpu().numpy()).all()
    empty = dict(seqs)
    empty["num_instances"] = torch.tensor(0)
    rc, _, _, _ = cabi_forward(native, hmm, empty)
    assert rc == 0


def test_zero_probability_emissions_stay_minus_inf(native, oracle_mod):
    hmm = load_model("3mer")
    seqs = load_signals(shortest_reads(3))
    last = int(seqs["data"][0, int(seqs["lens"][0]) - 1].item())
    hmm["output_prob"] = hmm["output_prob"].clone()
    hmm["output_prob"][last, 5] = -np.inf
    exp, exp_alpha = oracle_mod.forward(hmm, seqs, want_alpha=True)
    rc, res, a1, a2 = cabi_forward(native, to_dev(hmm), to_dev(seqs), 2, alpha=True)
    assert rc == 0
    a = (a1 if int(seqs["lens"][0]) & 1 else a2)[0].cpu().numpy().reshape(16, 64)
    assert np.isneginf(a[:, 5]).all() and not np.isnan(a).any()
    assert max_rel(res.cpu().numpy(), exp) <= REL_ORACLE


def test_bad_arguments_are_rejected_with_a_message(native):
    from parpy_b200 import synthetic
    hmm, seqs = to_dev(synthetic.hmm_model(3)), to_dev(synthetic.hmm_sequences(4, 5, 9))
    bad = dict(hmm)
    bad["num_states"] = torch.tensor(1000)
    rc, _, _, _ = cabi_forward(native, bad, seqs)
    assert rc != 0 and "multiple of 64" in native.error_message()
    rc, _, _, _ = cabi_forward(native, hmm, seqs, FLAGS["streaming"], alpha=False)
    assert rc != 0 and "alpha1 and alpha2" in native.error_message()
    # the context is still healthy afterwards
    rc, res, _, _ = cabi_forward(native, hmm, seqs)
    assert rc == 0 and np.isfinite(res.cpu().numpy()).all()


def test_out_of_range_lengths_are_clamped_and_flagged(native):
    from parpy_b200 import synthetic
    hmm, seqs = synthetic.hmm_model(3), synthetic.hmm_sequences(4, 5, 9, pad_value=0)
    st = ctypes.c_uint32(7)
    assert native.lib().parpy_b200_forward_status(ctypes.byref(st)) == 0
    seqs["lens"][2] = 10_000
    rc, res, _, _ = cabi_forward(native, to_dev(hmm), to_dev(seqs))
    assert rc == 0
    assert native.lib().parpy_b200_forward_status(ctypes.byref(st)) == 0
    assert st.value & 1
    assert np.isfinite(res.cpu().numpy()).all()
    assert native.lib().parpy_b200_forward_status(ctypes.byref(st)) == 0 and st.value == 0


# ---- the Python call surface, written the way the reference's tests are ------------
def _forward_like_reference(hmm, seqs, opts, device):
    # test/test_forward.py:162-167
    import parpy_b200 as parpy

    @parpy.jit
    def forward_kernel(hmm, seqs, alpha1, alpha2, result):
        pass

    n, b = int(hmm["num_states"]), int(seqs["num_instances"])
    alpha1 = torch.zeros((b, n), dtype=torch.float32, device=device)
    alpha2 = torch.zeros_like(alpha1)
    result = torch.zeros(b, dtype=torch.float32, device=device)
    forward_kernel(hmm, seqs, alpha1, alpha2, result, opts=opts)
    return result, alpha1, alpha2


@pytest.mark.parametrize("nthreads", [512, 2048])
@pytest.mark.parametrize("device", ["cpu", "cuda"])
def test_forward_python_surface(device, nthreads):
    # test/test_forward.py:180-207 (single block / multi block), host arrays and device arrays
    import parpy_b200 as parpy
    hmm, seqs, exp = load_model("3mer"), load_signals(), torch.from_numpy(load_expected("3mer"))
    if device == "cuda":
        hmm = {k: v.cuda() for k, v in hmm.items()}      # 0-d entries on the device too, as in the benchmark
        seqs = {k: v.cuda() for k, v in seqs.items()}
    p = {"inst": parpy.threads(int(seqs["num_instances"])), "state": parpy.threads(nthreads)}
    opts = parpy.par(p)
    probs, a1, a2 = _forward_like_reference(hmm, seqs, opts, device)
    if device == "cuda":
        torch.cuda.synchronize()
    assert torch.allclose(probs.cpu(), exp, atol=1e-5), f"{probs}\n{exp}"
    assert not a1.any() and not a2.any()        # resident kernel: scratch untouched


def test_tuner_loop_of_the_reference_benchmark_gives_one_answer():
    # benchmarks/forward.py:200-218 (ParPyTuned): the benchmark times forward_parpy(hmm, seqs, nthreads)
    # for nthreads = 2^10 .. 2^18 <= num_states and keeps the fastest. The native kernel picks its own
    # mapping, so every setting must return the same log-likelihoods; 5-mer workload (16384 states).
    import statistics
    from parpy_b200 import hmm as hmm_mod, synthetic
    hmm = hmm_mod.to_device(synthetic.hmm_model(5))
    seqs = hmm_mod.to_device(synthetic.hmm_sequences(100, 200, 200))
    best_time, best_nthreads, results = float("inf"), 0, {}
    for nthreads in [2 ** n for n in range(10, 19) if 2 ** n <= int(hmm["num_states"])]:
        times = []
        for run in range(1 + 5):                      # nwarmup=1, nruns=5
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            results[nthreads] = hmm_mod.forward_parpy(hmm, seqs, nthreads)
            e1.record()
            torch.cuda.synchronize()
            if run:
                times.append(e0.elapsed_time(e1))
        if statistics.mean(times) < best_time:
            best_time, best_nthreads = statistics.mean(times), nthreads
    assert sorted(results) == [1024, 2048, 4096, 8192, 16384] and best_nthreads in results
    first = results[1024]
    assert torch.isfinite(first).all()
    for r in results.values():
        assert torch.equal(r, first)


def test_forward_python_surface_numpy_and_write_alpha(oracle_mod):
    import parpy_b200 as parpy
    from parpy_b200.hmm import forward_kernel
    idx = shortest_reads(3)
    hmm_t, seqs_t = load_model("3mer"), load_signals(idx)
    exp, exp_alpha = oracle_mod.forward(hmm_t, seqs_t, want_alpha=True)
    hmm = {k: v.numpy() for k, v in hmm_t.items()}
    seqs = {k: v.numpy() for k, v in seqs_t.items()}
    result = np.zeros(3, dtype=np.float32)
    a1 = np.zeros((3, 1024), dtype=np.float32)
    a2 = np.zeros_like(a1)
    opts = parpy.par({"inst": parpy.threads(3)})
    opts.b200 = {"write_alpha": True}
    forward_kernel(hmm, seqs, result, a1, a2, opts=opts)
    assert max_rel(result, exp) <= REL_ORACLE
    for i in range(3):
        got = a1[i] if int(seqs["lens"][i]) & 1 else a2[i]
        assert max_rel(got, exp_alpha[i]) <= REL_ORACLE
    # non-contiguous and read-only arrays are rejected like the reference does
    with pytest.raises(ValueError, match="contiguous"):
        forward_kernel(hmm, seqs, np.zeros(6, dtype=np.float32)[::2], a1, a2, opts=opts)


def test_forward_parpy_wrapper_and_sharded_gather_single_rank():
    from parpy_b200 import dist, hmm as hmm_mod, synthetic
    hmm, seqs = synthetic.hmm_model(5), synthetic.hmm_sequences(24, 20, 200, seed=4)
    full = hmm_mod.forward_parpy(hmm_mod.to_device(hmm), hmm_mod.to_device(seqs), 1024).cpu().numpy()
    parts = []
    for rank in range(3):
        local, idx = dist.shard_sequences(seqs, rank, 3)
        r = hmm_mod.forward_parpy(hmm_mod.to_device(hmm), hmm_mod.to_device(local)).cpu().numpy()
        parts.append((idx, r))
    merged = np.empty(24, dtype=np.float32)
    for idx, r in parts:
        merged[idx] = r
    assert np.array_equal(merged, full)


def test_reference_cuda_agrees_on_5mer_fixture(native, oracle_mod):
    # the reference's own CUDA implementation (benchmarks/5mer/hmm.cu built into oracle/_ref)
    if not oracle_mod.trellis_available(5):
        pytest.skip("oracle/_ref/trellis_5mer.so has not been built")
    idx = shortest_reads(6)
    hmm, seqs, exp = load_model("5mer"), load_signals(idx), load_expected("5mer")[idx]
    ref = oracle_mod.trellis_forward(5, hmm, seqs)
    assert np.allclose(ref, exp, atol=1e-5, rtol=1e-5), max_rel(ref, exp)
    rc, res, _, _ = cabi_forward(native, to_dev(hmm), to_dev(seqs))
    assert rc == 0 and max_rel(res.cpu().numpy(), ref) <= REL_ORACLE


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_device_table_preparation_matches_the_reference_loader(native, dtype):
    # benchmarks/forward.py:20-63 restated in NumPy (logs in the file's dtype, base-reversal column
    # permutation, [4,K] -> [K,4]) against parpy_b200_hmm_prepare_tables
    k, n_obs = 4, 101
    K = 4 ** k
    rng = np.random.default_rng(5)
    obs = rng.random((n_obs, K)).astype(dtype)
    obs[3, 7] = 0.0                                              # zero probability -> -inf
    trans = rng.random((4, K)).astype(dtype)
    dur = rng.random(16).astype(dtype)
    with np.errstate(divide="ignore"):
        lobs = np.log(obs)
    rev = np.array([sum(((i // 4 ** x) % 4) * 4 ** (k - x - 1) for x in range(k)) for i in range(K)])
    exp_out = lobs[:, rev].astype(np.float32)
    exp_t1 = np.log(trans).reshape(4, K).transpose(1, 0).astype(np.float32)
    exp_t2 = np.log(dur).astype(np.float32)
    exp_init = np.full((16, K), -np.inf, dtype=np.float32)
    exp_init[0, :] = np.log(1.0 / float(K))
    P = ctypes.c_void_p
    d_obs, d_tr, d_du = (torch.from_numpy(a).cuda() for a in (obs, trans, dur))
    out = torch.empty((n_obs, K), device="cuda")
    t1 = torch.empty((K, 4), device="cuda")
    t2 = torch.empty(16, device="cuda")
    init = torch.empty(16 * K, device="cuda")
    rc = native.lib().parpy_b200_hmm_prepare_tables(
        P(d_obs.data_ptr()), P(d_tr.data_ptr()), P(d_du.data_ptr()), int(dtype == np.float64), k, n_obs,
        P(out.data_ptr()), P(t1.data_ptr()), P(t2.data_ptr()), P(init.data_ptr()), None)
    torch.cuda.synchronize()
    assert rc == 0, native.error_message()
    assert np.array_equal(init.cpu().numpy().reshape(16, K), exp_init)
    for got, exp in ((out, exp_out), (t1, exp_t1), (t2, exp_t2)):
        g = got.cpu().numpy()
        assert np.array_equal(np.isneginf(g), np.isneginf(exp))
        fin = np.isfinite(exp)
        assert np.all(np.abs(g[fin] - exp[fin]) <= 2.5e-7 * np.maximum(np.abs(exp[fin]), 1.0))   # <= ~2 ulp of the logs
    # padded int8 batch (benchmarks/forward.py:74-79)
    sigs = [rng.integers(4, 97, n).astype(np.int16) for n in (5, 1, 300, 17)]
    offs = np.zeros(5, dtype=np.int64)
    np.cumsum([len(s) for s in sigs], out=offs[1:])
    flat, d_off = torch.from_numpy(np.concatenate(sigs)).cuda(), torch.from_numpy(offs).cuda()
    data = torch.full((4, 300), 99, dtype=torch.int8, device="cuda")
    lens = torch.zeros(4, dtype=torch.int64, device="cuda")
    rc = native.lib().parpy_b200_hmm_pad_signals(P(flat.data_ptr()), P(d_off.data_ptr()), 4, 300,
                                                 P(data.data_ptr()), P(lens.data_ptr()), None)
    torch.cuda.synchronize()
    assert rc == 0 and lens.cpu().tolist() == [5, 1, 300, 17]
    exp = np.zeros((4, 300), dtype=np.int8)
    for i, s in enumerate(sigs):
        exp[i, :len(s)] = s
    assert np.array_equal(data.cpu().numpy(), exp)


def test_read_model_from_the_reference_3mer_file_and_score_the_fixture(native):
    # tests/golden/3mer-model.hdf5 is the reference's test/data/3mer-model.hdf5, byte for byte
    import os
    from conftest import GOLDEN
    from parpy_b200 import hmm as hmm_mod
    hmm = hmm_mod.read_model(os.path.join(GOLDEN, "3mer-model.hdf5"))
    stored = load_model("3mer")
    for key in ("trans1", "trans2", "output_prob", "initial_prob"):
        g, e = hmm[key].cpu().numpy().reshape(-1), stored[key].numpy().reshape(-1)
        assert np.array_equal(np.isneginf(g), np.isneginf(e)), key
        fin = np.isfinite(e)
        assert np.all(np.abs(g[fin] - e[fin]) <= 2.5e-7 * np.maximum(np.abs(e[fin]), 1.0)), key
    assert float(hmm["gamma"]) == float(stored["gamma"]) and int(hmm["num_states"]) == 1024
    assert float(hmm["synthetic_248"]) == float(stored["synthetic_248"])
    seqs = to_dev(load_signals())
    res = hmm_mod.forward_parpy(hmm, seqs, 512).cpu().numpy()
    assert np.allclose(res, load_expected("3mer"), atol=1e-5, rtol=1e-5)


def test_large_batches_long_sequences_and_side_streams(native, oracle_mod):
    from parpy_b200 import synthetic
    hmm = synthetic.hmm_model(5, seed=41)
    dh = to_dev(hmm)
    # 5000 sequences (more than the 4096 the scheduler sorts): every result equals the small-batch result
    many = synthetic.hmm_sequences(5000, 1, 40, seed=42)
    rc, res, _, _ = cabi_forward(native, dh, to_dev(many))
    assert rc == 0, native.error_message()
    got = res.cpu().numpy()
    idx = np.arange(0, 5000, 97)
    sub = {"data": many["data"][idx].contiguous(), "lens": many["lens"][idx].contiguous(),
           "maxlen": many["maxlen"], "num_instances": torch.tensor(len(idx))}
    rc, res2, _, _ = cabi_forward(native, dh, to_dev(sub))
    assert rc == 0 and np.array_equal(res2.cpu().numpy(), got[idx])
    assert max_rel(got[idx], oracle_mod.forward(hmm, sub)) <= REL_ORACLE
    # one long sequence (40000 steps): finite, and a prefix is more likely than the whole
    longs = synthetic.hmm_sequences(2, 40000, 40000, seed=43)
    longs["lens"][1] = 20000
    rc, res, _, _ = cabi_forward(native, dh, to_dev(longs))
    r = res.cpu().numpy()
    assert rc == 0 and np.isfinite(r).all() and r[1] > r[0]
    # two side streams in flight at once: each has its own scratch
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    a, b = to_dev(synthetic.hmm_sequences(300, 5, 200, seed=44)), to_dev(synthetic.hmm_sequences(200, 5, 200, seed=45))
    torch.cuda.synchronize()
    with torch.cuda.stream(s1):
        rc1, r1, _, _ = cabi_forward(native, dh, a)
    with torch.cuda.stream(s2):
        rc2, r2, _, _ = cabi_forward(native, dh, b)
    torch.cuda.synchronize()
    rc3, e1, _, _ = cabi_forward(native, dh, a)
    rc4, e2, _, _ = cabi_forward(native, dh, b)
    torch.cuda.synchronize()
    assert rc1 == rc2 == rc3 == rc4 == 0
    assert torch.equal(r1, e1) and torch.equal(r2, e2)


# ---- the static schedule and the observation check --------------------------------------------------------
def _schedule(native, lens, clusters):
    d = lens.cuda()
    out = torch.full((len(lens),), -1, dtype=torch.int32, device="cuda")
    rc = native.lib().parpy_b200_forward_schedule(ctypes.c_void_p(d.data_ptr()), len(lens), clusters,
                                                  ctypes.c_void_p(out.data_ptr()),
                                                  ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, native.error_message()
    return out.cpu().numpy()


@pytest.mark.parametrize("batch,lo,hi,clusters", [(500, 1000, 4000, 33), (62, 1000, 4000, 33), (4096, 1, 300, 37),
                                                  (100, 2000, 2000, 148), (7, 5, 9, 33), (1000, 10, 100000, 16)])
def test_static_schedule_is_a_partition_and_beats_greedy_packing(native, batch, lo, hi, clusters):
    from parpy_b200 import dist, synthetic
    lens = synthetic.hmm_sequences(batch, lo, min(hi, 300), seed=batch)["lens"] if hi > 4000 else \
        synthetic.hmm_sequences(batch, lo, hi, seed=batch)["lens"]
    if hi > 4000:   # a heavy tail: a few very long sequences among short ones
        lens = lens.clone()
        lens[::97] = hi
    cl = _schedule(native, lens, clusters)
    used = min(clusters, batch)
    assert cl.min() >= 0 and cl.max() < used                       # every sequence has exactly one cluster
    loads = np.bincount(cl, weights=lens.numpy().astype(np.float64), minlength=used)
    greedy = dist.cluster_schedule(lens.numpy(), clusters)          # longest first to the least loaded
    assert loads.max() <= greedy.max()
    assert np.array_equal(cl, _schedule(native, lens, clusters))   # deterministic
    if batch == 500:
        # the benchmark batch on its 33 clusters: greedy leaves 2 %, the repaired schedule under 0.1 %
        assert loads.max() / loads.mean() < 1.001 < greedy.max() / greedy.mean()


def test_results_do_not_depend_on_the_number_of_resident_clusters(native, monkeypatch):
    from parpy_b200 import synthetic
    hmm, seqs = to_dev(synthetic.hmm_model(6, seed=2)), to_dev(synthetic.hmm_sequences(90, 1, 50, seed=3))
    base = {}
    for flags in (0, FLAGS["log_space"], FLAGS["scaled"]):
        rc, base[flags], _, _ = cabi_forward(native, hmm, seqs, flags)
        assert rc == 0, native.error_message()
    assert torch.equal(base[0], base[FLAGS["scaled"]])          # the default for 4096 k-mers and more
    assert max_rel(base[0].cpu().numpy(), base[FLAGS["log_space"]].cpu().numpy()) <= REL_ORACLE
    for n in ("1", "2", "7"):
        monkeypatch.setenv("PARPY_B200_FWD_CLUSTERS", n)
        for flags in base:
            rc, res, _, _ = cabi_forward(native, hmm, seqs, flags)
            assert rc == 0, native.error_message()
            assert torch.equal(res, base[flags])


def test_table_height_given_or_not_same_bits(native):
    # parpy_b200_forward_ex knows the height of the emission table; for the scaled kernel a prologue then
    # writes the exponentials of the whole table once per call and the kernel reads factors instead of
    # taking the exponential per use. Same exponential, so the results are the same bits as through
    # parpy_b200_forward, which cannot know how many rows the table has.
    from parpy_b200 import synthetic
    for k in (5, 6, 7):
        hmm, seqs = to_dev(synthetic.hmm_model(k, seed=60 + k)), to_dev(synthetic.hmm_sequences(11, 2, 90, seed=70 + k))
        for flags in (0, FLAGS["scaled"], FLAGS["log_space"]):
            rc, a, _, _ = cabi_forward(native, hmm, seqs, flags)
            rc2, b, _, _ = cabi_forward(native, hmm, seqs, flags, entry="parpy_b200_forward_ex")
            assert rc == 0 and rc2 == 0, native.error_message()
            assert torch.equal(a, b), (k, flags)


def test_a_forward_wait_that_gives_up_reaches_the_host(native):
    # The scaled kernel's waits for its neighbours' layer-0 values are bounded; when one runs out
    # the kernel raises status bit 2 instead of hanging. Here a probe CTA waits on a barrier nothing
    # completes (no other CTA involved, nothing in flight), gives up after 64 polls, and the host
    # sees the bit; a forward pass that follows is healthy and leaves the word clean.
    from parpy_b200 import hmm as hmm_mod, synthetic
    clean = {"length_clamped": False, "observation_clamped": False, "wait_timed_out": False}
    hmm_mod.forward_status()
    assert hmm_mod.forward_status() == clean
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert native.lib().parpy_b200_forward_wait_probe(64, stream) == 0, native.error_message()
    assert hmm_mod.forward_status() == dict(clean, wait_timed_out=True)
    assert hmm_mod.forward_status() == clean                                  # read-and-clear
    hmm, seqs = to_dev(synthetic.hmm_model(6, seed=3)), to_dev(synthetic.hmm_sequences(9, 5, 80, seed=4))
    # A caller that never reads the status word still learns of it: the kernel also sets a word in
    # pinned host memory, and the next forward call on the device refuses to launch until the status
    # has been read.
    assert native.lib().parpy_b200_forward_wait_probe(0, stream) == 0
    torch.cuda.synchronize()
    rc, _, _, _ = cabi_forward(native, hmm, seqs)
    assert rc != 0 and "ran out" in native.error_message()
    assert hmm_mod.forward_status() == dict(clean, wait_timed_out=True)
    rc, a, _, _ = cabi_forward(native, hmm, seqs)
    rc2, b, _, _ = cabi_forward(native, hmm, seqs, FLAGS["log_space"])
    assert rc == 0 and rc2 == 0 and max_rel(a.cpu().numpy(), b.cpu().numpy()) <= REL_ORACLE
    assert hmm_mod.forward_status() == clean
    assert native.lib().parpy_b200_forward_wait_probe(-1, stream) != 0 and "outside" in native.error_message()


def test_out_of_range_observations_are_clamped_and_flagged(native):
    # A byte that is not a row of the emission table (>= n_obs) inside a sequence: with n_obs given
    # the kernels read row n_obs - 1 instead of memory past the table and raise status bit 1.
    import parpy_b200 as parpy
    from parpy_b200 import hmm as hmm_mod, synthetic
    for k in (3, 5, 6):
        hmm = synthetic.hmm_model(k, seed=k)
        seqs = synthetic.hmm_sequences(5, 30, 60, seed=k + 1, pad_value=0)
        good = {k2: (v.clone() if isinstance(v, torch.Tensor) else v) for k2, v in seqs.items()}
        good["data"][2, 17] = 100                                 # the last valid level
        bad = {k2: (v.clone() if isinstance(v, torch.Tensor) else v) for k2, v in seqs.items()}
        bad["data"][2, 17] = -56                                  # byte 200 on the host side of a staged array
        hmm_mod.forward_status()
        opts = parpy.par({"inst": parpy.threads(5)})
        want = torch.zeros(5)
        hmm_mod.forward_kernel(hmm, good, want, None, None, opts=opts)
        assert hmm_mod.forward_status() == {"length_clamped": False, "observation_clamped": False, "wait_timed_out": False}
        got = torch.zeros(5)
        hmm_mod.forward_kernel(hmm, bad, got, None, None, opts=opts)
        assert hmm_mod.forward_status() == {"length_clamped": False, "observation_clamped": True, "wait_timed_out": False}
        assert torch.equal(got, want)
        assert hmm_mod.forward_status() == {"length_clamped": False, "observation_clamped": False, "wait_timed_out": False}
    # Viterbi: same rule, its own status word
    hmm = hmm_mod.to_device(synthetic.hmm_model(5, seed=9))
    good = hmm_mod.to_device(good)
    bad = hmm_mod.to_device(bad)
    hmm_mod.viterbi_status()
    want, _ = hmm_mod.viterbi(hmm, good, 32, 8)
    assert hmm_mod.viterbi_status() == {"wait_timed_out": False, "observation_clamped": False}
    got, _ = hmm_mod.viterbi(hmm, bad, 32, 8, check=False)
    assert hmm_mod.viterbi_status() == {"wait_timed_out": False, "observation_clamped": True}
    assert torch.equal(got, want)


@pytest.mark.parametrize("k,nthreads", [(4, 2048), (4, 4096), (5, 2048), (5, 16384)])
def test_transcription_of_the_emitted_cuda_agrees_with_the_oracle(native, oracle_mod, k, nthreads):
    # oracle/parpy_emitted.cu: the program ParPy's compiler emits for forward_kernel with
    # 'state': threads(nthreads) > 1024 (one launch per time step, two-kernel reductions), written
    # out by hand; it is the benchmark's "ParPy-generated CUDA" arm, so it has to compute the same
    # thing: against the CPU oracle, and against this library's kernel on the same inputs.
    from parpy_b200 import synthetic
    if not oracle_mod.parpy_emitted_available():
        pytest.skip("oracle/libparpy_emitted.so not built")
    hmm = synthetic.hmm_model(k, seed=40 + k)
    seqs = synthetic.hmm_sequences(9, 1, 70, seed=50 + k, pad_value=0)
    exp = oracle_mod.forward(hmm, seqs)
    got = oracle_mod.parpy_emitted_forward(to_dev(hmm), to_dev(seqs), nthreads).cpu().numpy()
    assert max_rel(got, exp) <= REL_ORACLE
    rc, res, _, _ = cabi_forward(native, to_dev(hmm), to_dev(seqs))
    assert rc == 0 and max_rel(res.cpu().numpy(), got) <= REL_ORACLE


@pytest.mark.parametrize("finite", ["0", "1"])
def test_7mer_zero_probabilities_in_every_table(native, oracle_mod, monkeypatch, finite):
    # -inf log-probabilities in the emission table (whole rows and single k-mers), in the transition
    # table and in the duration table: dead states stay exactly -inf and no alpha turns into NaN; an
    # impossible sequence scores NaN, the (-inf) - (-inf) of the reference's final reduction
    # (benchmarks/forward.py:168-173). PARPY_B200_FWD_FINITE=1 runs the variant that keeps log 0 as a
    # large negative number inside the kernel and must give the same answers.
    from parpy_b200 import synthetic
    monkeypatch.setenv("PARPY_B200_FWD_FINITE", finite)
    hmm = synthetic.hmm_model(7, seed=61)
    seqs = synthetic.hmm_sequences(6, 3, 60, seed=62, pad_value=0)
    hmm["output_prob"] = hmm["output_prob"].clone()
    hmm["trans1"] = hmm["trans1"].clone()
    hmm["trans2"] = hmm["trans2"].clone()
    last = int(seqs["data"][2, int(seqs["lens"][2]) - 1].item())
    hmm["output_prob"][last, :] = -np.inf                     # sequence 2 becomes impossible at its last step
    hmm["output_prob"][:, 5::97] = -np.inf                    # some k-mers never emit anything
    hmm["trans1"][3::11, 1] = -np.inf                         # some k-mer transitions are impossible
    hmm["trans2"][9] = -np.inf                                # one duration never starts
    exp, exp_alpha = oracle_mod.forward(hmm, seqs, want_alpha=True)
    rc, res, a1, a2 = cabi_forward(native, to_dev(hmm), to_dev(seqs), 2, alpha=True)
    assert rc == 0, native.error_message()
    got = res.cpu().numpy()
    dead = np.isnan(exp)
    assert dead[2] and not dead.all() and np.array_equal(np.isnan(got), dead)
    assert max_rel(got[~dead], exp[~dead]) <= REL_ORACLE
    for i in range(6):
        a = (a1 if int(seqs["lens"][i]) & 1 else a2)[i].cpu().numpy()
        assert not np.isnan(a).any()
        assert np.array_equal(np.isneginf(a), np.isneginf(exp_alpha[i]))
        assert max_rel(a, exp_alpha[i]) <= REL_ORACLE
