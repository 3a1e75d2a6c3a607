"""Windowed Viterbi decoding: the CPU oracle against an independent NumPy
restatement (CPU), and against the reference's own CUDA and the library's kernel
(GPU). Decoded states are integers: every comparison is exact."""
import numpy as np
import pytest
import torch

from conftest import load_model, load_signals, shortest_reads
from oracle import oracle
from parpy_b200 import synthetic


def viterbi_numpy_single_window(hmm, obs):
    """Plain Viterbi over one window (no re-anchoring), vectorised over states,
    candidate order and strict '>' as in benchmarks/7mer/hmm.cu:116-176."""
    f = np.float32
    N = int(hmm["num_states"])
    K = N // 16
    t1, t2 = hmm["trans1"].numpy(), hmm["trans2"].numpy()
    outp, init = hmm["output_prob"].numpy(), hmm["initial_prob"].numpy()
    gamma, syn = f(float(hmm["gamma"])), f(float(hmm["synthetic_248"]))
    s = np.arange(N)
    kmer, layer = s % K, s // K
    preds = np.stack([j * (K // 4) + (s // 4) % (K // 4) for j in range(4)])           # [4, N]
    tr = (t1[preds % K, s % 4] + t2[layer][None, :]).astype(f)
    p5 = np.where(layer == 15, s, s + K)
    c5 = np.where(layer == 15, gamma, np.where(layer == 14, syn, f(0.0))).astype(f)
    chi = (init + outp[obs[0]][kmer]).astype(f)
    back = []
    with np.errstate(invalid="ignore"):
        for t in range(1, len(obs)):
            cand = np.concatenate([(tr + chi[preds]).astype(f), (c5 + chi[np.minimum(p5, N - 1)]).astype(f)[None]])
            idx = np.concatenate([preds, p5[None]])
            best = np.full(N, -np.inf, dtype=f)
            arg = np.full(N, -1, dtype=np.int64)
            for j in range(5):
                take = cand[j] > best
                best = np.where(take, cand[j], best)
                arg = np.where(take, idx[j], arg)
            back.append(arg)
            chi = (best + outp[obs[t]][kmer]).astype(f)
    cur = int(np.argmax(chi))          # first maximum
    path = [cur]
    for arg in reversed(back):
        cur = int(arg[cur]) if arg[cur] >= 0 else cur
        path.append(cur)
    return np.array(path[::-1], dtype=np.uint32)


def test_oracle_matches_plain_viterbi_inside_one_window():
    hmm = load_model("3mer")
    seqs = load_signals(shortest_reads(2))
    for i in range(2):
        obs = seqs["data"][i, :300].numpy().view(np.uint8)
        one = {"data": seqs["data"][i:i + 1, :300].contiguous(), "lens": torch.tensor([300])}
        got = oracle.viterbi(hmm, one, batch_size=1024, batch_overlap=128)[0]
        assert np.array_equal(got, viterbi_numpy_single_window(hmm, obs))


def test_oracle_windowing_rules():
    hmm = synthetic.hmm_model(3, seed=3)
    seqs = synthetic.hmm_sequences(5, 1, 90, seed=4)
    paths = oracle.viterbi(hmm, seqs, batch_size=16, batch_overlap=4)
    for i, path in enumerate(paths):
        n = int(seqs["lens"][i])
        assert len(path) == n and path.max() < 1024
        # every consecutive pair is an allowed transition of the model, except at a window
        # start, where the reference pins the state at t to the state decoded at t-1
        # (hmm.cu:364-376): there the pair repeats
        K = 64
        for pos, (a, b) in enumerate(zip(path[:-1], path[1:]), start=1):
            la, ka, lb, kb = a // K, a % K, b // K, b % K
            chain = (ka == kb) and (la == lb + 1 or (la == 15 and lb == 15))
            shift = (la == 0) and (kb // 4 == ka % (K // 4))
            restart = pos % (16 - 4) == 0 and a == b
            assert chain or shift or restart, (i, pos, a, b)
    # Windows of two steps: the arg-max of a full window is read one step before its end
    # (hmm.cu:414-434 reads the first chi buffer), so the backward pass can start from a state
    # that nothing reaches at the last step. The reference's back pointer is uninitialised
    # there; oracle and kernel both use the state's first k-mer candidate.
    K = 64
    for path in oracle.viterbi(hmm, seqs, batch_size=2, batch_overlap=0):
        for w in range(0, len(path) - 1, 2):
            a, b = int(path[w]), int(path[w + 1])
            la, ka, lb, kb = a // K, a % K, b // K, b % K
            chain = (ka == kb) and (la == lb + 1 or (la == 15 and lb == 15))
            shift = (la == 0) and (kb // 4 == ka % (K // 4))
            first_candidate = a == (b // 4) % (K // 4)
            assert chain or shift or first_candidate, (w, a, b)
    # a window at least as long as the sequence is plain Viterbi
    obs = seqs["data"][0, :int(seqs["lens"][0])].numpy().view(np.uint8)
    whole = oracle.viterbi(hmm, {"data": seqs["data"][:1], "lens": seqs["lens"][:1]}, 1024, 128)[0]
    assert np.array_equal(whole, viterbi_numpy_single_window(hmm, obs))


# ---- GPU ------------------------------------------------------------------------------------
def _dev(d):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) and v.dim() > 0 else v) for k, v in d.items()}


@pytest.mark.gpu
def test_oracle_agrees_with_the_reference_cuda_on_the_5mer_fixture():
    if not oracle.trellis_available(5):
        pytest.skip("oracle/_ref/trellis_5mer.so has not been built")
    hmm, seqs = load_model("5mer"), load_signals(shortest_reads(3))      # ~2800 steps: 4 windows each
    ref = oracle.trellis_viterbi(5, hmm, seqs)
    ours = oracle.viterbi(hmm, seqs)
    for r, o in zip(ref, ours):
        assert np.array_equal(r, o)


@pytest.mark.gpu
def test_kernel_matches_oracle_on_the_5mer_fixture():
    from parpy_b200 import hmm as hmm_mod
    hmm, seqs = load_model("5mer"), load_signals(shortest_reads(5))
    got = hmm_mod.viterbi_paths(_dev(hmm), _dev(seqs))
    exp = oracle.viterbi(hmm, seqs)
    for g, e in zip(got, exp):
        assert np.array_equal(g, e)


@pytest.mark.gpu
@pytest.mark.parametrize("k,batch,overlap,nseq,maxlen", [(5, 16, 4, 23, 120), (5, 7, 2, 9, 40), (5, 2, 0, 4, 9),
                                                       (6, 32, 8, 5, 100), (7, 1024, 128, 2, 1100)])
def test_kernel_matches_oracle_small_windows_and_ragged_lengths(k, batch, overlap, nseq, maxlen):
    from parpy_b200 import hmm as hmm_mod
    hmm = synthetic.hmm_model(k, seed=10 + k)
    # observations valid over the whole width, then ragged lengths on top (never beyond the data)
    seqs = synthetic.hmm_sequences(nseq, maxlen, maxlen, seed=20 + k)
    lens = torch.randint(1, maxlen + 1, (nseq,), generator=torch.Generator().manual_seed(30 + k))
    lens[0] = 1
    if nseq > 2:
        lens[1] = min(maxlen, batch - overlap)           # exactly one window stride
        lens[2] = min(maxlen, batch)                     # exactly one full window
    if k == 7:
        lens[0], lens[1] = 1100, 897                     # full window + remainder; stride + 1
    seqs["lens"] = lens
    exp = oracle.viterbi(hmm, seqs, batch, overlap)
    got = hmm_mod.viterbi_paths(_dev(hmm), _dev(seqs), batch, overlap)
    for i, (g, e) in enumerate(zip(got, exp)):
        assert np.array_equal(g, e), (i, int(seqs["lens"][i]))


@pytest.mark.gpu
@pytest.mark.parametrize("noise", [0.0, 3e-7, 1e-5, 1e-3])
def test_kernel_matches_oracle_when_candidates_nearly_tie(noise):
    # The kernel decides the winner among the four k-mer candidates once per k-mer when their
    # margin provably exceeds the rounding errors, and evaluates every candidate at every layer
    # otherwise. Models built to sit on that boundary: transition log-probabilities that are
    # equal up to a relative noise of 0 (exact ties), about one ulp, and a few hundred ulps, and
    # emissions quantised to a handful of values so that scores collide; sequences long enough
    # for scores of magnitude 1e4.
    from parpy_b200 import hmm as hmm_mod
    hmm = synthetic.hmm_model(5, seed=41)
    g = torch.Generator().manual_seed(42)
    base = torch.full((1024, 4), -1.3862944, dtype=torch.float32)
    hmm["trans1"] = (base * (1.0 + noise * torch.randn(1024, 4, generator=g))).contiguous()
    hmm["output_prob"] = (torch.round(hmm["output_prob"] * 2.0) / 2.0).contiguous()
    seqs = synthetic.hmm_sequences(3, 2500, 2500, seed=43)
    seqs["lens"] = torch.tensor([2500, 1024, 1500])
    exp = oracle.viterbi(hmm, seqs)
    got = hmm_mod.viterbi_paths(_dev(hmm), _dev(seqs))
    for i, (a, b) in enumerate(zip(got, exp)):
        assert np.array_equal(a, b), (noise, i, int(np.argmax(a != b)))


@pytest.mark.gpu
@pytest.mark.parametrize("k,nseq,lo,hi", [(7, 40, 600, 2600), (6, 150, 300, 1500)])
def test_layer0_exchange_variants_agree_at_scale(monkeypatch, k, nseq, lo, hi):
    # Clusters of 2 to 8 CTAs pass layer 0 either with st.shared::cluster + barrier.cluster or with
    # st.async + mbarriers over four buffers. More sequences than resident clusters, ragged lengths,
    # several windows each; the decoded paths of the two must be identical, run after run.
    from parpy_b200 import hmm as hmm_mod
    hmm = synthetic.hmm_model(k, seed=50 + k)
    seqs = synthetic.hmm_sequences(nseq, lo, hi, seed=60 + k)
    dh, ds = _dev(hmm), _dev(seqs)
    monkeypatch.setenv("PARPY_B200_VIT_ASYNC", "0")
    ref = hmm_mod.viterbi_paths(dh, ds)
    monkeypatch.setenv("PARPY_B200_VIT_ASYNC", "1")
    for rep in range(3):
        got = hmm_mod.viterbi_paths(dh, ds)
        for i, (a, b) in enumerate(zip(got, ref)):
            assert np.array_equal(a, b), (rep, i, int(np.argmax(a != b)))
    # the layout with all 16 layers in registers (512-thread CTAs, twice the CTAs per sequence) against
    # the default one for these sizes (1024-thread CTAs, layers 4..15 in tensor memory), both exchanges
    monkeypatch.setenv("PARPY_B200_VIT_TMEM", "0")
    for async_x in ("0", "1"):
        monkeypatch.setenv("PARPY_B200_VIT_ASYNC", async_x)
        got = hmm_mod.viterbi_paths(dh, ds)
        for i, (a, b) in enumerate(zip(got, ref)):
            assert np.array_equal(a, b), (async_x, i, int(np.argmax(a != b)))


@pytest.mark.gpu
def test_viterbi_argument_checks(native):
    from parpy_b200 import hmm as hmm_mod
    hmm, seqs = _dev(synthetic.hmm_model(3)), _dev(synthetic.hmm_sequences(2, 5, 9))
    with pytest.raises(RuntimeError, match="5 <= k <= 8"):
        hmm_mod.viterbi(hmm, seqs)
    hmm5 = _dev(synthetic.hmm_model(5))
    with pytest.raises(RuntimeError, match="window of"):
        hmm_mod.viterbi(hmm5, seqs, batch_size=8, batch_overlap=8)


@pytest.mark.gpu
def test_a_wait_that_gives_up_reaches_the_host():
    # The decoding kernel's waits for another CTA's data are bounded; when one runs out the kernel
    # raises a status bit instead of hanging. Here a probe CTA waits on a barrier nothing completes
    # (no other CTA involved, nothing in flight), gives up after 64 polls, and the host sees the bit.
    import ctypes
    from parpy_b200 import _native, hmm as hmm_mod
    hmm_mod.viterbi_status()
    assert hmm_mod.viterbi_status() == {"wait_timed_out": False, "observation_clamped": False}
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _native.check(_native.lib().parpy_b200_viterbi_wait_probe(64, stream), "wait_probe")
    assert hmm_mod.viterbi_status() == {"wait_timed_out": True, "observation_clamped": False}
    assert hmm_mod.viterbi_status() == {"wait_timed_out": False, "observation_clamped": False}   # read-and-clear
    # a decode that follows is healthy, and hmm.viterbi raises when the bit is up after its own call
    hmm = hmm_mod.to_device(synthetic.hmm_model(5, seed=1))
    seqs = hmm_mod.to_device(synthetic.hmm_sequences(3, 20, 40, seed=2))
    out, _ = hmm_mod.viterbi(hmm, seqs, 16, 4)
    assert int(out.max()) < 16 * 1024
    _native.check(_native.lib().parpy_b200_viterbi_wait_probe(0, stream), "wait_probe")
    with pytest.raises(RuntimeError, match="wait inside the kernel ran out"):
        hmm_mod.viterbi(hmm, seqs, 16, 4)
    hmm_mod.viterbi(hmm, seqs, 16, 4)
