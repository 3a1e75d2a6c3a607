"""Timing of the kernels that surround the headline path, on the configurations
the reference's tests and benchmarks use (seeded synthetic inputs):

    python -m parpy_b200.bench_kernels [--quick]

Prints one JSON line per kernel: device time (CUDA events on the launching
stream, L2 flushed between repetitions), algorithmic bytes, achieved GB/s and
the fraction of the measured HBM copy bandwidth. `bench.py` at the repository
root covers the 7-mer forward pass; this module covers softmax, the fused
sum+max reduction, row reductions, CSR SpMV, SDDMM and the 5-mer forward pass.
"""
import argparse
import ctypes
import json
import os
import statistics
import sys

import torch

from . import _native, kernels, synthetic
from . import hmm as hmm_mod

P = ctypes.c_void_p
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def timed(fn, reps=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ms = []
    for _ in range(reps):
        if flush is not None:
            flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
    return ms


def report(name, ms, nbytes, extra=None):
    peak, kind = hbm_peak()
    best, med = min(ms), statistics.median(ms)
    line = {"kernel": name, "ms_median": med, "ms_best": best, "algorithmic_bytes": nbytes,
            "gbs_median": nbytes / med / 1e6, "gbs_best": nbytes / best / 1e6,
            "frac_of_hbm_median": nbytes / med / 1e6 / peak, "hbm_peak_gbs": peak, "peak_source": kind}
    if extra:
        line.update(extra)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true", help="smaller SpMV / reduction sizes")
    ap.add_argument("--ref-cuda", action="store_true",
                    help="also time the reference's CUDA Viterbi (needs oracle/_ref, built where the "
                         "reference checkout is present) on a few sequences")
    ap.add_argument("--only", default="", help="comma-separated sections to run: softmax, reduce, spmv, "
                                               "sddmm, forward5, viterbi (default: all)")
    ap.add_argument("--profile", action="store_true",
                    help="one warm-up and one timed launch per kernel (for captures under a profiler)")
    args = ap.parse_args()
    want = lambda name: not args.only or name in args.only.split(",")
    if args.profile:
        global timed
        plain = timed
        timed = lambda fn, reps=1, warmup=1, flush=None: plain(fn, 1, 1, flush)
    lib = _native.lib()
    stream = lambda: P(torch.cuda.current_stream().cuda_stream)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    g = torch.Generator().manual_seed(1234)

    # softmax: the reference test's shape, and a shape large enough to measure bandwidth
    for shape in ((256, 1024), (32768, 1024), (4096, 16384)) if want("softmax") else ():
        x = torch.randn(shape, generator=g, dtype=torch.float32).cuda()
        out = torch.empty_like(x)
        ms = timed(lambda: _native.check(lib.parpy_b200_softmax(P(x.data_ptr()), shape[0], shape[1],
                                                                P(out.data_ptr()), stream())), flush=flush)
        # a plain device copy of the same shape under the same timing: what this size allows
        copy_ms = timed(lambda: out.copy_(x), flush=flush)
        report(f"softmax[{shape[0]},{shape[1]}]", ms, 8 * x.numel(),
               {"copy_same_shape_ms_median": statistics.median(copy_ms)})
        del x, out

    if want("reduce"):
        bench_reductions(args, lib, stream, flush)
    if want("spmv"):
        bench_spmv(args, lib, stream, flush, g)
    if want("sddmm"):
        bench_sddmm(lib, stream, flush, g)
    if want("forward5"):
        bench_forward5(flush)
    if want("viterbi"):
        bench_viterbi(args, flush)


def bench_reductions(args, lib, stream, flush):
    # fused sum + max over a long vector (2^30 elements = 4 GiB)
    n = 1 << (26 if args.quick else 30)
    v = torch.empty(n, dtype=torch.float32, device="cuda").normal_(generator=torch.Generator(device="cuda").manual_seed(1234))
    ms = timed(lambda: kernels.sum_max(v), reps=5, flush=flush)
    report(f"sum_max[2^{n.bit_length() - 1}]", ms, 4 * n)
    out1 = torch.empty(1, device="cuda")
    ms = timed(lambda: _native.check(lib.parpy_b200_reduce_rows(0, P(v.data_ptr()), P(out1.data_ptr()), 1, n, stream())),
               reps=5, flush=flush)
    report(f"sum_2d[2^{n.bit_length() - 1}]", ms, 4 * n)
    rows = v[: 8192 * 8192].view(8192, 8192)
    outr = torch.empty(8192, device="cuda")
    ms = timed(lambda: _native.check(lib.parpy_b200_reduce_rows(2, P(rows.data_ptr()), P(outr.data_ptr()), 8192, 8192, stream())),
               flush=flush)
    report("max_rows[8192,8192]", ms, 4 * rows.numel())
    del v, rows


def bench_spmv(args, lib, stream, flush, g):
    # CSR SpMV, power-law rows
    nr = 1 << (20 if args.quick else 22)
    A = synthetic.zipf_csr(nr, nr, mean_nnz=32, cap=4096, seed=1234)
    d = {k: t.cuda() for k, t in A.items() if isinstance(t, torch.Tensor)}
    x = torch.randn(nr, generator=g).cuda()
    y = torch.zeros(nr, device="cuda")
    nnz = d["values"].numel()
    ms = timed(lambda: _native.check(lib.parpy_b200_spmv(P(d["values"].data_ptr()), P(d["rows"].data_ptr()),
                                                         P(d["cols"].data_ptr()), nr, nnz, P(x.data_ptr()),
                                                         P(y.data_ptr()), stream())), flush=flush)
    report(f"spmv[{nr}x{nr}, nnz={nnz}]", ms, nnz * 12 + nr * 12 + nr * 4 + nr * 4, {"nnz": nnz})
    del d, x, y


def bench_sddmm(lib, stream, flush, g):
    # SDDMM, 8192 x 8192 mask at 1 %, K = 64
    N, K = 8192, 64
    C = synthetic.uniform_csr(N, N, 0.01, seed=1234)
    Cd = {"crows": C["crows"].cuda(), "rows": torch.empty(C["nnz"], dtype=torch.int64, device="cuda"),
          "cols": C["cols"].cuda(), "values": C["values"].cuda()}
    Am, Bm = torch.randn(N, K, generator=g).cuda(), torch.randn(K, N, generator=g).cuda()
    D = torch.empty(C["nnz"], device="cuda")
    for alpha, beta in ((1.0, 0.0), (1.5, 2.0)):
        ms = timed(lambda: _native.check(lib.parpy_b200_sddmm_csr(
            P(Am.data_ptr()), P(Bm.data_ptr()), P(Cd["crows"].data_ptr()), P(Cd["rows"].data_ptr()),
            P(Cd["cols"].data_ptr()), P(Cd["values"].data_ptr()), P(D.data_ptr()), N, K, N, C["nnz"],
            alpha, beta, stream())), flush=flush)
        nbytes = 4 * (Am.numel() + Bm.numel()) + C["nnz"] * (8 + 8 + 4 + 4) + 8 * (N + 1)
        report(f"sddmm_csr[{N}x{N} 1%, K={K}, alpha={alpha}, beta={beta}]", ms, nbytes, {"nnz": C["nnz"]})


def bench_forward5(flush):
    # 5-mer forward: 100 sequences of 2000 steps (latency-bound configuration)
    hmm = synthetic.hmm_model(5)
    seqs = synthetic.hmm_sequences(100, 2000, 2000)
    dh, ds = hmm_mod.to_device(hmm), hmm_mod.to_device(seqs)
    ms = timed(lambda: hmm_mod.forward_parpy(dh, ds), flush=flush)
    report("hmm_forward_5mer[B=100,T=2000]", ms, synthetic.forward_algorithmic_bytes(hmm, seqs),
           {"state_steps_per_s": synthetic.state_steps(hmm, seqs) / statistics.median(ms) * 1e3})


def bench_viterbi(args, flush):
    # windowed Viterbi decoding (windows of 1024 steps, overlap 128), 5-mer and 7-mer models
    for k, nseq, lo, hi in ((5, 100, 2000, 2000), (7, 66, 1000, 4000)):
        hmm = synthetic.hmm_model(k)
        seqs = synthetic.hmm_sequences(nseq, lo, hi)
        dh, ds = hmm_mod.to_device(hmm), hmm_mod.to_device(seqs)
        ms = timed(lambda: hmm_mod.viterbi(dh, ds), reps=3 if args.profile is False else 1, warmup=1, flush=flush)
        work = synthetic.state_steps(hmm, seqs)
        extra = {"state_steps_per_s": work / statistics.median(ms) * 1e3,
                 "backpointer_bytes": int(seqs["lens"].sum()) * (4 ** k // 4) * 32}
        if args.ref_cuda:
            import time
            sys.path.insert(0, ROOT)
            from oracle import oracle
            if oracle.trellis_available(k):
                n = 4
                sub = {"data": seqs["data"][:n].contiguous(), "lens": seqs["lens"][:n].contiguous()}
                oracle.trellis_viterbi(k, hmm, {"data": sub["data"][:1], "lens": sub["lens"][:1]})
                t0 = time.perf_counter()
                oracle.trellis_viterbi(k, hmm, sub, num_parallel=n)
                dt = time.perf_counter() - t0
                extra["reference_cuda_state_steps_per_s"] = int(hmm["num_states"]) * int(sub["lens"].sum()) / dt
                extra["reference_cuda_sample"] = f"first {n} sequences, num_parallel={n}, host arrays in and out"
        report(f"viterbi_{k}mer[B={nseq}, len {lo}-{hi}]", ms, synthetic.forward_algorithmic_bytes(hmm, seqs), extra)


if __name__ == "__main__":
    sys.exit(main())
