#!/usr/bin/env python
"""Timing of the kernels that surround the headline path, on the configurations
the reference's tests and benchmarks use (seeded synthetic inputs):

    python bench_kernels.py [--quick] [--only softmax,reduce,spmv,sddmm,spmm,forward5,viterbi]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench_kernels.py --gpus N        # row-block / slice sharded kernels

Prints one JSON line per kernel: device time (CUDA events on the launching
stream, L2 flushed between repetitions), algorithmic bytes, achieved GB/s and
the fraction of the measured HBM copy bandwidth. `bench.py` covers the 7-mer
forward pass and calls :func:`surrounding` for its `surrounding` list; this
script covers softmax, the fused sum+max reduction, row reductions, CSR SpMV,
SDDMM, the 5-mer forward pass and Viterbi. With ``--gpus N`` the sparse kernels
and the reduction run on row blocks / slices, one per rank, followed by the one
all-gather that completes the result (time = max over ranks).
"""
import argparse
import ctypes
import json
import os
import statistics
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch

from parpy_b200 import _native, kernels, synthetic
from parpy_b200 import hmm as hmm_mod

P = ctypes.c_void_p


def hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def timed(fn, reps=10, warmup=3, flush=None):
    """Device time of `fn` per repetition (ms), CUDA events on the current stream,
    `flush` (a buffer larger than the L2) rewritten before every repetition."""
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
    return line


def stream():
    return P(torch.cuda.current_stream().cuda_stream)


class Runner:
    """Shared state of one benchmark run: the library, the L2 flush buffer, the
    seeded generator and the repetition policy."""

    def __init__(self, quick=False, profile=False, reps=None, ref_cuda=False):
        self.lib = _native.lib()
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        self.g = torch.Generator().manual_seed(1234)
        self.quick, self.profile, self.reps, self.ref_cuda = quick, profile, reps, ref_cuda

    def timed(self, fn, reps=10, warmup=3):
        if self.profile:
            reps, warmup = 1, 1
        elif self.reps is not None:
            reps = min(reps, self.reps)
        return timed(fn, reps, warmup, self.flush)


def bench_softmax(r, shapes=((256, 1024), (32768, 1024), (4096, 16384))):
    # the reference test's shape, and shapes large enough to measure bandwidth
    out_lines = []
    for shape in shapes:
        x = torch.randn(shape, generator=r.g, dtype=torch.float32).cuda()
        out = torch.empty_like(x)
        ms = r.timed(lambda: _native.check(r.lib.parpy_b200_softmax(P(x.data_ptr()), shape[0], shape[1],
                                                                    P(out.data_ptr()), stream())))
        # a plain device copy of the same shape under the same timing: what this size allows
        copy_ms = r.timed(lambda: out.copy_(x))
        out_lines.append(report(f"softmax[{shape[0]},{shape[1]}]", ms, 8 * x.numel(),
                                {"copy_same_shape_ms_median": statistics.median(copy_ms)}))
        del x, out
    return out_lines


def bench_reductions(r, rows_too=True):
    # fused sum + max over a long vector (2^30 elements = 4 GiB)
    n = 1 << (26 if r.quick else 30)
    v = torch.empty(n, dtype=torch.float32, device="cuda").normal_(
        generator=torch.Generator(device="cuda").manual_seed(1234))
    lines = []
    ms = r.timed(lambda: kernels.sum_max(v), reps=5)
    lines.append(report(f"sum_max[2^{n.bit_length() - 1}]", ms, 4 * n))
    if rows_too:
        out1 = torch.empty(1, device="cuda")
        ms = r.timed(lambda: _native.check(r.lib.parpy_b200_reduce_rows(0, P(v.data_ptr()), P(out1.data_ptr()),
                                                                        1, n, stream())), reps=5)
        lines.append(report(f"sum_2d[2^{n.bit_length() - 1}]", ms, 4 * n))
        rows = v[: 8192 * 8192].view(8192, 8192)
        outr = torch.empty(8192, device="cuda")
        ms = r.timed(lambda: _native.check(r.lib.parpy_b200_reduce_rows(2, P(rows.data_ptr()), P(outr.data_ptr()),
                                                                        8192, 8192, stream())))
        lines.append(report("max_rows[8192,8192]", ms, 4 * rows.numel()))
    del v
    return lines


def spmv_bytes(nnz, nrows, ncols):
    # value + int64 column per non-zero, row pointer + y read-modify-write per row, x once
    return nnz * 12 + nrows * 8 + nrows * 8 + ncols * 4


def bench_spmv(r):
    # CSR SpMV, power-law rows
    nr = 1 << (20 if r.quick else 22)
    A = synthetic.zipf_csr(nr, nr, mean_nnz=32, cap=4096, seed=1234)
    d = {k: t.cuda() for k, t in A.items() if isinstance(t, torch.Tensor)}
    x = torch.randn(nr, generator=r.g).cuda()
    y = torch.zeros(nr, device="cuda")
    nnz = d["values"].numel()
    ms = r.timed(lambda: _native.check(r.lib.parpy_b200_spmv(P(d["values"].data_ptr()), P(d["rows"].data_ptr()),
                                                             P(d["cols"].data_ptr()), nr, nnz, P(x.data_ptr()),
                                                             P(y.data_ptr()), stream())))
    line = report(f"spmv[{nr}x{nr}, nnz={nnz}]", ms, spmv_bytes(nnz, nr, nr), {"nnz": nnz})
    del d, x, y
    return [line]


def sddmm_bytes(n, k, ncols, nnz):
    # A and B once, per non-zero: int64 column, int64 row written, mask value, result; row pointers
    return 4 * (n * k + k * ncols) + nnz * (8 + 8 + 4 + 4) + 8 * (n + 1)


def bench_sddmm(r, shapes=((8192, 64), (8192, 1024))):
    # SDDMM, 8192 x 8192 mask at 1 %; K = 64 is the benchmark configuration, K = 1024 the
    # reference's other inner dimension (benchmarks/bench.py:206-244), where the dot products
    # are long enough to be bandwidth- rather than latency-bound
    lines = []
    for N, K in shapes:
        C = synthetic.uniform_csr(N, N, 0.01, seed=1234)
        Cd = {"crows": C["crows"].cuda(), "rows": torch.empty(C["nnz"], dtype=torch.int64, device="cuda"),
              "cols": C["cols"].cuda(), "values": C["values"].cuda()}
        Am, Bm = torch.randn(N, K, generator=r.g).cuda(), torch.randn(K, N, generator=r.g).cuda()
        D = torch.empty(C["nnz"], device="cuda")
        for alpha, beta in ((1.0, 0.0), (1.5, 2.0)):
            ms = r.timed(lambda: _native.check(r.lib.parpy_b200_sddmm_csr(
                P(Am.data_ptr()), P(Bm.data_ptr()), P(Cd["crows"].data_ptr()), P(Cd["rows"].data_ptr()),
                P(Cd["cols"].data_ptr()), P(Cd["values"].data_ptr()), P(D.data_ptr()), N, K, N, C["nnz"],
                alpha, beta, stream())))
            lines.append(report(f"sddmm_csr[{N}x{N} 1%, K={K}, alpha={alpha}, beta={beta}]", ms,
                                sddmm_bytes(N, K, N, C["nnz"]), {"nnz": C["nnz"]}))
        del Cd, Am, Bm, D
    return lines


def bench_forward5(r):
    # 5-mer forward: 100 sequences of 2000 steps (latency-bound configuration)
    hmm = synthetic.hmm_model(5)
    seqs = synthetic.hmm_sequences(100, 2000, 2000)
    dh, ds = hmm_mod.to_device(hmm), hmm_mod.to_device(seqs)
    ms = r.timed(lambda: hmm_mod.forward_parpy(dh, ds))
    return [report("hmm_forward_5mer[B=100,T=2000]", ms, synthetic.forward_algorithmic_bytes(hmm, seqs),
                   {"state_steps_per_s": synthetic.state_steps(hmm, seqs) / statistics.median(ms) * 1e3})]


def bench_viterbi(r):
    # windowed Viterbi decoding (windows of 1024 steps, overlap 128), 5-mer and 7-mer models
    lines = []
    for k, nseq, lo, hi in ((5, 100, 2000, 2000), (7, 66, 1000, 4000)):
        hmm = synthetic.hmm_model(k)
        seqs = synthetic.hmm_sequences(nseq, lo, hi)
        dh, ds = hmm_mod.to_device(hmm), hmm_mod.to_device(seqs)
        ms = r.timed(lambda: hmm_mod.viterbi(dh, ds), reps=3, warmup=1)
        work = synthetic.state_steps(hmm, seqs)
        extra = {"state_steps_per_s": work / statistics.median(ms) * 1e3,
                 "backpointer_bytes": int(seqs["lens"].sum()) * (4 ** k // 4) * 32}
        if r.ref_cuda:
            import time
            from oracle import oracle     # measurement only: the reference's own CUDA, built into oracle/_ref
            if oracle.trellis_available(k):
                n = 4
                sub = {"data": seqs["data"][:n].contiguous(), "lens": seqs["lens"][:n].contiguous()}
                oracle.trellis_viterbi(k, hmm, {"data": sub["data"][:1], "lens": sub["lens"][:1]})
                t0 = time.perf_counter()
                oracle.trellis_viterbi(k, hmm, sub, num_parallel=n)
                dt = time.perf_counter() - t0
                extra["reference_cuda_state_steps_per_s"] = int(hmm["num_states"]) * int(sub["lens"].sum()) / dt
                extra["reference_cuda_sample"] = f"first {n} sequences, num_parallel={n}, host arrays in and out"
        lines.append(report(f"viterbi_{k}mer[B={nseq}, len {lo}-{hi}]", ms,
                            synthetic.forward_algorithmic_bytes(hmm, seqs), extra))
    return lines


def bench_spmm(r):
    # CSR SpMM (test/test_spmm.py:16-24 shape family, larger): C += A @ B, A 65536 x 65536 with 32
    # non-zeros per row on average, B dense [65536, 64]
    n, k = 1 << 16, 64
    A = synthetic.zipf_csr(n, n, mean_nnz=32, cap=1024, seed=1234)
    d = {key: t.cuda() for key, t in A.items() if isinstance(t, torch.Tensor)}
    B = torch.randn(n, k, generator=r.g).cuda()
    C = torch.zeros(n, k, device="cuda")
    nnz = d["values"].numel()
    ms = r.timed(lambda: _native.check(r.lib.parpy_b200_spmm(P(d["values"].data_ptr()), P(d["rows"].data_ptr()),
                                                             P(d["cols"].data_ptr()), n, P(B.data_ptr()), k,
                                                             P(C.data_ptr()), stream())))
    # value + column per non-zero, row pointers, B once, C read-modify-write
    nbytes = nnz * 12 + n * 8 + 4 * n * k + 8 * n * k
    return [report(f"spmm[{n}x{n}, nnz={nnz}, B {n}x{k}]", ms, nbytes, {"nnz": nnz, "gathered_bytes": nnz * k * 4})]


SECTIONS = {"softmax": bench_softmax, "reduce": bench_reductions, "spmv": bench_spmv, "sddmm": bench_sddmm,
            "spmm": bench_spmm, "forward5": bench_forward5, "viterbi": bench_viterbi}


def surrounding(reps=5):
    """The surrounding-kernel workloads once each for `bench.py`'s `surrounding`
    list: softmax [256,1024] (+ a bandwidth-sized shape), fused sum+max over 2^30,
    CSR SpMV 4M x 4M, SDDMM 8192^2 at 1 % (K = 64 and 1024). Returns
    [{kernel, ms, gbs, frac_of_hbm}]."""
    r = Runner(reps=reps)
    lines = []
    lines += bench_softmax(r, shapes=((256, 1024), (32768, 1024)))
    lines += bench_reductions(r, rows_too=False)
    lines += bench_spmv(r)
    lines += [l for l in bench_sddmm(r) if "alpha=1.0" in l["kernel"]]
    return [{"kernel": l["kernel"], "ms": l["ms_median"], "gbs": l["gbs_median"],
             "frac_of_hbm": l["frac_of_hbm_median"]} for l in lines]


# ---- row-block / slice sharded kernels, one rank per GPU -----------------------------------
def sharded(args):
    import torch.distributed as td
    from parpy_b200 import dist
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}: launch with torchrun")
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    td.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    r = Runner(quick=args.quick)

    def timed_max(fn, reps=10):
        td.barrier()
        ms = statistics.median(r.timed(fn, reps=reps))
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        td.all_reduce(t, op=td.ReduceOp.MAX)
        return [float(t[0])]

    lines = []
    # SpMV: every rank builds the same matrix from the seed and keeps its row block
    nr = 1 << (20 if args.quick else 22)
    A = synthetic.zipf_csr(nr, nr, mean_nnz=32, cap=4096, seed=1234)
    nnz = int(A["rows"][-1])
    local, bounds = dist.shard_csr(A, rank, world)
    d = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in local.items()}
    del A
    x = torch.randn(nr, generator=r.g).cuda()
    y_local = torch.zeros(d["nrows"], device="cuda")
    sizes = [int(b) for b in (bounds[1:] - bounds[:-1])]

    def spmv_step():
        _native.check(r.lib.parpy_b200_spmv(P(d["values"].data_ptr()), P(d["rows"].data_ptr()),
                                            P(d["cols"].data_ptr()), d["nrows"], d["nnz"], P(x.data_ptr()),
                                            P(y_local.data_ptr()), stream()))
        dist._gather_blocks(y_local, sizes)
    lines.append(report(f"spmv_sharded[{nr}x{nr}, nnz={nnz}, {world} row blocks + all-gather of y]",
                        timed_max(spmv_step), spmv_bytes(nnz, nr, nr), {"n_gpus": world}))
    del d, x, y_local

    # SDDMM: mask rows sharded, A rows follow, B replicated
    N, K = 8192, 64
    C = synthetic.uniform_csr(N, N, 0.01, seed=1234)
    local, bounds = dist.shard_csr(C, rank, world, rows_key="crows")
    Cd = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in local.items()}
    Cd["rows"] = torch.empty(Cd["nnz"], dtype=torch.int64, device="cuda")
    Am = torch.randn(N, K, generator=r.g)[local["row_begin"]:local["row_end"]].contiguous().cuda()
    Bm = torch.randn(K, N, generator=r.g).cuda()
    D = torch.empty(Cd["nnz"], device="cuda")
    edges = [int(C["crows"][int(b)]) for b in bounds]
    nz_sizes = [edges[i + 1] - edges[i] for i in range(world)]

    def sddmm_step():
        _native.check(r.lib.parpy_b200_sddmm_csr(
            P(Am.data_ptr()), P(Bm.data_ptr()), P(Cd["crows"].data_ptr()), P(Cd["rows"].data_ptr()),
            P(Cd["cols"].data_ptr()), P(Cd["values"].data_ptr()), P(D.data_ptr()), Cd["nrows"], K, N, Cd["nnz"],
            1.0, 0.0, stream()))
        dist._gather_blocks(D, nz_sizes)
    lines.append(report(f"sddmm_sharded[{N}x{N} 1%, K={K}, {world} row blocks + all-gather of D]",
                        timed_max(sddmm_step), sddmm_bytes(N, K, N, C["nnz"]), {"n_gpus": world}))

    # sum + max: equal slices of one 2^30 vector
    n = 1 << (26 if args.quick else 30)
    sb = dist.slice_bounds(n, world)
    mine = int(sb[rank + 1] - sb[rank])
    v = torch.empty(mine, dtype=torch.float32, device="cuda").normal_(
        generator=torch.Generator(device="cuda").manual_seed(1234 + rank))
    lines.append(report(f"sum_max_sharded[2^{n.bit_length() - 1}, {world} slices + all-gather of pairs]",
                        timed_max(lambda: dist.sum_max_sharded(v), reps=5), 4 * n, {"n_gpus": world}))
    if rank == 0:
        for l in lines:
            print(json.dumps(l), flush=True)
    td.barrier()
    td.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true", help="smaller SpMV / reduction sizes")
    ap.add_argument("--ref-cuda", action="store_true",
                    help="also time the reference's CUDA Viterbi (needs oracle/_ref, built where the "
                         "reference checkout is present) on a few sequences")
    ap.add_argument("--only", default="", help="comma-separated sections to run: " + ", ".join(SECTIONS)
                    + " (default: all)")
    ap.add_argument("--profile", action="store_true",
                    help="one warm-up and one timed launch per kernel (for captures under a profiler)")
    ap.add_argument("--gpus", type=int, default=1, help="N > 1: the sharded sparse kernels and reduction")
    args = ap.parse_args()
    if args.gpus > 1:
        return sharded(args)
    r = Runner(quick=args.quick, profile=args.profile, ref_cuda=args.ref_cuda)
    for name, fn in SECTIONS.items():
        if not args.only or name in args.only.split(","):
            for line in fn(r):
                print(json.dumps(line), flush=True)


if __name__ == "__main__":
    sys.exit(main())
