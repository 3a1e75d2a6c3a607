#!/usr/bin/env python
"""Benchmark of the hot path: 7-mer HMM forward over a batch of 500 ragged
sequences (lengths uniform in [1000, 4000]).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward pass over the whole batch (all sequences, all time
steps). Prints ONE JSON line on rank 0. Under torchrun the batch is sharded by
sequence over the ranks (strong scaling, the default; `weak` in the line is the
same kernel with a full batch per GPU); every rank drives its own GPU and the
only collective is the final all-gather of the per-sequence log-likelihoods,
inside the timed step.

  value     state-steps/s, whole job, inputs resident in HBM (device-timed)
  e2e       the same metric through the Python call surface with pinned HOST
            arrays: host->device copies of tables and observations and the
            device->host copy of the result inside the timed region
  roofline  algorithmic bytes (8.25 B per state-step: alpha read+write, one
            emission row and one observation byte per sequence-step) over the
            live-measured duration, against the measured HBM copy bandwidth
  cpu_baseline / --impl reference
            the CPU restatement of the reference algorithm (oracle/) on the
            host cores, on a bounded sample of the same workload
  schedule  how evenly rank 0's sequences pack onto its resident clusters
  variants  the log-space kernel (opts.b200['forward'] = 'log_space') and the
            explicitly requested scaled kernel on the same batch (N = 1)
  surrounding
            softmax, sum+max, CSR SpMV and SDDMM on their benchmark shapes, once
            each after the timed region (N = 1; see bench_kernels.py)
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "hmm_forward_7mer_state_steps_per_s"
UNIT = "state-steps/s"
KMER = 7
BATCH = 500
MIN_LEN, MAX_LEN = 1000, 4000
SEED = 1234
FALLBACK_HBM_GBS = 6650.0
L2_FLUSH_BYTES = 256 << 20


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="strong",
                    help="strong (default): the 500-sequence batch sharded over the GPUs; "
                         "weak: 500 sequences per GPU")
    ap.add_argument("--variant", choices=["auto", "five_term", "log_space", "scaled", "streaming"], default="auto")
    ap.add_argument("--ref-cuda", action="store_true",
                    help="also time the reference's own CUDA implementation (oracle/_ref), once")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-surrounding", action="store_true",
                    help="skip the surrounding kernels (softmax, sum+max, SpMV, SDDMM) after the timed region")
    ap.add_argument("--no-variants", action="store_true", help="skip the extra runs of the log-space and scaled kernels")
    ap.add_argument("--batch", type=int, default=BATCH, help=argparse.SUPPRESS)
    ap.add_argument("--kmer", type=int, default=KMER, help=argparse.SUPPRESS)
    ap.add_argument("--min-len", type=int, default=MIN_LEN, help=argparse.SUPPRESS)
    ap.add_argument("--max-len", type=int, default=MAX_LEN, help=argparse.SUPPRESS)
    return ap.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def workload_config(args, world):
    return {
        "workload": f"hmm_forward_{args.kmer}mer",
        "num_states": 16 * 4 ** args.kmer,
        "batch_per_gpu": args.batch if args.scaling == "weak" else None,
        "global_batch": args.batch * (world if args.scaling == "weak" else 1),
        "seed": SEED,
        "seq_len": f"uniform[{args.min_len},{args.max_len}]",
        "obs_levels": 101,
        "parallelism": f"sequence-sharded x{world}",
        "cache": "L2 flushed between timed steps (256 MiB write)",
        "variant": args.variant,
    }


# ---- CPU baseline: the oracle port on the host cores -------------------------------
def cpu_sample(hmm, seqs, cores):
    """A bounded sample of the workload: the first 2*cores sequences cut to 256
    time steps each (about 10 s of CPU work at ~2e7 state-steps/s/core)."""
    import torch
    n = max(2, 2 * cores)
    steps = 256
    sub = {
        "data": seqs["data"][:n, :steps].contiguous(),
        "lens": torch.clamp(seqs["lens"][:n], max=steps).contiguous(),
    }
    desc = f"first {n} sequences of the batch, cut to {steps} time steps, {cores} OpenMP threads"
    return sub, desc


def host_cores():
    """Host threads this process may use: the CPU affinity mask, not OMP_NUM_THREADS
    (launchers such as torchrun set that to 1 for every rank)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def time_cpu_once(hmm, sub, cores):
    from oracle import oracle
    t0 = time.perf_counter()
    oracle.forward(hmm, sub, num_threads=cores)
    dt = time.perf_counter() - t0
    work = int(hmm["num_states"]) * int(sub["lens"].sum())
    return work, dt


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    from oracle import oracle
    from parpy_b200 import synthetic
    cores = host_cores()
    hmm = synthetic.hmm_model(args.kmer, seed=SEED)
    seqs = synthetic.hmm_sequences(args.batch, args.min_len, args.max_len, seed=SEED)
    sub, desc = cpu_sample(hmm, seqs, cores)
    for _ in range(args.warmup):
        time_cpu_once(hmm, sub, cores)
    times, work = [], 0
    for _ in range(args.steps):
        work, dt = time_cpu_once(hmm, sub, cores)
        times.append(dt)
    total = sum(times)
    value = work * args.steps / total
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(args, max(world, args.gpus)),
        "ran_on": "host CPU cores of rank 0 (no GPU, no L2 flush); each step scores the sample below",
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    # Extra, outside the contract's fields: the CUDA implementation the reference ships for this
    # model (benchmarks/7mer/hmm.cu, compiled unmodified into oracle/_ref), once, on the full batch.
    try:
        import torch
        if torch.cuda.is_available() and oracle.trellis_available(args.kmer):
            torch.cuda.set_device(0)
            line["reference_cuda"] = time_reference_cuda(args, hmm, seqs, None,
                                                         synthetic.state_steps(hmm, seqs))
    except Exception as exc:     # the CPU line above is the arm's result; this is a side note
        line["reference_cuda"] = {"unavailable": str(exc)[:200]}
    # Second side note: the CUDA program ParPy's compiler emits for forward_kernel (hand transcription
    # of its code-generation rules, oracle/parpy_emitted.cu), called the way forward_parpy calls it.
    try:
        import torch
        if torch.cuda.is_available() and oracle.parpy_emitted_available():
            torch.cuda.set_device(0)
            line["parpy_emitted_cuda"] = time_parpy_emitted(args, hmm, seqs, synthetic.state_steps(hmm, seqs))
    except Exception as exc:
        line["parpy_emitted_cuda"] = {"unavailable": str(exc)[:200]}
    print(json.dumps(line), flush=True)


# ---- clocks -------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for ln in open(self.path):
                f = [x.strip() for x in ln.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                      "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons),
                       samples=len(sm))
        return out


# ---- our arm ---------------------------------------------------------------------------
def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import ctypes
    import torch
    import torch.distributed as td
    import parpy_b200 as parpy
    from parpy_b200 import _native, dist, hmm as hmm_mod, synthetic

    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    if args.gpus > 1 and world == 1:
        raise SystemExit("launch multi-GPU runs with torchrun (one process per GPU)")
    torch.cuda.set_device(local_rank)
    lib = _native.lib()  # fail loudly if the CUDA library is missing
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        td.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    # ---- inputs: identical tables on every rank ----------------------------------------
    hmm = synthetic.hmm_model(args.kmer, seed=SEED)
    n_states = int(hmm["num_states"])
    # resident clusters of the forward kernel on this GPU (its persistent work queue has that many takers)
    clusters = ctypes.c_int32(0)
    _native.check(lib.parpy_b200_forward_plan(n_states, args.batch, None, None, None, ctypes.byref(clusters)),
                  "forward_plan")
    clusters = int(clusters.value)
    all_seqs = synthetic.hmm_sequences(args.batch, args.min_len, args.max_len, seed=SEED)
    global_lens = all_seqs["lens"].numpy()

    def inputs_for(scaling):
        """(local sequences, partition or None): strong = the one batch sharded over the ranks;
        weak = a batch of that size per rank (same lengths, rank-specific observations)."""
        if scaling == "strong":
            if world == 1:
                return all_seqs, None
            parts = dist.partition(global_lens, world, clusters)
            local, _ = dist.shard_sequences(all_seqs, rank, world, clusters)
            return local, dist.gather_plan(parts, torch.device("cuda", local_rank))
        local = synthetic.hmm_sequences(args.batch, args.min_len, args.max_len, seed=SEED,
                                        data_seed=None if rank == 0 else SEED + 17 * rank)
        return local, None

    dev_hmm = hmm_mod.to_device(hmm)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda")

    def barrier():
        if world > 1:
            td.barrier()
        torch.cuda.synchronize()

    def measure(scaling, variant, with_e2e):
        """Times `steps` forward passes of this rank's share (device-resident inputs, then host
        inputs through the Python call). Returns a dict of this rank's figures."""
        seqs, parts = inputs_for(scaling)
        batch = int(seqs["num_instances"])
        dev_seqs = hmm_mod.to_device(seqs)
        opts = parpy.par({"inst": parpy.threads(max(batch, 1))})
        if variant != "auto":
            opts.b200 = {"forward": variant}
        alpha = None
        if variant == "streaming":
            alpha = (torch.zeros(batch, n_states, device="cuda"), torch.zeros(batch, n_states, device="cuda"))
        a1, a2 = alpha if alpha is not None else (None, None)
        result = torch.zeros(batch, dtype=torch.float32, device="cuda")
        gather_buf = [torch.empty_like(result) for _ in range(world)] if world > 1 and scaling == "weak" else None

        def gather(local_result):
            if world == 1:
                return
            if scaling == "weak":
                td.all_gather(gather_buf, local_result)
            else:
                dist.gather_results(local_result, plan=parts)

        def step_device():
            hmm_mod.forward_kernel(dev_hmm, dev_seqs, result, a1, a2, opts=opts)
            gather(result)

        for _ in range(max(args.warmup, 0)):
            step_device()
        barrier()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        events = []
        barrier()
        for _ in range(args.steps):
            flush.fill_(1)                      # evict L2 between timed steps (untimed)
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            step_device()
            e1.record()
            events.append((e0, e1))
        barrier()
        step_ms = [a.elapsed_time(b) for a, b in events]
        out = {"step_ms": step_ms, "total_ms": sum(step_ms), "clocks": sampler.stop() if rank == 0 else None,
               "work": synthetic.state_steps(hmm, seqs), "bytes": synthetic.forward_algorithmic_bytes(hmm, seqs),
               "batch": batch, "result": result, "seqs": seqs, "e2e_s": 0.0, "h2d": 0, "d2h": 0}
        if not with_e2e:
            return out

        # ---- end to end: pinned host arrays through the public call ----------------------
        pin = lambda d: {k: (v.pin_memory() if isinstance(v, torch.Tensor) and v.dim() > 0 else v) for k, v in d.items()}
        pin_hmm, pin_seqs = pin(hmm), pin(seqs)
        host_result = torch.zeros(batch, dtype=torch.float32).pin_memory()
        out["h2d"] = sum(v.numel() * v.element_size() for d in (pin_hmm, pin_seqs) for v in d.values()
                         if isinstance(v, torch.Tensor) and v.dim() > 0)
        out["d2h"] = host_result.numel() * 4

        def step_e2e():
            hmm_mod.forward_kernel(pin_hmm, pin_seqs, host_result, a1, a2, opts=opts)
            if world > 1:
                gather(host_result.cuda(non_blocking=True))

        for _ in range(min(args.warmup, 2)):
            step_e2e()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step_e2e()
        barrier()
        out["e2e_s"] = time.perf_counter() - t0
        assert torch.equal(host_result.cuda(), result), "end-to-end result differs from the device-resident run"
        return out

    def reduce_ranks(m):
        """Max time over ranks, work summed over ranks."""
        stats = torch.tensor([m["total_ms"], m["e2e_s"], float(m["work"]), float(m["bytes"])],
                             dtype=torch.float64, device="cuda")
        if world > 1:
            mx, sm = stats.clone(), stats.clone()
            td.all_reduce(mx, op=td.ReduceOp.MAX)
            td.all_reduce(sm, op=td.ReduceOp.SUM)
            return float(mx[0]), float(mx[1]), float(sm[2]), float(sm[3])
        return m["total_ms"], m["e2e_s"], float(m["work"]), float(m["bytes"])

    head = measure(args.scaling, args.variant, with_e2e=True)
    status = hmm_mod.forward_status()            # read-and-clear: clamps met, bounded waits that ran out
    if status["wait_timed_out"]:
        raise SystemExit("a bounded wait inside the forward kernel ran out: the results are not valid")
    total_ms, e2e_s, work, nbytes = reduce_ranks(head)
    weak = None
    if world > 1 and args.scaling == "strong":
        # the same kernel with a full batch on every GPU, as an extra figure
        wm = measure("weak", args.variant, with_e2e=False)
        w_ms, _, w_work, _ = reduce_ranks(wm)
        weak = {"value": w_work * args.steps / (w_ms * 1e-3), "ms_per_step": w_ms / args.steps,
                "global_batch": args.batch * world}

    if rank == 0:
        peak, peak_kind = measured_peak()
        value = work * args.steps / (total_ms * 1e-3)
        # dominant kernel: the resident forward kernel, one launch per step per rank;
        # the step also holds a one-CTA scheduling prologue of a few microseconds
        launch_s = statistics.mean(head["step_ms"]) * 1e-3
        achieved = head["bytes"] / launch_s / 1e9
        lens_local = head["seqs"]["lens"].numpy()
        import numpy as np
        if len(lens_local) <= 4096:     # the static schedule the kernel built for rank 0's share
            owner = hmm_mod.forward_schedule(lens_local, clusters)
            loads = np.bincount(owner, weights=lens_local.astype(np.float64), minlength=min(clusters, len(lens_local)))
            mx, mean = int(loads.max()), float(loads.mean())
        else:                           # work queue: longest-first greedy packing as the model
            mx, mean = dist.cluster_balance(lens_local, clusters)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, world),
            "e2e": {"value": work * args.steps / e2e_s, "unit": UNIT,
                    "h2d_bytes_per_step": int(head["h2d"]), "d2h_bytes_per_step": int(head["d2h"])},
            # per step and rank: the schedule kernel, the forward kernel and, for the scaled kernel, the
            # prologue that writes the exponentials of the emission table
            "gpu_launches": (3 if args.variant in ("auto", "scaled") and args.kmer >= 6
                             and "PARPY_B200_SCALED_EXPTAB_OFF" not in os.environ else 2) * args.steps * world,
            "clocks": head["clocks"],
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": ncu_traffic_bytes(args, head["h2d"]),
                         "peak_source": peak_kind,
                         "note": "algorithmic bytes (8.25 B/state-step) per launch over the measured "
                                 "launch duration; alpha stays on chip, so DRAM traffic is far lower"},
            "step_ms": head["step_ms"],
            "arithmetic": (args.variant if args.variant != "auto" else
                           "scaled (what a call without options runs on 4096 k-mers and more)" if args.kmer >= 6
                           else "log_space"),
            "status": status,
            # rank 0's share on its persistent clusters: the launch lasts as long as the busiest
            # cluster's step total, the work done is the mean
            "schedule": {"resident_clusters": clusters, "sequences_rank0": head["batch"],
                         "busiest_cluster_steps": mx, "mean_cluster_steps": mean,
                         "balance": mean / mx if mx else None},
        }
        if weak is not None:
            line["weak"] = weak
        if world == 1 and args.variant == "auto" and not args.no_variants:
            b = head["result"].cpu().numpy()
            line["variants"] = {}
            for name, what in (("log_space", "log-space kernel (opts.b200['forward'] = 'log_space'), same batch"),
                               ("scaled", "linear-domain kernel requested explicitly (opts.b200['forward'] = "
                                          "'scaled'; what a call without options runs on this state space)")):
                sc = measure("strong", name, with_e2e=False)
                a = sc["result"].cpu().numpy()
                line["variants"][name] = {
                    "value": sc["work"] * args.steps / (sc["total_ms"] * 1e-3),
                    "ms_per_step": sc["total_ms"] / args.steps,
                    "max_rel_vs_default": float(abs((a - b) / b).max()), "what": what}
        if world == 1 and not args.no_cpu_baseline:
            cores = host_cores()
            sub, desc = cpu_sample(hmm, all_seqs, cores)
            w, dt = time_cpu_once(hmm, sub, cores)
            line["cpu_baseline"] = {"value": w / dt, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": desc}
        if args.ref_cuda and world == 1:
            line["reference_cuda"] = time_reference_cuda(args, hmm, all_seqs, head["result"], head["work"])
        if world == 1 and not args.no_surrounding:
            del head, flush
            torch.cuda.empty_cache()
            try:
                import bench_kernels
                line["surrounding"] = bench_kernels.surrounding()
            except Exception as exc:            # the headline figures above stand on their own
                line["surrounding"] = {"unavailable": str(exc)[:200]}
        print(json.dumps(line), flush=True)
    if world > 1:
        td.barrier()
        td.destroy_process_group()


# ncu captures (--set full, 66 sequences of 200-400 steps) of the resident kernels measured
# dram__bytes_read.sum = 8.00 MB and dram__bytes_write.sum = 0 B per launch for 7,956,782 B of inputs
# (tables + observations + lengths), the same for the scaled and the log-space kernel: a launch reads
# its inputs from DRAM once and keeps alpha on chip, so DRAM traffic follows the input size, not
# the step count.
NCU_DRAM_BYTES_PER_INPUT_BYTE = 8000000.0 / 7956782.0


def ncu_traffic_bytes(args, input_bytes):
    """DRAM bytes per launch of the resident kernel, scaled from the committed
    ncu capture by input bytes; None for variants that were not captured."""
    if args.variant not in ("auto", "scaled", "log_space") or args.kmer != 7:
        return None
    return NCU_DRAM_BYTES_PER_INPUT_BYTE * input_bytes


def time_parpy_emitted(args, hmm, seqs, work):
    """What ParPy's own compiler would run for this benchmark (benchmarks/forward.py:189-218): the
    emitted one-launch-per-time-step program with result and alpha zero-filled inside the call, for
    the 'state' thread counts its tuner tries above one block; the best is kept (ParPyTuned)."""
    import torch
    from oracle import oracle
    n = int(hmm["num_states"])
    dev = lambda d: {k: (v.cuda() if isinstance(v, torch.Tensor) and v.dim() > 0 else v) for k, v in d.items()}
    dh, ds = dev(hmm), dev(seqs)
    batch = int(seqs["num_instances"])
    alpha = (torch.empty((batch, n), device="cuda"), torch.empty((batch, n), device="cuda"))
    small = {"data": ds["data"][:2, :8].contiguous(), "lens": torch.clamp(ds["lens"][:2], max=8)}
    best = None
    for nthreads in (n, n // 4, n // 16):
        if nthreads <= 1024:
            continue
        oracle.parpy_emitted_forward(dh, small, nthreads)      # load the module
        t0 = time.perf_counter()
        oracle.parpy_emitted_forward(dh, ds, nthreads, alpha=alpha)
        dt = time.perf_counter() - t0
        if best is None or dt < best[0]:
            best = (dt, nthreads)
    return {"value": work / best[0], "unit": UNIT, "seconds": best[0], "state_threads": best[1],
            "what": "hand transcription of the CUDA ParPy emits for forward_kernel (one launch per time step, "
                    "two-kernel reductions, zero fill of alpha inside the call), best of three thread counts"}


def time_reference_cuda(args, hmm, seqs, ours, work):
    """The reference's own CUDA implementation (benchmarks/7mer/hmm.cu compiled
    unmodified into oracle/_ref) on the same batch, host arrays in and out as
    its ABI requires; one run, wall clock."""
    import numpy as np
    import torch
    from oracle import oracle
    if not oracle.trellis_available(args.kmer):
        return {"unavailable": "oracle/_ref has no build for this k"}
    oracle.trellis_forward(args.kmer, hmm, {"data": seqs["data"][:2], "lens": seqs["lens"][:2]})  # warm-up
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ref = oracle.trellis_forward(args.kmer, hmm, seqs)
    dt = time.perf_counter() - t0
    out = {"value": work / dt, "unit": UNIT, "seconds": dt,
           "what": "benchmarks/7mer/hmm.cu forward(), incl. its cudaMalloc/H2D/D2H per call"}
    if ours is not None:
        got = ours.cpu().numpy()
        out["max_rel_vs_ours"] = float(np.max(np.abs(got - ref) / np.abs(ref)))
    return out


if __name__ == "__main__":
    main()
