"""World-size-2 runs of the sharded paths on CPU ranks (gloo), with the CPU
oracle standing in for the GPU kernels: sequences sharded for the forward pass
(one all-gather reassembles the per-sequence results in the original order),
CSR row blocks for SpMV and SDDMM, vector slices for the sum/max reduction."""
import os
import socket

import numpy as np
import torch
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_path):
    import sys
    sys.path.insert(0, ROOT)
    import torch.distributed as td
    from oracle import oracle
    from parpy_b200 import dist, synthetic
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    td.init_process_group("gloo", rank=rank, world_size=world)
    hmm = synthetic.hmm_model(3, seed=11)
    seqs = synthetic.hmm_sequences(13, 5, 60, seed=2)
    local, idx = dist.shard_sequences(seqs, rank, world)
    res = torch.from_numpy(oracle.forward(hmm, local, num_threads=1))
    full = dist.gather_results(res, seqs["lens"].numpy())
    if rank == 0:
        np.save(out_path, full.numpy())
    td.barrier()
    td.destroy_process_group()


def test_two_rank_sharded_forward_matches_single_rank(tmp_path):
    from oracle import oracle
    from parpy_b200 import synthetic
    out = str(tmp_path / "full.npy")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    hmm = synthetic.hmm_model(3, seed=11)
    seqs = synthetic.hmm_sequences(13, 5, 60, seed=2)
    expect = oracle.forward(hmm, seqs)
    assert np.array_equal(np.load(out), expect)


def test_cluster_aware_partition_is_a_partition_and_never_worse():
    from parpy_b200 import dist, synthetic
    lens = synthetic.hmm_sequences(500, 1000, 4000)["lens"].numpy()
    for world in (2, 4, 8):
        parts = dist.partition(lens, world, 33)
        assert sorted(np.concatenate(parts).tolist()) == list(range(500))
        tall = lambda ps: max(dist.rank_makespan(lens[p], 33) for p in ps)
        for other in (dist.lpt_partition(lens, world), dist.balanced_partition(lens, world, 33),
                      dist.packed_partition(lens, world, 33)):
            assert sorted(np.concatenate(other).tolist()) == list(range(500))
            assert tall(parts) <= tall(other)
        # the per-cluster total cannot be below the mean, nor below the longest sequence
        assert tall(parts) >= max(lens.sum() / (33 * world), lens.max())
    # one rank: the schedule of the kernel's own queue (longest first, next free cluster)
    load = dist.cluster_schedule(np.array([5, 9, 2, 7, 3]), 2)
    assert sorted(load.tolist()) == [12, 14]          # 9+3+2 | 7+5
    assert dist.partition(lens, 1, 33)[0].tolist() == list(range(500))
    # the packing model: greedy + repair of the fullest bin never ends above the greedy packing, keeps
    # every sequence in exactly one bin, and reaches the floor when the floor is reachable
    where, load = dist.pack_bins(lens, 33)
    assert load.sum() == lens.sum() and np.array_equal(np.bincount(where, weights=lens, minlength=33), load)
    assert load.max() <= dist.cluster_schedule(lens, 33).max()
    where, load = dist.pack_bins(np.array([5, 9, 2, 7, 3]), 2)
    assert sorted(load.tolist()) == [12, 14]          # no subset sums to 13
    where, load = dist.pack_bins(np.array([8, 7, 6, 5, 4]), 2)
    assert sorted(load.tolist()) == [15, 15]          # greedy gives 17 | 13 (8+5+4 | 7+6); one exchange evens it
    assert dist.pack_bins(np.array([], dtype=np.int64), 4)[1].tolist() == [0, 0, 0, 0]


def _sparse_worker(rank, world, port, out_path):
    import sys
    sys.path.insert(0, ROOT)
    import torch.distributed as td
    from oracle import oracle
    from parpy_b200 import dist, synthetic
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    td.init_process_group("gloo", rank=rank, world_size=world)
    # SpMV: y += A @ x on row blocks balanced by non-zeros
    A = synthetic.zipf_csr(300, 300, mean_nnz=6, cap=64, seed=5)
    g = torch.Generator().manual_seed(3)
    x, y = torch.randn(300, generator=g), torch.randn(300, generator=g)

    def spmv_local(A_local, x, y_local):
        y_local.copy_(torch.from_numpy(oracle.spmv(A_local, x, y_local)))
    dist.spmv_sharded(A, x, y, local_op=spmv_local)
    # SDDMM on mask row blocks
    C = synthetic.uniform_csr(64, 96, 0.1, seed=6)
    C["rows"] = torch.zeros(C["nnz"], dtype=torch.int64)
    Am, Bm = torch.randn(64, 8, generator=g), torch.randn(8, 96, generator=g)
    D = torch.zeros(C["nnz"])

    def sddmm_local(A_rows, B, C_local, D_local, alpha, beta):
        rows = oracle.sddmm_decompress(C_local["crows"])
        C_local["rows"].copy_(torch.from_numpy(rows))
        D_local.copy_(torch.from_numpy(oracle.sddmm(A_rows, B, rows, C_local["cols"], C_local["values"], alpha, beta)))
    dist.sddmm_sharded(Am, Bm, C, D, 1.5, 2.0, local_op=sddmm_local)
    # sum and max of a vector held in slices
    v = torch.randn(1001, generator=g)
    sb = dist.slice_bounds(1001, world)
    pair = dist.sum_max_sharded(v[int(sb[rank]):int(sb[rank + 1])],
                                local_op=lambda t: torch.stack([t.sum(), t.max()]))
    np.savez(out_path + f".{rank}.npz", y=y.numpy(), D=D.numpy(), rows=C["rows"].numpy(), pair=pair.numpy())
    td.barrier()
    td.destroy_process_group()


def test_two_rank_sharded_sparse_kernels_match_single_rank(tmp_path):
    from oracle import oracle
    from parpy_b200 import dist, synthetic
    out = str(tmp_path / "sparse")
    mp.spawn(_sparse_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    A = synthetic.zipf_csr(300, 300, mean_nnz=6, cap=64, seed=5)
    g = torch.Generator().manual_seed(3)
    x, y = torch.randn(300, generator=g), torch.randn(300, generator=g)
    C = synthetic.uniform_csr(64, 96, 0.1, seed=6)
    Am, Bm = torch.randn(64, 8, generator=g), torch.randn(8, 96, generator=g)
    v = torch.randn(1001, generator=g)
    rows = oracle.sddmm_decompress(C["crows"])
    got = [np.load(out + f".{r}.npz") for r in range(2)]
    for z in got:                                   # every rank ends with the complete result
        assert np.array_equal(z["y"], oracle.spmv(A, x, y))
        assert np.array_equal(z["rows"], rows)
        assert np.array_equal(z["D"], oracle.sddmm(Am, Bm, rows, C["cols"], C["values"], 1.5, 2.0))
        assert z["pair"][1] == v.max().item()
        assert abs(z["pair"][0] - v.sum().item()) <= 1e-4 * v.abs().sum().item()
    assert np.array_equal(got[0]["pair"], got[1]["pair"])
    # the row blocks balance non-zeros, cover every row once and are contiguous
    b = dist.row_block_partition(A["rows"], 4)
    assert b[0] == 0 and b[-1] == 300 and (np.diff(b) >= 0).all()
    nz = np.diff(A["rows"].numpy()[b])
    assert nz.sum() == int(A["rows"][-1]) and nz.max() - nz.min() <= 2 * 64
    assert np.array_equal(dist.row_block_partition(A["rows"].numpy(), 4), b)
