"""World-size-2 run of the sharded forward path on CPU ranks (gloo): each rank
scores its LPT shard with the CPU oracle standing in for the GPU kernel, one
all-gather reassembles the per-sequence results in the original order."""
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
