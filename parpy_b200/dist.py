"""Multi-GPU sharding for the batched paths: one process per GPU, sequences (or
row blocks) partitioned across ranks, every rank runs the single-GPU kernel on
its shard, and one all-gather of the per-sequence results is the only
collective. The reference has no multi-device code; this module is additive.

The partition is a deterministic function of the lengths, so every rank
computes the same assignment without communicating.
"""
import numpy as np


def lpt_partition(lens, world):
    """Longest-processing-time bin packing: sequences sorted by length
    (descending, index ascending on ties) are assigned one by one to the rank
    with the least total length (lowest rank on ties). Returns ``world`` sorted
    int64 index arrays."""
    lens = np.asarray(lens, dtype=np.int64)
    order = np.lexsort((np.arange(len(lens)), -lens))
    load = np.zeros(world, dtype=np.int64)
    bins = [[] for _ in range(world)]
    for i in order:
        r = int(np.argmin(load))
        bins[r].append(int(i))
        load[r] += lens[i]
    return [np.array(sorted(b), dtype=np.int64) for b in bins]


def shard_sequences(seqs, rank, world):
    """The ``seqs`` dictionary restricted to this rank's sequences (host side;
    call before moving data to the device) and the global indices it holds."""
    import torch
    lens = seqs["lens"].cpu().numpy() if hasattr(seqs["lens"], "cpu") else np.asarray(seqs["lens"])
    idx = lpt_partition(lens, world)[rank]
    tidx = torch.from_numpy(idx)
    data = seqs["data"].cpu()[tidx] if hasattr(seqs["data"], "cpu") else torch.from_numpy(np.asarray(seqs["data"]))[tidx]
    llens = torch.from_numpy(lens)[tidx]
    maxlen = int(llens.max()) if len(idx) else 1
    local = {
        "data": data[:, :maxlen].contiguous(),
        "lens": llens.contiguous(),
        "maxlen": torch.tensor(maxlen, dtype=torch.int64),
        "num_instances": torch.tensor(len(idx), dtype=torch.int64),
    }
    return local, idx


def gather_results(local_result, lens, group=None):
    """All-gathers the per-sequence results of every rank and returns them in
    the original sequence order. ``lens`` are the global lengths (host), from
    which every rank re-derives the partition."""
    import torch
    import torch.distributed as td
    world = td.get_world_size(group)
    parts = lpt_partition(lens, world)
    width = max(len(p) for p in parts)
    padded = torch.zeros(width, dtype=local_result.dtype, device=local_result.device)
    padded[:local_result.numel()] = local_result
    gathered = [torch.empty_like(padded) for _ in range(world)]
    td.all_gather(gathered, padded, group=group)
    out = torch.empty(sum(len(p) for p in parts), dtype=local_result.dtype, device=local_result.device)
    for r, p in enumerate(parts):
        out[torch.from_numpy(p).to(out.device)] = gathered[r][:len(p)]
    return out


def row_block_partition(row_ptr, world):
    """Contiguous row blocks with balanced non-zero counts for CSR operators:
    returns ``world + 1`` row boundaries."""
    row_ptr = np.asarray(row_ptr, dtype=np.int64)
    nnz = int(row_ptr[-1])
    targets = (np.arange(1, world, dtype=np.int64) * nnz) // world
    cuts = np.searchsorted(row_ptr, targets, side="left")
    return np.concatenate(([0], cuts, [len(row_ptr) - 1])).astype(np.int64)
