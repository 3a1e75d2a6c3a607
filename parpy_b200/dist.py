"""Multi-GPU sharding for the batched paths: one process per GPU, sequences (or
row blocks) partitioned across ranks, every rank runs the single-GPU kernel on
its shard, and one all-gather of the per-sequence (per-row, per-non-zero)
results is the only collective. The reference has no multi-device code; this
module is additive.

Every partition is a deterministic function of host-side sizes, so all ranks
compute the same assignment without communicating. Nothing here hands another
GPU's memory to a kernel: ranks exchange results through the process group only.
"""
import heapq

import numpy as np


# ---- sequences (HMM forward / Viterbi) ------------------------------------------------
def _longest_first(lens):
    lens = np.asarray(lens, dtype=np.int64)
    return lens, np.lexsort((np.arange(len(lens)), -lens))


def lpt_partition(lens, world):
    """Longest-processing-time bin packing: sequences sorted by length
    (descending, index ascending on ties) are assigned one by one to the rank
    with the least total length (lowest rank on ties). Returns ``world`` sorted
    int64 index arrays."""
    lens, order = _longest_first(lens)
    load = np.zeros(world, dtype=np.int64)
    bins = [[] for _ in range(world)]
    for i in order:
        r = int(np.argmin(load))
        bins[r].append(int(i))
        load[r] += lens[i]
    return [np.array(sorted(b), dtype=np.int64) for b in bins]


def cluster_schedule(lens, clusters):
    """What the forward kernel's work queue does with one rank's sequences: the
    resident clusters pop sequences longest first, each taking the next one when
    it finishes its current one (time = number of steps). Returns the per-cluster
    step totals."""
    lens, order = _longest_first(lens)
    clusters = max(1, min(int(clusters), max(len(lens), 1)))
    heap = [(0, c) for c in range(clusters)]
    load = np.zeros(clusters, dtype=np.int64)
    for i in order:
        t, c = heapq.heappop(heap)
        load[c] = t + int(lens[i])
        heapq.heappush(heap, (int(load[c]), c))
    return load


def cluster_balance(lens, clusters):
    """(max, mean) of the per-cluster step totals of :func:`cluster_schedule`; a
    rank's kernel time follows the maximum, its useful work the mean."""
    load = cluster_schedule(lens, clusters)
    return int(load.max()) if len(load) else 0, float(load.mean()) if len(load) else 0.0


def balanced_partition(lens, world, clusters_per_rank):
    """Partition for few sequences per resident cluster. A rank runs its shard on
    ``clusters_per_rank`` persistent clusters, so its time is the largest
    per-cluster total, not its total length divided by the cluster count. The
    sequences are therefore packed longest-first into ``world * clusters_per_rank``
    bins (least loaded bin first) and bin b goes to rank ``b % world``: every
    rank receives bins of every size class, and its own longest-first queue
    reproduces a packing of about the same height. Returns ``world`` sorted
    int64 index arrays."""
    lens, order = _longest_first(lens)
    nbins = world * int(clusters_per_rank)
    heap = [(0, b) for b in range(nbins)]
    bins = [[] for _ in range(world)]
    for i in order:
        t, b = heapq.heappop(heap)
        bins[b % world].append(int(i))
        heapq.heappush(heap, (t + int(lens[i]), b))
    return [np.array(sorted(b), dtype=np.int64) for b in bins]


def pack_bins(lens, nbins, rounds=4000):
    """Packs sequences into ``nbins`` bins so that the fullest bin is as low as a
    local search gets it: longest-first greedy packing, then repeatedly the
    fullest bin gives one sequence to, or exchanges one with, another bin,
    whichever lowers the larger of the two bins most, until no such step
    exists. This is the model of what a rank's device-side schedule does with
    its shard (greedy + repair of the fullest bin) and, over ``world *
    clusters`` bins, the packing the partition is cut from. Deterministic.
    Returns (bin index of every sequence, per-bin totals)."""
    lens, order = _longest_first(lens)
    n = len(lens)
    nbins = max(1, int(nbins))
    load = np.zeros(nbins, dtype=np.int64)
    where = np.zeros(n, dtype=np.int64)
    heap = [(0, b) for b in range(nbins)]
    for i in order:
        t, b = heapq.heappop(heap)
        where[i] = b
        load[b] = t + int(lens[i])
        heapq.heappush(heap, (int(load[b]), b))
    if n == 0 or nbins == 1:
        return where, load
    floor = max(int(lens.max()), -(-int(lens.sum()) // nbins))   # no packing is lower than this
    for _ in range(rounds):
        b = int(np.argmax(load))
        top = int(load[b])
        if top <= floor:
            break
        best = (top, -1, -1)   # (larger of the two bins afterwards, sequence leaving b, sequence entering b or -1)
        mine = np.nonzero(where == b)[0]
        other = np.nonzero(where != b)[0]
        c_min = int(np.argmin(np.where(np.arange(nbins) == b, np.iinfo(np.int64).max, load)))
        for i in mine:
            li = int(lens[i])
            moved = max(top - li, int(load[c_min]) + li)
            if moved < best[0]:
                best = (moved, int(i), -1)
            if len(other):
                lj = lens[other]
                after = np.maximum(top - li + lj, load[where[other]] + li - lj)
                k = int(np.argmin(after))
                if int(after[k]) < best[0]:
                    best = (int(after[k]), int(i), int(other[k]))
        if best[1] < 0:
            break
        i, j = best[1], best[2]
        c = c_min if j < 0 else int(where[j])
        load[b] -= lens[i]
        load[c] += lens[i]
        where[i] = c
        if j >= 0:
            load[c] -= lens[j]
            load[b] += lens[j]
            where[j] = b
    return where, load


def packed_partition(lens, world, clusters_per_rank):
    """Partition cut from one packing of all sequences into ``world *
    clusters_per_rank`` bins (:func:`pack_bins`): the bins, fullest first, are
    dealt to the ranks in serpentine order, and a rank's shard is the union of
    its bins. Every rank's own schedule can then reproduce bins no fuller than
    the global packing's fullest. Returns ``world`` sorted int64 index arrays."""
    lens = np.asarray(lens, dtype=np.int64)
    nbins = world * int(clusters_per_rank)
    where, load = pack_bins(lens, nbins)
    by_load = np.lexsort((np.arange(nbins), -load))
    rank_of_bin = np.zeros(nbins, dtype=np.int64)
    for pos, b in enumerate(by_load):
        lap, k = divmod(pos, world)
        rank_of_bin[b] = k if lap % 2 == 0 else world - 1 - k
    owner = rank_of_bin[where] if len(lens) else np.zeros(0, dtype=np.int64)
    return [np.nonzero(owner == r)[0].astype(np.int64) for r in range(world)]


def rank_makespan(lens, clusters):
    """Fullest bin of :func:`pack_bins` over one rank's sequences: the number of
    time steps its busiest resident cluster runs."""
    lens = np.asarray(lens, dtype=np.int64)
    if len(lens) == 0:
        return 0
    return int(pack_bins(lens, min(int(clusters), len(lens)))[1].max())


def partition(lens, world, clusters_per_rank=None):
    """The sequence partition every rank derives: :func:`lpt_partition`, or, when
    the number of resident clusters per rank is given, whichever of it,
    :func:`balanced_partition` and :func:`packed_partition` leaves the busiest
    cluster of any rank with the fewest time steps (ties: in that order)."""
    parts = lpt_partition(lens, world)
    if clusters_per_rank is None or world == 1:
        return parts
    lens = np.asarray(lens, dtype=np.int64)
    height = lambda ps: max(rank_makespan(lens[p], clusters_per_rank) for p in ps)
    best, best_h = parts, height(parts)
    for alt in (balanced_partition(lens, world, clusters_per_rank), packed_partition(lens, world, clusters_per_rank)):
        h = height(alt)
        if h < best_h:
            best, best_h = alt, h
    return best


def shard_sequences(seqs, rank, world, clusters_per_rank=None):
    """The ``seqs`` dictionary restricted to this rank's sequences (host side;
    call before moving data to the device) and the global indices it holds."""
    import torch
    lens = seqs["lens"].cpu().numpy() if hasattr(seqs["lens"], "cpu") else np.asarray(seqs["lens"])
    idx = partition(lens, world, clusters_per_rank)[rank]
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


def _gather_blocks(local, sizes, group=None):
    """All-gathers one block per rank (``sizes[r]`` leading entries of rank r's
    block are valid) with a single collective into one flat buffer: blocks are
    padded to the largest size. Returns the list of valid blocks in rank order
    (views of that buffer)."""
    import torch
    import torch.distributed as td
    world = td.get_world_size(group)
    width = int(max(sizes)) if len(sizes) else 0
    tail = tuple(local.shape[1:])
    if local.shape[0] == width and local.is_contiguous():
        padded = local
    else:
        padded = torch.zeros((width,) + tail, dtype=local.dtype, device=local.device)
        padded[:local.shape[0]] = local
    flat = torch.empty((world * width,) + tail, dtype=local.dtype, device=local.device)
    try:
        td.all_gather_into_tensor(flat, padded, group=group)
    except (RuntimeError, NotImplementedError):      # a backend without the flat form
        td.all_gather(list(flat.view((world, width) + tail).unbind(0)), padded, group=group)
    return [flat[r * width:r * width + int(sizes[r])] for r in range(world)]


def gather_plan(parts, device):
    """What :func:`gather_results` needs beyond the partition, prepared once: the
    padded block width and, on ``device``, the position of every sequence in the
    concatenation of the ranks' padded blocks. A caller that gathers after every
    step builds it once; the gather is then one collective and one index kernel,
    with no host-to-device traffic."""
    import torch
    sizes = [int(len(p)) for p in parts]
    width = max(sizes) if sizes else 0
    total = sum(sizes)
    perm = np.empty(total, dtype=np.int64)
    for r, p in enumerate(parts):
        perm[np.asarray(p, dtype=np.int64)] = r * width + np.arange(len(p), dtype=np.int64)
    return {"sizes": sizes, "width": width, "perm": torch.from_numpy(perm).to(device)}


def gather_results(local_result, lens=None, group=None, clusters_per_rank=None, parts=None, plan=None):
    """All-gathers the per-sequence results of every rank and returns them in
    the original sequence order. ``lens`` are the global lengths (host), from
    which every rank re-derives the partition (pass the same
    ``clusters_per_rank`` as to :func:`shard_sequences`); a caller that gathers
    repeatedly passes the partition as ``parts`` or, better, a
    :func:`gather_plan` as ``plan``."""
    import torch
    import torch.distributed as td
    world = td.get_world_size(group)
    if plan is None:
        if parts is None:
            parts = partition(lens, world, clusters_per_rank)
        plan = gather_plan(parts, local_result.device)
    width = plan["width"]
    if local_result.shape[0] == width and local_result.is_contiguous():
        padded = local_result
    else:
        padded = torch.zeros(width, dtype=local_result.dtype, device=local_result.device)
        padded[:local_result.shape[0]] = local_result
    flat = torch.empty(world * width, dtype=local_result.dtype, device=local_result.device)
    try:
        td.all_gather_into_tensor(flat, padded, group=group)
    except (RuntimeError, NotImplementedError):      # a backend without the flat form
        td.all_gather(list(flat.view(world, width).unbind(0)), padded, group=group)
    return flat.index_select(0, plan["perm"])


# ---- row blocks (CSR SpMV, SDDMM) and vector slices (reductions) ------------------------
def row_block_partition(row_ptr, world):
    """Contiguous row blocks with balanced non-zero counts for CSR operators:
    returns ``world + 1`` row boundaries (NumPy int64). ``row_ptr`` may be a
    NumPy array or a torch tensor on any device (only ``world - 1`` boundary
    searches leave the device)."""
    nrows = len(row_ptr) - 1
    if hasattr(row_ptr, "is_cuda"):      # a torch tensor
        import torch
        nnz = int(row_ptr[-1])
        targets = (torch.arange(1, world, dtype=torch.int64) * nnz) // world
        cuts = torch.searchsorted(row_ptr.contiguous(), targets.to(row_ptr.device)).cpu().numpy()
    else:
        row_ptr = np.asarray(row_ptr, dtype=np.int64)
        nnz = int(row_ptr[-1])
        targets = (np.arange(1, world, dtype=np.int64) * nnz) // world
        cuts = np.searchsorted(row_ptr, targets, side="left")
    return np.concatenate(([0], cuts, [nrows])).astype(np.int64)


def shard_csr(A, rank, world, rows_key="rows"):
    """This rank's row block of a CSR dictionary (``values``, ``cols`` and the row
    pointers under ``rows_key``, as test/test_spmv.py:20-27 and
    benchmarks/sddmm.py:43-52 build them): row pointers rebased to start at 0,
    the block's slices of ``values`` / ``cols``. Returns the local dictionary
    (extra keys ``row_begin``, ``row_end``, ``nnz_begin``, ``nnz_end``) and the
    ``world + 1`` row boundaries."""
    ptrs = A[rows_key]
    bounds = row_block_partition(ptrs, world)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    z0, z1 = int(ptrs[lo]), int(ptrs[hi])
    local = {
        rows_key: (ptrs[lo:hi + 1] - z0),
        "cols": A["cols"][z0:z1],
        "values": A["values"][z0:z1],
        "nrows": hi - lo, "nnz": z1 - z0,
        "row_begin": lo, "row_end": hi, "nnz_begin": z0, "nnz_end": z1,
    }
    if hasattr(local[rows_key], "contiguous"):
        local = {k: (v.contiguous() if hasattr(v, "contiguous") else v) for k, v in local.items()}
    return local, bounds


def _default_spmv(A_local, x, y_local):
    import parpy_b200 as parpy
    from . import kernels
    A = {k: A_local[k] for k in ("values", "rows", "cols", "nrows")}
    kernels.spmv_row(A, x, y_local, opts=parpy.par({"row": parpy.threads(max(1, A_local["nrows"]))}))


def spmv_sharded(A, x, y, group=None, local_op=None):
    """``y += A @ x`` (test/test_spmv.py:12-18) with the rows of ``A`` split into
    ``world`` contiguous blocks of about equal non-zero count. ``A``, ``x`` and
    ``y`` are the full operands, identical on every rank; each rank runs the
    single-GPU kernel on its block and one all-gather completes ``y`` in place
    on every rank. ``local_op(A_local, x, y_local)`` replaces the native kernel
    (the CPU test suite passes the oracle)."""
    import torch
    import torch.distributed as td
    rank, world = td.get_rank(group), td.get_world_size(group)
    local, bounds = shard_csr(A, rank, world)
    y_local = y[local["row_begin"]:local["row_end"]].clone()
    (local_op or _default_spmv)(local, x, y_local)
    blocks = _gather_blocks(y_local, np.diff(bounds), group)
    for r in range(world):
        y[int(bounds[r]):int(bounds[r + 1])] = blocks[r]
    return y


def _default_sddmm(A_rows, B, C_local, D_local, alpha, beta):
    import parpy_b200 as parpy
    from . import kernels
    C = {k: C_local[k] for k in ("crows", "rows", "cols", "values", "nnz")}
    n = C_local["nrows"]
    kernels.parpy_sddmm_csr_kernel(A_rows, B, C, D_local, n, alpha, beta,
                                   opts=parpy.par({"i": parpy.threads(max(1, C_local["nnz"]))}))


def sddmm_sharded(A, B, C, D, alpha, beta, group=None, local_op=None):
    """``D[i] = alpha * A[row_i, :] . B[:, col_i] + beta * C.values[i]``
    (benchmarks/sddmm.py:28-41) with the rows of the mask ``C`` (``crows``,
    ``cols``, ``values``, ``rows``, ``nnz``) split into contiguous blocks of about
    equal non-zero count. Full operands on every rank; each rank computes the
    values of its block's non-zeros (and their row indices, which the reference's
    kernel also writes into ``C['rows']``) and one all-gather each completes
    ``D`` and ``C['rows']`` in place."""
    import torch
    import torch.distributed as td
    rank, world = td.get_rank(group), td.get_world_size(group)
    local, bounds = shard_csr(C, rank, world, rows_key="crows")
    lo, hi = local["row_begin"], local["row_end"]
    local["rows"] = torch.zeros(local["nnz"], dtype=torch.int64, device=D.device)
    D_local = torch.zeros(local["nnz"], dtype=D.dtype, device=D.device)
    (local_op or _default_sddmm)(A[lo:hi].contiguous(), B, local, D_local, alpha, beta)
    crows = C["crows"]
    edges = [int(crows[int(b)]) for b in bounds]
    sizes = np.diff(edges)
    d_blocks = _gather_blocks(D_local, sizes, group)
    r_blocks = _gather_blocks(local["rows"] + lo, sizes, group)
    for r in range(world):
        D[edges[r]:edges[r + 1]] = d_blocks[r]
        C["rows"][edges[r]:edges[r + 1]] = r_blocks[r]
    return D


def slice_bounds(n, world, align=4):
    """``world + 1`` boundaries of equal contiguous slices of an ``n``-vector,
    multiples of ``align`` elements (16 bytes of float32) except the last."""
    per = -(-n // world)
    per = -(-per // align) * align
    return np.minimum(np.arange(world + 1, dtype=np.int64) * per, n)


def _default_sum_max(v_local):
    from . import kernels
    return kernels.sum_max(v_local)


def sum_max_sharded(v_local, group=None, local_op=None):
    """Sum and maximum of a float32 vector whose slices live one per rank: the
    single-GPU one-pass kernel on the local slice, one all-gather of the
    ``(sum, max)`` pairs, partial sums added in rank order (so every rank holds
    the same bits). Returns a 2-element tensor on ``v_local``'s device."""
    import torch
    import torch.distributed as td
    world = td.get_world_size(group)
    pair = (local_op or _default_sum_max)(v_local).reshape(1, 2)
    parts = torch.cat(_gather_blocks(pair, [1] * world, group), dim=0)
    total = parts[0, 0].clone()
    for r in range(1, world):
        total = total + parts[r, 0]
    return torch.stack([total, parts[:, 1].max()])
