"""Sharding of the five operations over the GPUs of one node (one process per GPU).

Nothing in the reference is distributed; this layer is new. The operations partition
without any exchange on the data path:

* HPE, SAP: batch rows are independent -> contiguous row blocks; the coefficient and index
  tables are replicated.
* OPSA, OPSAW, SASAW: with a sorted scatter index every range of output rows owns a
  contiguous range of entries -> cut the output rows where the entry count balances; each
  rank gets its rows' entries, with the scatter index rebased to its first row. W (gathered
  by an unsorted index) is replicated.
* The only collective: grad_W of OPSAW/SASAW is scattered by the unsorted index, so every
  rank holds a partial grad_W of full size -> one all-reduce (NCCL on GPUs).

Helpers work on NumPy arrays or torch tensors on the host; the collectives take whatever
``torch.distributed`` backend the process group was created with.
"""
import numpy as np


def batch_range(n_rows, world, rank):
    """Rows [start, stop) of rank ``rank``: contiguous blocks, sizes differing by at most one."""
    base, extra = divmod(int(n_rows), int(world))
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def segment_cuts(indices_output, n_rows, world, known_ascending=False):
    """Row cut points rho[0..world] (rho[0] = 0, rho[world] = n_rows) and the matching entry
    cut points eps[0..world] for an ascending scatter index, such that every rank gets whole
    output rows and about the same number of entries. ``known_ascending``: the caller has
    already looked (the check reads the whole index)."""
    idx = np.asarray(indices_output)
    if not known_ascending and idx.size and np.any(idx[1:] < idx[:-1]):
        raise ValueError("segment sharding needs an ascending scatter index")
    n_entries = idx.shape[0]
    rho, eps = [0], [0]
    for r in range(1, world):
        target = (n_entries * r) // world
        # first row whose entries start at or after the target position
        row = int(idx[target]) if target < n_entries else n_rows
        # (the needle in the index's own dtype: NumPy would otherwise convert the whole index)
        start_of_row = int(np.searchsorted(idx, idx.dtype.type(row), side="left"))
        if start_of_row < target:  # the target falls inside a row: cut after it
            row += 1
            start_of_row = int(np.searchsorted(idx, idx.dtype.type(row), side="left"))
        row = max(row, rho[-1])
        rho.append(min(row, n_rows))
        eps.append(max(start_of_row, eps[-1]))
    rho.append(int(n_rows))
    eps.append(int(n_entries))
    return rho, eps


def shard_scatter(arrays, index_name, n_rows, world, rank, per_entry):
    """The part of a scatter-op input dict that rank ``rank`` works on.

    ``arrays``: name -> array; ``index_name``: the sorted scatter index; ``per_entry``: names
    of the arrays with one row per entry. Returns (local dict, (row_start, row_stop)): the
    per-entry arrays are sliced, the scatter index is rebased to the rank's first row."""
    rho, eps = segment_cuts(arrays[index_name], n_rows, world)
    lo, hi = eps[rank], eps[rank + 1]
    local = dict(arrays)
    for name in per_entry:
        if name in arrays:
            local[name] = _own(arrays[name][lo:hi])
    local[index_name] = arrays[index_name][lo:hi] - rho[rank]
    return local, (rho[rank], rho[rank + 1])


def _own(view):
    """A copy of a slice in storage of its own. A slice that starts in the middle of an array
    is rarely aligned to 16 bytes, and the streaming kernels (bulk asynchronous copies) only
    take aligned operands: a view would run on the slower general kernels."""
    return view.clone() if hasattr(view, "clone") else view.copy()


def all_reduce_sum(tensor):
    """In-place sum over all ranks (grad_W of OPSAW / SASAW)."""
    import torch.distributed as dist
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(tensor, op=dist.ReduceOp.SUM)
    return tensor


def all_gather_rows(local_rows, row_counts):
    """Concatenation over ranks of tensors that hold different numbers of leading rows
    (the optional step when one process wants the whole output)."""
    import torch
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return local_rows
    # ranks hold different numbers of rows: pad to the largest, gather, trim
    most = int(max(row_counts))
    padded = torch.zeros((most,) + tuple(local_rows.shape[1:]), dtype=local_rows.dtype,
                         device=local_rows.device)
    padded[: local_rows.shape[0]] = local_rows
    parts = [torch.empty_like(padded) for _ in row_counts]
    dist.all_gather(parts, padded)
    return torch.cat([p[: int(n)] for p, n in zip(parts, row_counts)], dim=0)
