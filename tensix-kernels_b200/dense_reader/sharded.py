"""sharded.py: the dense_reader path over the GPUs of one box, one process per GPU (torch.distributed).

The reference runs on one device; BASELINE's north star adds this: large weights (the LM head, the MLP's gate/up) are
split by output columns, each rank packs and streams only its own columns (linear.native_weight on its rows of the
[out, in] matrix, linear.matmul on the replicated activations), and the small results are joined by one all-gather:
the [M, N_local] outputs, or the top-k records followed by a merge every rank does for itself. There is no sharding of
K, so no reduction and no dependence of any value on the number of GPUs.

The collectives are torch.distributed's (NCCL on GPUs; gloo in the CPU tests of the host logic).
"""

import torch
import torch.distributed as dist


def column_shards(n, world, unit=128):
    """[(first column, end column)] per rank: contiguous ranges of whole units (128: a panel of the stream; 2048: a
    top-k record unit), as even as whole units allow, the earlier ranks one unit larger; the last range ends at n."""
    units = -(-n // unit)
    base, extra = divmod(units, world)
    out, u = [], 0
    for r in range(world):
        take = base + (1 if r < extra else 0)
        out.append((min(n, u * unit), min(n, (u + take) * unit)))
        u += take
    return out


def shard_rows(t, shards, rank):
    """A rank's rows of a [out, in] matrix (its output columns)."""
    a, b = shards[rank]
    return t[a:b]


def gather_outputs(y_local, shards, group=None):
    """Join the ranks' [..., M, N_local] outputs (a torch tensor each) into [..., M, N] on every rank: one
    all_gather_into_tensor of equal-sized (padded) pieces."""
    world = len(shards)
    widths = [b - a for a, b in shards]
    wmax = max(widths)
    lead = y_local.shape[:-1]
    piece = y_local
    if y_local.shape[-1] != wmax:
        piece = y_local.new_zeros(*lead, wmax)
        piece[..., : y_local.shape[-1]] = y_local
    flat = y_local.new_empty(world * piece.numel())
    dist.all_gather_into_tensor(flat, piece.contiguous().reshape(-1), group=group)
    buf = flat.reshape(world, *lead, wmax)
    return torch.cat([buf[r][..., : widths[r]] for r in range(world)], dim=-1)


def gather_records(rec_local, group=None):
    """Join the ranks' record tensors ([records_local, 2 * rows * k] int32, the same shape on every rank; a rank
    with fewer units leaves its last records empty) into [world * records_local, 2 * rows * k]."""
    world = dist.get_world_size(group)
    flat = rec_local.new_empty(world * rec_local.numel())
    dist.all_gather_into_tensor(flat, rec_local.contiguous().reshape(-1), group=group)
    return flat.reshape(world * rec_local.shape[0], rec_local.shape[1])


def topk_merge(vals, idx, top):
    """The best `top` of the candidates of every row, value descending and index ascending among equal values
    (vals [rows, n] float32 with -inf for empty slots, idx [rows, n] int64 with -1): (values [rows, top], indices
    [rows, top]). The order is total, so every rank gets the same answer from the same gathered records."""
    if vals.shape[1] < top:  # fewer candidates than asked for: the rest are empty slots
        pad = top - vals.shape[1]
        vals = torch.cat([vals, vals.new_full((vals.shape[0], pad), float("-inf"))], dim=1)
        idx = torch.cat([idx, idx.new_full((idx.shape[0], pad), -1)], dim=1)
    big = torch.iinfo(torch.int64).max
    key_idx = torch.where(idx < 0, torch.full_like(idx, big), idx)
    # stable two-key sort: by index ascending first, then by value descending
    o1 = torch.argsort(key_idx, dim=1, stable=True)
    v1, i1 = torch.gather(vals, 1, o1), torch.gather(idx, 1, o1)
    o2 = torch.argsort(v1, dim=1, descending=True, stable=True)
    return torch.gather(v1, 1, o2)[:, :top], torch.gather(i1, 1, o2)[:, :top]
