"""sharded.py: the dense_reader path over the GPUs of one box, one process per GPU (torch.distributed).

The reference runs on one device; on a box of GPUs large weights (the LM head, the MLP's gate/up) are
split by output columns, each rank packs and streams only its own columns (linear.native_weight on its rows of the
[out, in] matrix, linear.matmul on the replicated activations), and the small results are joined by one all-gather:
the [M, N_local] outputs, or the top-k records followed by a merge every rank does for itself. There is no sharding of
K, so no reduction and no dependence of any value on the number of GPUs.

Two ways to join: torch.distributed's collectives (gather_outputs, gather_records: NCCL on GPUs, gloo in the CPU
tests of the host logic), or Exchange: the stream kernel itself stores every output element and record into the other
ranks' buffers over NVLink as it finishes them, and the call completes when every rank's part has arrived, so there is
no collective launch at all.
"""

import ctypes

import torch
import torch.distributed as dist

from dense_reader import _tkd

_TYPESTR = {torch.bfloat16: None, torch.float32: "<f4", torch.int32: "<i4", torch.uint8: "|u1", torch.int16: "<i2"}


class _Raw:
    """Device memory at an address, for torch.as_tensor (the CUDA array interface)."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2}


def device_view(ptr, shape, dtype, device):
    """A torch tensor over `ptr` (no copy; the memory must outlive it)."""
    n = 1
    for d in shape:
        n *= d
    if dtype == torch.bfloat16:  # (the array interface has no bfloat16: go through its 16-bit words)
        return torch.as_tensor(_Raw(ptr, (n,), "<i2"), device=device).view(torch.bfloat16).reshape(list(shape))
    return torch.as_tensor(_Raw(ptr, (n,), _TYPESTR[dtype]), device=device).reshape(list(shape))


class Exchange:
    """One buffer per rank that every rank of the group can write: `nbytes` of device memory from tkd_peer_alloc,
    mapped into every other rank's process through its inter-process handle (CUDA IPC; the handles travel by
    all_gather_object), plus the flag words the kernels signal completion with.

    Tensors carved from it with tensor() sit at the same offset on every rank (every rank makes the same calls in the
    same order). linear.matmul(..., exchange=ex) then writes whatever of its output and records lies inside the buffer
    to all ranks: with out a [1, 1, M, N_total] tensor of the buffer and col0 the rank's first column tile, every rank
    ends up with the whole row. With wait (the default) the call's kernel ends only when all ranks' parts have
    arrived; a call must not write a tensor again before every rank has read what the last call but one left there
    (alternate between two tensors). wait="lagged": each kernel ends when all ranks' parts of the exchanged call BEFORE
    it have arrived, so that an exchange's latency passes during the next call's run (wait_all() flushes the last one;
    a tensor may be written again four calls later). wait=False: nothing waits but wait_all(). wait="deferred": the
    kernel only stores; a one-thread kernel on a second stream, ordered behind the call by an event, announces it (its
    system-wide fence, the flags' flight and a bounded check that every rank announced the call before overlap the
    next call instead of ending this one); wait_all() joins that stream and waits for the last call."""

    def __init__(self, device, nbytes, group=None, wait=True):
        self.device, self.group, self.wait = device, group, wait
        self.side = torch.cuda.Stream(device=device.torch) if wait == "deferred" else None
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        assert self.world <= _tkd.MAX_RANKS, "dense_reader: an exchange spans the GPUs of one box (8)"
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self._used = 256  # the flag words come first
        ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        with torch.cuda.device(device.torch):
            _tkd.check(_tkd.lib().tkd_peer_alloc(self.nbytes + 256, ctypes.byref(ptr), handle), "tkd_peer_alloc")
        self.base = ptr.value
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.peer_base = []  # the other ranks' buffers, in rank order
        for r, h in enumerate(handles):
            if r == self.rank:
                continue
            q = ctypes.c_void_p()
            with torch.cuda.device(device.torch):
                _tkd.check(_tkd.lib().tkd_peer_open(ctypes.create_string_buffer(h, 64), ctypes.byref(q)), "tkd_peer_open")
            self.peer_base.append(q.value)
        dist.barrier(group=group)

    def tensor(self, shape, dtype):
        """A zeroed ttnn-like tensor inside the buffer."""
        from common import ttnn_like as ttnn

        tdt = ttnn._TORCH[dtype]
        n = 1
        for d in shape:
            n *= d
        size = (n * torch.empty(0, dtype=tdt).element_size() + 255) // 256 * 256
        assert self._used + size <= self.nbytes + 256, "dense_reader: the exchange buffer is full"
        t = device_view(self.base + self._used, list(shape), tdt, self.device.torch)
        self._used += size
        return ttnn.Tensor(t, dtype, ttnn.TILE_LAYOUT, self.device, None)

    def _peers_of(self, ptr):
        if ptr is None or not self.base <= ptr < self.base + self.nbytes + 256:
            return None
        return [b + (ptr - self.base) for b in self.peer_base]

    def fill(self, a, out_ptr, rec_ptr):
        """Put this exchange into a launch descriptor: the peers' addresses of the output and of the records (where
        those lie inside the buffer) and the flag words."""
        mode = {"lagged": 2, "deferred": 3}.get(self.wait, int(bool(self.wait)))
        a.nranks, a.rank, a.flags, a.exchange_wait = self.world, self.rank, self.base, mode
        outs, recs = self._peers_of(out_ptr), self._peers_of(rec_ptr)
        for q, b in enumerate(self.peer_base):
            a.peer_flags[q] = b
            a.peer_out[q] = outs[q] if outs else None
            a.peer_records[q] = recs[q] if recs else None

    def after_launch(self, status=None):
        """wait="deferred": announce the call just launched on the current stream, from the side stream."""
        if self.side is None:
            return
        done = torch.cuda.Event()
        done.record(torch.cuda.current_stream())
        self.side.wait_event(done)
        peers = (ctypes.c_void_p * 7)(*self.peer_base)
        _tkd.check(_tkd.lib().tkd_exchange_publish(self.base, peers, self.world, self.rank, 1,
                                                   status.data_ptr() if status is not None else None, self.side.cuda_stream),
                   "tkd_exchange_publish")

    def wait_all(self, status=None, stream=None):
        """Order a wait for every rank's last exchanged call behind the current stream's work (for wait=False or
        "deferred", or after a kernel's own wait gave up)."""
        if self.side is not None:
            (torch.cuda.current_stream() if stream is None else stream).wait_stream(self.side)
        sp = torch.cuda.current_stream().cuda_stream if stream is None else stream.cuda_stream
        _tkd.check(_tkd.lib().tkd_exchange_wait(self.base, self.world, status.data_ptr() if status is not None else None, sp),
                   "tkd_exchange_wait")

    def close(self):
        """Unmap the peers' buffers and free this rank's (collective: nobody may still be writing)."""
        torch.cuda.synchronize(self.device.torch)
        dist.barrier(group=self.group)
        for q in self.peer_base:
            _tkd.lib().tkd_peer_close(q)
        self.peer_base = []
        dist.barrier(group=self.group)
        if self.base:
            _tkd.lib().tkd_peer_free(self.base)
            self.base = None


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
