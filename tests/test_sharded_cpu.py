"""The multi-GPU host logic on CPU ranks (gloo, world size 2 and 3): column shards, the all-gather of outputs and of
top-k records, and the global merge, against the unsharded oracle."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dense_reader import sharded
from oracle import oracle as orc


def test_column_shards():
    assert sharded.column_shards(151936, 8, 2048) == [(0, 20480), (20480, 40960), (40960, 61440), (61440, 79872),
                                                       (79872, 98304), (98304, 116736), (116736, 135168), (135168, 151936)]
    assert sharded.column_shards(14336, 8, 128) == [(1792 * r, 1792 * (r + 1)) for r in range(8)]
    s = sharded.column_shards(300, 4, 128)
    assert s == [(0, 128), (128, 256), (256, 300), (300, 300)] and sum(b - a for a, b in s) == 300


def test_topk_merge_order():
    vals = torch.tensor([[1.0, 3.0, 3.0, float("-inf"), 2.0, 3.0]])
    idx = torch.tensor([[10, 7, 5, -1, 1, 9]])
    v, i = sharded.topk_merge(vals, idx, 4)
    assert v.tolist() == [[3.0, 3.0, 3.0, 2.0]] and i.tolist() == [[5, 7, 9, 1]]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)
        k, n, m, kk = 256, 2048 * 2 + 384, 2, 8
        w = torch.randn(n, k, generator=g) * 0.02
        x = torch.randn(m, k, generator=g)
        shards = sharded.column_shards(n, world, 2048)
        a, b = shards[rank]
        wk = orc.block_float(sharded.shard_rows(w, shards, rank).T.contiguous().numpy(), "bfp8") if b > a else np.zeros((k, 0), np.float32)
        y_loc = orc.reference(x, torch.from_numpy(wk)).to(torch.bfloat16)  # this rank's columns only
        y = sharded.gather_outputs(y_loc.reshape(1, 1, m, -1), shards).reshape(m, n)
        want = orc.reference(x, torch.from_numpy(orc.block_float(w.T.contiguous().numpy(), "bfp8"))).to(torch.bfloat16)
        assert torch.equal(y, want)
        # records: one per 2048-column unit of the shard, padded to the largest shard's unit count
        units_max = max(-(-(e - s) // 2048) for s, e in shards)
        rec = torch.zeros(units_max, 2 * m * kk, dtype=torch.int32)
        for u in range(-(-(b - a) // 2048)):
            c0, c1 = u * 2048, min((u + 1) * 2048, b - a)
            for t in range(m):
                keys, idx = orc.topk_canonical(orc.bf16_bits(y_loc[t, c0:c1]), c1 - c0, kk, a + c0)
                rec[u, t * kk : (t + 1) * kk] = torch.from_numpy(keys.astype(np.int64)).to(torch.int32)
                rec[u, (m + t) * kk : (m + t + 1) * kk] = torch.from_numpy(idx.astype(np.int64)).to(torch.int32)
        allrec = sharded.gather_records(rec)
        vals, idx = orc.records_host(allrec, m, kk)
        v, i = sharded.topk_merge(vals, idx, 32)
        for t in range(m):
            # what one GPU holding the whole head would keep: the best 8 of every 2048-column unit, then the best 32
            cand = []
            for c0 in range(0, n, 2048):
                cols = sorted(range(c0, min(n, c0 + 2048)), key=lambda c: (-float(want[t, c]), c))[:kk]
                cand += cols
            order = sorted(cand, key=lambda c: (-float(want[t, c]), c))[:32]
            assert i[t].tolist() == order + [-1] * (32 - len(order)), (rank, t)  # (empty slots last)
            assert torch.equal(v[t][: len(order)], want[t, order].float())
        out[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_lm_head_on_cpu_ranks(world):
    port = _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
        assert dict(out) == {r: "ok" for r in range(world)}
