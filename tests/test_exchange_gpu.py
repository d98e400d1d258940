"""The in-kernel exchange between the GPUs of a column-sharded weight (linear.matmul(..., exchange=)), through the
C-ABI: the peer stores, the completion flags and tkd_exchange_wait on one GPU (two ranks' calls one after the other on
one stream, the waits behind both, so that nothing ever waits for a kernel that has not been launched), and the real
thing over CUDA IPC on two GPUs where the box has them (tests/exchange_worker.py under torchrun)."""

import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from common import ttnn_like as ttnn  # noqa: E402
from dense_reader import linear, sharded  # noqa: E402

ROOT = Path(__file__).resolve().parents[1]


def fake_rank(device, rank, world, bufs, nbytes, wait=False):
    """An Exchange over plain buffers of one GPU: rank `rank`'s view of `bufs` (no IPC, no process group)."""
    ex = object.__new__(sharded.Exchange)
    ex.device, ex.group, ex.wait = device, None, wait
    ex.side = torch.cuda.Stream(device=device.torch) if wait == "deferred" else None
    ex.rank, ex.world, ex.nbytes, ex._used = rank, world, nbytes, 256
    ex.base = bufs[rank].data_ptr()
    ex.peer_base = [b.data_ptr() for r, b in enumerate(bufs) if r != rank]
    return ex


def dev_x(device, x):
    return ttnn.from_torch(x.reshape(1, 1, *x.shape).to(torch.bfloat16), dtype=ttnn.bfloat16, layout=ttnn.TILE_LAYOUT,
                           device=device)


@pytest.mark.parametrize("fmt,out32,wait", [(ttnn.bfloat8_b, False, False), (ttnn.bfloat4_b, True, False),
                                            (ttnn.bfloat8_b, False, "deferred")])
def test_outputs_reach_every_rank(device, fmt, out32, wait):
    """(wait "deferred": the kernels only store, each call is announced by tkd_exchange_publish from the rank's second
    stream; an announcement waits for the other ranks' announcements of the step before, all launched by then.)"""
    world, m, k = 3, 3, 2048
    shards = sharded.column_shards(1024 * 3 - 96, world)  # the last rank's shard is ragged
    n = shards[-1][1]
    g = torch.Generator().manual_seed(5)
    w = torch.randn(n, k, generator=g) * 0.02
    tx = dev_x(device, torch.randn(m, k, generator=g))
    full = ttnn.to_torch(linear.matmul(tx, linear.native_weight(device, w, fmt)[0], None, out32=out32))
    nbytes = 1 << 20
    bufs = [torch.zeros(nbytes + 256, dtype=torch.uint8, device=device.torch) for _ in range(world)]
    ranks = [fake_rank(device, r, world, bufs, nbytes, wait) for r in range(world)]
    outs = [[ex.tensor([1, 1, m, n], ttnn.float32 if out32 else ttnn.bfloat16) for _ in range(2)] for ex in ranks]
    tws = [linear.native_weight(device, sharded.shard_rows(w, shards, r), fmt)[0] for r in range(world)]
    status = torch.zeros(1, dtype=torch.int32, device=device.torch)
    for step in range(3):
        for r, ex in enumerate(ranks):
            linear.matmul(tx, tws[r], None, out=outs[r][step & 1], col0=shards[r][0] // 32, out32=out32, exchange=ex)
        for ex in ranks:
            ex.wait_all(status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for r in range(world):
            assert torch.equal(ttnn.to_torch(outs[r][step & 1]), full), (step, r)
            flags = bufs[r][:64].view(torch.int32).tolist()
            assert flags[:world] == [step + 1] * world and flags[8] == step + 1, flags
        for r in range(world):
            outs[r][step & 1].t.zero_()
    linear.check_status(device)


def test_records_reach_every_rank(device):
    world, k, kk, rows = 2, 1024, 8, 2
    shards = sharded.column_shards(2048 * 3 + 640, world, unit=2048)
    n = shards[-1][1]
    g = torch.Generator().manual_seed(6)
    w = (torch.randn(n, k, generator=g) * 4).round() / 64
    tx = dev_x(device, (torch.randn(rows, k, generator=g) * 2).round())
    units = -(-n // 2048)
    r_full = linear.topk_result(device, units, rows, kk)
    y_full = ttnn.allocate_tensor_on_device([1, 1, rows, n], ttnn.bfloat16, ttnn.TILE_LAYOUT, device)
    linear.matmul(tx, linear.native_weight(device, w, ttnn.bfloat8_b)[0], None, out=y_full,
                  topk={"r": r_full, "k": kk, "rows": rows, "slot0": 0, "base": 0, "n": n, "write_y": False})
    want = ttnn.to_torch(r_full)
    nbytes = 1 << 20
    bufs = [torch.zeros(nbytes + 256, dtype=torch.uint8, device=device.torch) for _ in range(world)]
    ranks = [fake_rank(device, r, world, bufs, nbytes) for r in range(world)]
    recs = []
    for ex in ranks:
        t = ex.tensor(list(r_full.shape), r_full.dtype)
        recs.append(t)
    for r, ex in enumerate(ranks):
        a, b = shards[r]
        tw = linear.native_weight(device, w[a:b], ttnn.bfloat8_b)[0]
        y = ttnn.allocate_tensor_on_device([1, 1, rows, b - a], ttnn.bfloat16, ttnn.TILE_LAYOUT, device)
        linear.matmul(tx, tw, None, out=y, exchange=ex,
                      topk={"r": recs[r], "k": kk, "rows": rows, "slot0": a // 2048, "base": a, "n": b - a, "write_y": False})
    for ex in ranks:
        ex.wait_all()
    torch.cuda.synchronize()
    for r in range(world):
        assert torch.equal(ttnn.to_torch(recs[r]), want), r
    linear.check_status(device)


def test_wait_gives_up_and_reports(device):
    """A wait for a rank that never reports runs out (about a second) and writes TKD_ERR_TIMEOUT to the status word;
    the kernel returns, the context stays usable, and the same wait succeeds once the flag is there."""
    import ctypes

    from dense_reader import _tkd

    flags = torch.zeros(_tkd.FLAG_WORDS, dtype=torch.int32, device=device.torch)
    flags[_tkd.FLAG_SEQ] = 1  # this rank has completed one exchanged call ...
    flags[0] = 1              # ... and said so; rank 1 never does
    status = torch.zeros(1, dtype=torch.int32, device=device.torch)
    sp = torch.cuda.current_stream().cuda_stream
    _tkd.check(_tkd.lib().tkd_exchange_wait(flags.data_ptr(), 2, status.data_ptr(), sp), "tkd_exchange_wait")
    torch.cuda.synchronize()
    assert int(status.item()) == _tkd.ERR_TIMEOUT
    status.zero_()
    flags[1] = 1
    _tkd.check(_tkd.lib().tkd_exchange_wait(flags.data_ptr(), 2, status.data_ptr(), sp), "tkd_exchange_wait")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert ctypes.c_int(_tkd.lib().tkd_exchange_wait(None, 2, None, sp)).value == 1  # bad argument, nothing launched


def test_peer_memory_alloc_view_free(device):
    import ctypes

    from dense_reader import _tkd

    ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
    _tkd.check(_tkd.lib().tkd_peer_alloc(4096, ctypes.byref(ptr), handle), "tkd_peer_alloc")
    assert any(handle.raw)
    v = sharded.device_view(ptr.value, [4, 8], torch.bfloat16, device.torch)
    assert not v.any()
    v += 1.5
    again = sharded.device_view(ptr.value, [32], torch.int16, device.torch)
    assert np.array_equal(again.cpu().numpy().view(np.uint16), np.full(32, 0x3FC0, np.uint16))
    del v, again
    _tkd.check(_tkd.lib().tkd_peer_free(ptr.value), "tkd_peer_free")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_exchange_between_two_gpus():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", str(ROOT / "tests" / "exchange_worker.py")]
    done = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-4000:]
    assert done.stdout.count("exchange ok") == 2, done.stdout[-2000:]
