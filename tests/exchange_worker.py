"""One rank of the two-GPU exchange test (run under torchrun by tests/test_exchange_gpu.py): a column-sharded weight,
every call's output and top-k records delivered into both ranks' buffers by the stream kernel itself, compared bit for
bit with the unsharded call on this rank's own GPU."""

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path[:0] = [str(ROOT), str(ROOT / "tensix-kernels_b200")]

from common import ttnn_like as ttnn  # noqa: E402
from dense_reader import linear, sharded  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    device = ttnn.open_device(device_id=local)
    m, k, kk = 2, 4096, 8
    shards = sharded.column_shards(2048 * 5 + 512, world, unit=2048)
    n = shards[-1][1]
    g = torch.Generator().manual_seed(9)  # (the same matrix on every rank)
    w = torch.randn(n, k, generator=g) * 0.02
    xs = [torch.randn(m, k, generator=g) for _ in range(4)]
    tw_full = linear.native_weight(device, w, ttnn.bfloat8_b)[0]
    a, b = shards[rank]
    tw = linear.native_weight(device, w[a:b], ttnn.bfloat8_b)[0]
    units = -(-n // 2048)
    ex = sharded.Exchange(device, 4 << 20)
    outs = [ex.tensor([1, 1, m, n], ttnn.bfloat16) for _ in range(2)]
    r0 = linear.topk_result(device, units, m, kk)
    recs = [ex.tensor(list(r0.shape), r0.dtype) for _ in range(2)]
    for step, x in enumerate(xs):
        tx = ttnn.from_torch(x.reshape(1, 1, m, k).to(torch.bfloat16), dtype=ttnn.bfloat16, layout=ttnn.TILE_LAYOUT, device=device)
        want = ttnn.to_torch(linear.matmul(tx, tw_full, None))
        y_full = ttnn.allocate_tensor_on_device([1, 1, m, n], ttnn.bfloat16, ttnn.TILE_LAYOUT, device)
        linear.matmul(tx, tw_full, None, out=y_full,
                      topk={"r": r0, "k": kk, "rows": m, "slot0": 0, "base": 0, "n": n, "write_y": False})
        # the sharded calls: when each returns control to the stream, both ranks' parts are in this rank's buffer
        got = linear.matmul(tx, tw, None, out=outs[step & 1], col0=a // 32, exchange=ex)
        y_loc = ttnn.allocate_tensor_on_device([1, 1, m, b - a], ttnn.bfloat16, ttnn.TILE_LAYOUT, device)
        linear.matmul(tx, tw, None, out=y_loc, exchange=ex,
                      topk={"r": recs[step & 1], "k": kk, "rows": m, "slot0": a // 2048, "base": a, "n": b - a, "write_y": False})
        torch.cuda.synchronize()
        linear.check_status(device)
        assert torch.equal(ttnn.to_torch(got), want), ("outputs", rank, step)
        assert torch.equal(ttnn.to_torch(recs[step & 1]), ttnn.to_torch(r0)), ("records", rank, step)
    ex.close()
    print("exchange ok", rank, flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
