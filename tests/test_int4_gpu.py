# SPDX-License-Identifier: Apache-2.0
# Copyright 2026 Xylolabs
# Ported from XylolabsInc/tensix-kernels, int4/tests/test_int4.py (Apache-2.0): the first four tests, their shapes, seeds and bars are that
# file's; the imports and the device API under them are this package's. The tests after them are this package's own.
"""The reference's int4 checks (int4/tests/test_int4.py), same shapes, seeds and bars, against this package's API on a
B200: random codes in -7..7 and bf16 group scales (G = 32), x with a few outlier channels; y against x rounded to bf16
times q * s in float32 (relative Frobenius error below 1 %, PCC above 0.9999; the dequantised bfloat8_b weight below 2 %);
one loader against two bit for bit. Then parity with the CPU oracle: the packed weight's held values exactly q * s, and y
for one to eight rows and ragged shapes within 1e-2 (compared in bf16)."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from common import device as cdev  # noqa: E402
from common import ttnn_like as ttnn  # noqa: E402
from common.testing import check, same  # noqa: E402
from dense_reader import linear  # noqa: E402
from int4 import w4a16  # noqa: E402
from oracle import oracle as orc  # noqa: E402


def make_case(n, k, seed):
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(-7, 8, (n, k), generator=g).to(torch.int8)
    scales = (torch.rand(n, k // 32, generator=g) * 0.01 + 0.001).to(torch.bfloat16)
    return codes, scales


def make_x(device, k, seed, memory_config):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(1, k, generator=g)
    x[:, torch.randperm(k, generator=g)[:8]] *= 20  # a few outlier channels
    x = x.to(torch.bfloat16)
    tx = ttnn.from_torch(x.reshape(1, 1, 1, k), dtype=ttnn.bfloat16, layout=ttnn.TILE_LAYOUT, device=device,
                         memory_config=memory_config)
    return x, tx


def host(y, n):
    return ttnn.to_torch(y).float().reshape(-1, y.shape[-1])[:1, :n]


def test_matmul(device):
    matmul_case(device, "hifi4")


def test_hifi2(device):
    matmul_case(device, "hifi2")


def matmul_case(device, fid):
    for k, n in ((1024, 1152), (3072, 1024)):
        codes, scales = make_case(n, k, k + n)
        wq = w4a16.int4_weight(device, codes)
        ts = w4a16.group_scales(device, scales)
        for mc, where in ((ttnn.L1_MEMORY_CONFIG, "L1"), (ttnn.DRAM_MEMORY_CONFIG, "DRAM")):
            x, tx = make_x(device, k, n, mc)
            ref = w4a16.reference(x, codes, scales)
            y = host(w4a16.w4a16_linear(tx, wq, ts, fidelity=fid), n)
            check(f"int4 {fid} K {k} N {n} x in {where}", y, ref)
            same(f"int4 {fid} K {k} N {n} x in {where}: one loader against two",
                 host(w4a16.w4a16_linear(tx, wq, ts, split=False, fidelity=fid), n), y)
            ttnn.deallocate(tx)
        ttnn.deallocate(wq["t"])
        ttnn.deallocate(ts)
    linear.check_status(device)


def test_fewer_banks(device):
    k, n = 1024, 1024
    banks = cdev.dram_banks(device)
    fewer = max(1, banks // 2)
    codes, scales = make_case(n, k, 7)
    wq = w4a16.int4_weight(device, codes, max_banks=fewer)
    assert wq["banks"] == fewer and wq["t"].memory_config().shard_spec.num_cores() == fewer
    ts = w4a16.group_scales(device, scales)
    x, tx = make_x(device, k, 8, ttnn.L1_MEMORY_CONFIG)
    check(f"int4 hifi4 weight over {fewer} of {banks} banks", host(w4a16.w4a16_linear(tx, wq, ts, fidelity="hifi4"), n),
          w4a16.reference(x, codes, scales))


def test_dequantize(device):
    k, n = 2048, 1152
    codes, scales = make_case(n, k, 9)
    wq = w4a16.int4_weight(device, codes)
    ts = w4a16.group_scales(device, scales)
    wd = w4a16.dequantize(wq, ts)
    got = ttnn.to_torch(wd).float().reshape(k, -1)[:, :n]
    check("dequantized bfloat8_b weight against q * s", got, w4a16.dequantized(codes, scales).T, rel=0.02)
    again = w4a16.dequantize(wq, ts, out=wd)
    same("dequantize into a given output: the same tensor and values",
         ttnn.to_torch(again).float().reshape(k, -1)[:, :n], got)
    linear.check_status(device)


# ---- parity with the CPU oracle -------------------------------------------------------------------------------------

def close_bf16(got, want, tol=1e-2):
    g, w = got.to(torch.bfloat16).float(), torch.as_tensor(want).to(torch.bfloat16).float()
    scale = w.abs().amax(dim=-1, keepdim=True).clamp(min=1e-30)
    err = ((g - w).abs() / scale).max().item()
    assert err < tol, err


@pytest.mark.parametrize("k,n", [(96, 64), (1024 + 32, 1024 + 48), (4096, 2048 + 16)])
def test_held_values_and_rows_against_oracle(device, k, n):
    """The packed stream holds q * s exactly (K with a half-filled last super-atom, N with a ragged last panel), and
    one to eight rows (the stream kernel's range for this format) agree with the oracle."""
    codes, scales = make_case(n, k, 3 * k + n)
    wq = w4a16.int4_weight(device, codes)
    ts = w4a16.group_scales(device, scales)
    w = w4a16.packed(wq, ts)
    held = ttnn.to_torch(w)[0, 0, :, :n]
    assert torch.equal(held, torch.from_numpy(orc.int4_dequantized(codes.numpy(), scales)).T), "held values differ from q * s"
    for m in (1, 3, 8):
        g = torch.Generator().manual_seed(m)
        x = torch.randn(m, k, generator=g)
        tx = ttnn.from_torch(x.reshape(1, 1, m, k).to(torch.bfloat16), dtype=ttnn.bfloat16, layout=ttnn.TILE_LAYOUT,
                             device=device)
        y = ttnn.to_torch(linear.matmul(tx, w, None)).float().reshape(-1, n)[:m]
        close_bf16(y, orc.int4_reference(x, codes.numpy(), scales))
    linear.check_status(device)


def test_more_than_eight_rows_is_refused(device):
    from dense_reader import _tkd

    codes, scales = make_case(256, 128, 1)
    wq = w4a16.int4_weight(device, codes)
    w = w4a16.packed(wq, w4a16.group_scales(device, scales))
    tx = ttnn.from_torch(torch.zeros(1, 1, 9, 128, dtype=torch.bfloat16), dtype=ttnn.bfloat16, layout=ttnn.TILE_LAYOUT,
                         device=device)
    with pytest.raises(_tkd.TkdError):
        linear.matmul(tx, w, None)
