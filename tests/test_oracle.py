"""The CPU oracle against the golden vectors made from the reference's own host code (tests/golden/gen_golden.py)."""

import hashlib
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle as orc

G = Path(__file__).resolve().parent / "golden"
sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()  # noqa: E731


@pytest.fixture(scope="module")
def q():
    return np.load(G / "quantiser_bfp4.npz")


@pytest.fixture(scope="module")
def h():
    return np.load(G / "host_helpers.npz")


def test_bfp4_tiles_match_reference(q):
    g = torch.Generator().manual_seed(0)
    w = torch.randn(256, 512, generator=g) * 0.02
    w[3, 5], w[7, 9] = 0.0, -1e-30
    assert sha(w.numpy()) == str(q["w1_sha"])
    for quant in (orc.quantise_c, orc.quantise_np):
        e, c = quant(w.numpy(), "bfp4")
        assert np.array_equal(orc.tiles(e, c, "bfp4"), q["t1"])
        v = orc.dequantise(e, c, "bfp4")
        assert sha(v) == str(q["v1_sha"])
        assert np.array_equal(v[0, :64], q["v1_row0"])
        assert v[3, 5] == 0.0 and v[7, 9] == 0.0
        # idempotent on its own grid
        e2, c2 = quant(v, "bfp4")
        assert np.array_equal(orc.dequantise(e2, c2, "bfp4"), v)


def test_bfp4_formats_weight_sha(q):
    g = torch.Generator().manual_seed(2)
    w = (torch.randn(2048, 1024, generator=g) * 0.02).T.contiguous().numpy()
    e, c = orc.quantise_c(w, "bfp4")
    t = orc.tiles(e, c, "bfp4")
    assert sha(t) == str(q["t2_sha"])
    assert np.array_equal(t[:2, :2], q["t2_head"])
    e2, c2 = orc.quantise_np(w, "bfp4")
    assert np.array_equal(e, e2) and np.array_equal(c, c2)


def test_rounding_cases(q):
    e, c = orc.quantise_c(q["w3"], "bfp4")
    assert e[0, 0] == 127
    v = orc.dequantise(e, c, "bfp4")
    assert np.array_equal(v, q["v3"])
    want = [1.0, 0.5, 0.25, 0, 0, 0.25, 0.25, 0.5, 0.5, 0.75, 1.0, 1.0, -1.0, 0, 1.75, -1.0]
    assert v[0, :16].tolist() == want


def test_wide_spread_and_specials(q):
    for quant in (orc.quantise_c, orc.quantise_np):
        e, c = quant(q["w4"], "bfp4")
        assert np.array_equal(orc.tiles(e, c, "bfp4"), q["t4"])
        assert np.array_equal(orc.dequantise(e, c, "bfp4"), q["v4"])


def test_bfp8_c_against_numpy_and_properties():
    """bfloat8_b has no vector in the reference (parity unpinned): the two restatements agree, values are within half
    a step of the input, and the grid is a fixed point."""
    g = torch.Generator().manual_seed(3)
    w = (torch.randn(96, 128, generator=g) * torch.exp2(torch.randint(-12, 3, (96, 128), generator=g).float())).numpy()
    w[0, :16] = 0
    w[5, 7] = 1e-41
    e, c = orc.quantise_c(w, "bfp8")
    e2, c2 = orc.quantise_np(w, "bfp8")
    assert np.array_equal(e, e2) and np.array_equal(c, c2)
    v = orc.dequantise(e, c, "bfp8")
    step = np.ldexp(np.float32(1), np.repeat(e.astype(np.int32), 16, axis=1) - 133)
    clamp = np.abs(w) > 127 * step  # the largest magnitude does not bump the exponent
    assert np.all(np.abs(v - w)[~clamp] <= step[~clamp])  # truncating shift, then nearest: below one step
    e3, c3 = orc.quantise_c(v, "bfp8")
    assert np.array_equal(orc.dequantise(e3, c3, "bfp8"), v)
    t = orc.tiles(e, c, "bfp8")
    assert t.shape == (3, 4, 1088)
    assert np.array_equal(t[0, 0, :16], e[:16, 0]) and np.array_equal(t[0, 0, 64:80], c[0, :16])


def test_host_helpers(h):
    gate = torch.arange(128.0).reshape(64, 2)
    assert np.array_equal(orc.interleave_glu(gate, -gate).numpy(), h["il"])
    assert np.array_equal(orc.bf16_ceil(torch.from_numpy(h["ceil_in"])).numpy(), h["ceil_out"])
    for s, want in zip(h["ceil_in"], h["ceil_out"]):
        assert orc.lib().orc_bf16_ceil(float(s)) == want or s == 0.0
    assert np.array_equal(orc.keys_of(h["bf16_bits"].astype(np.uint16)), h["keys"].astype(np.uint32))
    for b, k in zip(h["bf16_bits"], h["keys"]):
        assert orc.lib().orc_key(int(b)) == int(k)
    vals, idx = orc.records_host(torch.from_numpy(h["rec"]), 2, 4)
    assert np.array_equal(vals.numpy().view(np.uint32), h["rec_vals"].view(np.uint32))
    assert np.array_equal(idx.numpy(), h["rec_idx"])
    x, wk, sc = torch.from_numpy(h["x"]), h["wk"], h["sc"]
    assert np.array_equal(orc.reference(x, wk).numpy(), h["ref"])
    assert np.array_equal(orc.reference(x, wk, sc).numpy(), h["ref_sc"])
    y64 = orc.matmul_f64(x, wk)
    assert np.allclose(y64, h["ref"], rtol=1e-5, atol=1e-6)


def test_epilogues_against_torch():
    g = torch.Generator().manual_seed(4)
    acc = torch.randn(3, 128, generator=g, dtype=torch.float64) * 3
    up = torch.randn(3, 128, generator=g, dtype=torch.float64)
    F = torch.nn.functional
    for act, fn in ((0, F.silu), (1, lambda t: F.gelu(t, approximate="tanh"))):
        got = orc.epilogue(acc.numpy(), 2, acc2=up.numpy(), act=act)
        assert np.allclose(got, (fn(acc) * up).numpy(), rtol=1e-12, atol=1e-12)
        il = torch.stack([acc.reshape(3, 4, 32), up.reshape(3, 4, 32)], dim=2).reshape(3, 256)
        got = orc.epilogue(il.numpy(), 1, act=act)
        assert np.allclose(got, (fn(acc) * up).numpy(), rtol=1e-12, atol=1e-12)
    res = torch.randn(3, 128, generator=g).to(torch.bfloat16)
    assert np.allclose(orc.epilogue(acc.numpy(), 3, res=res), (acc + res.double()).numpy())
    sc = torch.rand(128, generator=g) + 0.5
    assert np.allclose(orc.epilogue(acc.numpy(), 0, scale=sc.numpy()), (acc * sc.double()).numpy())


def test_topk_orders():
    """Canonical order (key descending, index ascending) against torch; the reference writer's scan keeps the same
    values but may keep other indices among ties (k 2, values 5, 5, 7 keep ids 1 and 2)."""
    g = torch.Generator().manual_seed(6)
    y = (torch.randn(2048, generator=g) * 4).round().to(torch.bfloat16)  # many ties
    bits = orc.bf16_bits(y)
    keys, idx = orc.topk_canonical(bits, 2011, 8, 1000)
    vals = np.array([orc.lib().orc_key_value(int(k)) for k in keys], np.float32)
    want = torch.topk(y[:2011].float(), 8).values.numpy()
    assert np.array_equal(vals, want)
    for a in range(7):
        assert keys[a] > keys[a + 1] or (keys[a] == keys[a + 1] and idx[a] < idx[a + 1])
    # every kept index is the lowest available among its ties
    yv = y[:2011].float().numpy()
    for v in np.unique(vals):
        kept = sorted(int(i) - 1000 for i, vv in zip(idx, vals) if vv == v)
        assert kept == list(np.flatnonzero(yv == v)[: len(kept)])
    rk, ri = orc.topk_scan_ref(bits, 0, 2048, 2011, 8, 1000)
    assert sorted(rk.tolist()) == sorted(keys.tolist())
    k2, i2 = orc.topk_scan_ref(orc.bf16_bits(torch.tensor([5.0, 5.0, 7.0])), 0, 3, 3, 2, 0)
    assert sorted(i2.tolist()) == [1, 2]
    k3, i3 = orc.topk_canonical(orc.bf16_bits(torch.tensor([5.0, 5.0, 7.0])), 3, 2, 0)
    assert i3.tolist() == [2, 0]
