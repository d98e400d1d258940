"""Parity of the CUDA path with the CPU oracle, through the package's API (which calls libtkd's C-ABI): bit-exact for
the quantiser, the packed weights' held values and the top-k indices; 1e-2 relative (compared in bf16) for the sums."""

from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from common import ttnn_like as ttnn  # noqa: E402
from dense_reader import linear  # noqa: E402
from oracle import oracle as orc  # noqa: E402

DT = {"bfp8": ttnn.bfloat8_b, "bfp4": ttnn.bfloat4_b, "bf16": ttnn.bfloat16}
GOLDEN = Path(__file__).resolve().parent / "golden"


def dev_x(device, x):
    return ttnn.from_torch(x.reshape(1, 1, *x.shape).to(torch.bfloat16), dtype=ttnn.bfloat16, layout=ttnn.TILE_LAYOUT,
                           device=device)


def host(y):
    return ttnn.to_torch(y).float().reshape(-1, y.shape[-1])


def close_bf16(got, want, tol=1e-2):
    """|got - want| within tol relative to the row's scale, both seen in bf16."""
    g, w = got.to(torch.bfloat16).float(), torch.as_tensor(want).to(torch.bfloat16).float()
    scale = w.abs().amax(dim=-1, keepdim=True).clamp(min=1e-30)
    err = ((g - w).abs() / scale).max().item()
    assert err < tol, err


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4", "bf16"])
@pytest.mark.parametrize("k,n", [(64, 32), (96, 48), (1024, 2048), (4096, 1024 + 16)])
def test_held_values_bit_exact(device, fmt, k, n):
    g = torch.Generator().manual_seed(k * 7 + n)
    w = torch.randn(n, k, generator=g) * 0.02 * torch.exp2(torch.randint(-6, 7, (n, 1), generator=g).float())
    w[0] = 0
    w[3, 5], w[7 % n, 9] = 0.0, -1e-30
    n_ok = n if n % 32 == 0 else n  # (native_weight takes any N; the stream pads to 16)
    tw, _ = linear.native_weight(device, w, DT[fmt])
    got = ttnn.to_torch(tw)[0, 0, :, :n_ok].numpy()
    want = orc.block_float(w.T.contiguous().numpy(), fmt)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # padded columns hold zeros
    assert not ttnn.to_torch(tw)[0, 0, :, n_ok:].any()


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_col_scale_and_block_float(device, fmt):
    g = torch.Generator().manual_seed(11)
    w = torch.randn(256, 128, generator=g) * 0.02
    w[:100] *= 40
    tw, ts = linear.native_weight(device, w, DT[fmt], col_scale=True)
    want_w, want_c = orc.native_values(w, fmt, col_scale=True)
    assert np.array_equal(ttnn.to_torch(tw)[0, 0, :, :256].numpy().view(np.uint32), want_w.view(np.uint32))
    assert np.array_equal(ttnn.to_torch(ts).float().reshape(-1).numpy(), want_c)
    t = torch.randn(2, 64, 96, generator=g)
    got = linear.block_float(t, DT[fmt])
    for i in range(2):
        assert np.array_equal(got[i].numpy().view(np.uint32), orc.block_float(t[i].numpy(), fmt).view(np.uint32))


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4"])
def test_wide_weight_runs(device, fmt):
    """A weight whose exponents inside a group of 16 columns spread further than the block-float stream encodes (the
    reference takes any float matrix, linear.py:144-156): here a dead input channel of 1e-17-size noise beside
    0.02-size rows, and the quantiser golden file's wide-spread matrix (zeros, denormals, huge values). The weight holds
    the oracle's values bit for bit and the matmul matches the oracle, also when only the tiny rows see activations."""
    g = torch.Generator().manual_seed(66)
    n, k = 256, 512
    w = torch.randn(n, k, generator=g) * 0.02
    w[:, 7] = torch.randn(n, generator=g) * 1e-17
    tw, _ = linear.native_weight(device, w, DT[fmt])
    assert tw.wide and tw.dtype == DT[fmt]
    wk = orc.native_values(w, fmt)[0]
    assert np.array_equal(ttnn.to_torch(tw)[0, 0, :, :n].numpy().view(np.uint32), wk.view(np.uint32))
    x = torch.randn(3, k, generator=g)
    x[1] = 0
    x[1, 7] = 3.0   # only the dead channel: the sums are of 1e-17 size
    x[2, 7] = 2.0 ** 60
    y = host(linear.matmul(dev_x(device, x), tw, None))
    want = orc.matmul_f64(x, wk)
    close_bf16(y, want)
    assert y[1].abs().max() > 0
    # a block list with a weight that is not wide: one launch, one stream format
    w2 = torch.randn(128, k, generator=g) * 0.02
    t2, _ = linear.native_weight(device, w2, DT[fmt])
    assert not t2.wide
    both = host(linear.matmul(dev_x(device, x), [(tw, 0), (t2, n // 32)], None))
    assert torch.equal(both[:, :n], y)
    close_bf16(both[:, n:], orc.matmul_f64(x, orc.native_values(w2, fmt)[0]))
    if fmt == "bfp4":
        gold = np.load(GOLDEN / "quantiser_bfp4.npz")
        w4 = torch.from_numpy(gold["w4"].astype(np.float32))  # [K, N]
        t4 = ttnn.from_torch(w4, dtype=ttnn.bfloat4_b, device=device)
        held = ttnn.to_torch(t4)[0, 0, :, : w4.shape[1]].numpy()
        assert np.array_equal(held.view(np.uint32), orc.block_float(w4.numpy(), "bfp4").view(np.uint32))
    linear.check_status(device)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4", "bf16"])
@pytest.mark.parametrize("m", [1, 4, 8, 13, 32])
def test_matmul_against_oracle(device, fmt, m):
    k, n = 2048 + 32, 1024 + 32  # K not a multiple of the slice, N not of the panel
    g = torch.Generator().manual_seed(100 + m)
    w = torch.randn(n, k, generator=g) * 0.02
    x = torch.randn(m, k, generator=g)
    tw, _ = linear.native_weight(device, w, DT[fmt])
    wk, _ = orc.native_values(w, fmt)
    y = host(linear.matmul(dev_x(device, x), tw, None))
    assert y.shape == (m, n)
    want = orc.matmul_f64(x, wk)
    close_bf16(y, want)
    linear.check_status(device)


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4", "bf16"])
@pytest.mark.parametrize("m,n", [(9, 1024 + 16), (17, 1024 + 128), (32, 2048 + 80)])
def test_many_rows_epilogues_against_oracle(device, fmt, m, n):
    """The kernel for 9 to 32 rows: every epilogue, N with a ragged last panel, K with a short last slice."""
    k = 1024 + 96
    g = torch.Generator().manual_seed(7 * m + n)
    w, w2 = torch.randn(n, k, generator=g) * 0.02, torch.randn(n, k, generator=g) * 0.02
    x = torch.randn(m, k, generator=g)
    tx = dev_x(device, x)
    tw, _ = linear.native_weight(device, w, DT[fmt])
    tw2, _ = linear.native_weight(device, w2, DT[fmt])
    wk, _ = orc.native_values(w, fmt)
    wk2, _ = orc.native_values(w2, fmt)
    plain = orc.matmul_f64(x, wk)
    close_bf16(host(linear.matmul(tx, tw, None)), plain)
    # fp32 output with an fp32 residual
    res = torch.randn(m, n, generator=g)
    tr = ttnn.from_torch(res.reshape(1, 1, m, n), dtype=ttnn.float32, layout=ttnn.TILE_LAYOUT, device=device)
    y32 = host(linear.matmul(tx, tw, None, residual=tr, out32=True)).double().numpy()
    np.testing.assert_allclose(y32, plain + res.double().numpy(), rtol=2e-3, atol=2e-3)
    # bf16 residual
    resb = res.to(torch.bfloat16)
    trb = ttnn.from_torch(resb.reshape(1, 1, m, n), dtype=ttnn.bfloat16, layout=ttnn.TILE_LAYOUT, device=device)
    close_bf16(host(linear.matmul(tx, tw, None, residual=trb)), plain + resb.double().numpy())
    # column scales
    sc = (torch.rand(n, generator=g) + 0.5).to(torch.bfloat16)
    close_bf16(host(linear.matmul(tx, tw, linear.scale_tensor(device, sc.float()))), plain * sc.double().numpy()[None, :])
    # SwiGLU from two weights
    gate, up = torch.from_numpy(plain), torch.from_numpy(orc.matmul_f64(x, wk2))
    close_bf16(host(linear.matmul(tx, tw, None, w_up=tw2, glu=True)), (torch.nn.functional.silu(gate) * up).numpy())
    linear.check_status(device)


def test_config_shapes_full_size(device):
    """The benchmark configurations at their own sizes against the oracle over every column: the README example
    (one token through a [4096, 2048] bfloat8_b weight), the MLP gate/up pair (two [14336, 4096] bfloat4_b weights,
    float32 column scales, SwiGLU; as two weights and as one interleaved weight) and the down projection ([4096, 14336]
    bfloat8_b, float32 residual and output) at 1, 8 and 32 rows."""
    g = torch.Generator().manual_seed(0)
    w = torch.randn(4096, 2048, generator=g) * 0.02
    x = torch.randn(1, 2048, generator=g)
    tw, _ = linear.native_weight(device, w, ttnn.bfloat8_b)
    close_bf16(host(linear.matmul(dev_x(device, x), tw, None)), orc.matmul_f64(x, orc.native_values(w, "bfp8")[0]))
    # the gate/up pair: silu((x Wg) sg) * ((x Wu) su), bfloat4_b
    k, n = 4096, 14336
    wg, wu = torch.randn(n, k, generator=g) * 0.02, torch.randn(n, k, generator=g) * 0.02
    sg, su = torch.rand(n, generator=g) + 0.5, torch.rand(n, generator=g) + 0.5
    x = torch.randn(1, k, generator=g)
    tg, _ = linear.native_weight(device, wg, ttnn.bfloat4_b)
    tu, _ = linear.native_weight(device, wu, ttnn.bfloat4_b)
    cs = (sg.to(device.torch), su.to(device.torch))
    y = host(linear.matmul(dev_x(device, x), tg, None, w_up=tu, glu=True, col_scales=cs))
    assert y.shape == (1, n)
    ag = orc.matmul_f64(x, orc.native_values(wg, "bfp4")[0])
    au = orc.matmul_f64(x, orc.native_values(wu, "bfp4")[0])
    close_bf16(y, orc.epilogue(ag, 2, acc2=au, scale=sg.numpy(), scale2=su.numpy()))
    # the same through an interleaved weight
    ti, _ = linear.native_weight(device, linear.interleave_glu(wg, wu), ttnn.bfloat4_b)
    si = linear.interleave_glu(sg[:, None], su[:, None]).reshape(-1).to(device.torch)
    y2 = host(linear.matmul(dev_x(device, x), ti, None, glu=True, col_scales=si))
    assert torch.equal(y, y2)
    del tg, tu, ti, wg, wu
    # the down projection: x W^T + residual in float32
    k, n = 14336, 4096
    w = torch.randn(n, k, generator=g) * 0.02
    tw, _ = linear.native_weight(device, w, ttnn.bfloat8_b)
    wk = orc.native_values(w, "bfp8")[0]
    for m in (1, 8, 32):
        x = torch.randn(m, k, generator=g)
        res = torch.randn(m, n, generator=g)
        tr = ttnn.from_torch(res.reshape(1, 1, m, n), dtype=ttnn.float32, layout=ttnn.TILE_LAYOUT, device=device)
        y = linear.matmul(dev_x(device, x), tw, None, residual=tr, out32=True)
        want = orc.epilogue(orc.matmul_f64(x, wk), 4, res32=res.numpy())
        got = host(y)[:m]
        assert got.dtype == torch.float32
        close_bf16(got, want)
        rel = ((got.double() - torch.from_numpy(want)).norm() / torch.from_numpy(want).norm()).item()
        assert rel < 1e-5, rel
    linear.check_status(device)


def test_lm_head_full_size(device):
    """The LM head at its own size: x [1, 4096] through a [151936, 4096] bfloat8_b weight, one top-8 record per 2048
    columns (74 full units and one of 384 columns), then the best 32 of them all. Every record equals the oracle's
    canonical top-k of the call's own bf16 outputs bit for bit, the merged 32 equal the oracle's merge of those
    records (and the canonical top-32 of the whole row), and the outputs match the oracle's sums over every column."""
    k, n, kk, top = 4096, 151936, 8, 32
    g = torch.Generator().manual_seed(5)
    w = torch.randn(n, k, generator=g) * 0.02
    x = torch.randn(1, k, generator=g)
    tw, _ = linear.native_weight(device, w, ttnn.bfloat8_b)
    units = linear.topk_units(n)
    assert units == 75
    r = linear.topk_result(device, units, 1, kk)
    out = ttnn.allocate_tensor_on_device([1, 1, 1, n], ttnn.bfloat16, ttnn.TILE_LAYOUT, device)
    spec = {"r": r, "k": kk, "rows": 1, "slot0": 0, "base": 0, "n": n, "write_y": True}
    tx = dev_x(device, x)
    linear.matmul(tx, tw, None, topk=spec, out=out)
    merged = linear.topk_merge(r, 1, kk, top)
    linear.check_status(device)
    y = host(out)
    rec = ttnn.to_torch(r).reshape(units, 2, 1, kk).numpy().view(np.uint32)
    bits = orc.bf16_bits(y[0])
    for u in range(units):
        c0, c1 = u * 2048, min((u + 1) * 2048, n)
        keys, idx = orc.topk_canonical(bits[c0:c1], c1 - c0, kk, c0)
        assert np.array_equal(rec[u, 0, 0], keys), u
        assert np.array_equal(rec[u, 1, 0], idx), u
    got = ttnn.to_torch(merged).numpy().view(np.uint32).reshape(2, 1, top)
    assert np.array_equal(got, orc.topk_merge_ref(rec, 1, kk, top))
    keys, idx = orc.topk_canonical(bits, n, top, 0)
    assert np.array_equal(got[0, 0], keys) and np.array_equal(got[1, 0], idx)
    # the same records with write_y False (the outputs stay in the call's scratch buffer)
    r2 = linear.topk_result(device, units, 1, kk)
    linear.matmul(tx, tw, None, topk={**spec, "r": r2, "write_y": False}, out=out)
    assert torch.equal(ttnn.to_torch(r2), ttnn.to_torch(r))
    del tw
    wk = orc.native_values(w, "bfp8")[0]
    close_bf16(y, orc.matmul_f64(x, wk))
    linear.check_status(device)


def test_records_as_bfloat16(device):
    """RECORDS_BF16 (the reference's linear.py:77-78, 775-778): the result tensor is bfloat16 with the same bytes as
    the uint32 words. The op, the host decode, the device merge and the LM head's pick take it unchanged."""
    from lm_head_topk import head_pick

    k, n, kk, rows = 1024, 2048 * 2 + 384, 8, 2
    g = torch.Generator().manual_seed(51)
    w = torch.randn(n, k, generator=g) * 0.02
    x = torch.randn(rows, k, generator=g)
    tw, _ = linear.native_weight(device, w, ttnn.bfloat8_b)
    tx = dev_x(device, x)
    units = linear.topk_units(n)
    spec = {"k": kk, "rows": rows, "slot0": 0, "base": 0, "n": n, "write_y": True}
    r32 = linear.topk_result(device, units, rows, kk)
    linear.matmul(tx, tw, None, topk={**spec, "r": r32})
    linear.RECORDS_BF16 = True
    try:
        r16 = linear.topk_result(device, units, rows, kk)
        assert r16.dtype == ttnn.bfloat16 and r16.shape[-1] == 4 * rows * kk
        linear.matmul(tx, tw, None, topk={**spec, "r": r16})
        a, b = ttnn.to_torch(r16), ttnn.to_torch(r32)
        assert torch.equal(a.contiguous().view(torch.int32).reshape(-1), b.reshape(-1))
        v16, i16 = linear.topk_records(r16, rows, kk)
        v32, i32 = linear.topk_records(r32, rows, kk)
        assert torch.equal(v16, v32) and torch.equal(i16, i32)
        m16 = linear.topk_merge(r16, rows, kk, 32)
        assert m16.dtype == ttnn.bfloat16
    finally:
        linear.RECORDS_BF16 = False
    m32 = linear.topk_merge(r32, rows, kk, 32)
    assert torch.equal(ttnn.to_torch(m16).contiguous().view(torch.int32).reshape(-1), ttnn.to_torch(m32).reshape(-1))
    p16 = ttnn.to_torch(head_pick.pick_records(r16, rows, kk, n))
    p32 = ttnn.to_torch(head_pick.pick_records(r32, rows, kk, n))
    assert torch.equal(p16.reshape(32, 32)[:rows, :3], p32.reshape(32, 32)[:rows, :3])
    linear.check_status(device)


def test_block_list_config4(device):
    """One launch over an attention layer's four projections (config 4) equals one call per weight, bit for bit, and
    matches the oracle."""
    k = 4096
    g = torch.Generator().manual_seed(40)
    shapes = [(4096, 0), (1024, 128), (1024, 160), (4096, 192)]
    ws = [torch.randn(n, k, generator=g) * 0.02 for n, _ in shapes]
    tws = [linear.native_weight(device, w, ttnn.bfloat8_b)[0] for w in ws]
    for m in (1, 4):
        x = torch.randn(m, k, generator=g)
        tx = dev_x(device, x)
        one = host(linear.matmul(tx, [(tw, c0) for tw, (_, c0) in zip(tws, shapes)], None))
        assert one.shape == (m, 32 * 192 + 4096)
        for tw, w, (n, c0) in zip(tws, ws, shapes):
            own = host(linear.matmul(tx, tw, None))
            assert torch.equal(one[:, 32 * c0 : 32 * c0 + n], own)
            close_bf16(own, orc.matmul_f64(x, orc.native_values(w, "bfp8")[0]))
    linear.check_status(device)


def test_topk_indices_exact(device):
    """Top-k candidate indices equal the oracle's canonical order (key descending, lower index first among ties) on
    the op's own bf16 outputs, including heavy ties, a last partial unit and write_y False."""
    k, n = 1024, 2048 * 2 + 384
    g = torch.Generator().manual_seed(50)
    w = (torch.randn(n, k, generator=g) * 4).round() / 64  # few distinct values: many exact ties in y
    x = (torch.randn(2, k, generator=g) * 2).round()
    tw, _ = linear.native_weight(device, w, ttnn.bfloat8_b)
    tx = dev_x(device, x)
    y = host(linear.matmul(tx, tw, None))
    units, kk, rows = 3, 8, 2
    for n_valid, base, write_y in ((n, 0, True), (n - 100, 5000, False)):
        r = linear.topk_result(device, units + 1, rows, kk)
        spec = {"r": r, "k": kk, "rows": rows, "slot0": 1, "base": base, "n": n_valid, "write_y": write_y}
        out = ttnn.from_torch(torch.full((1, 1, 2, n), -7.0, dtype=torch.bfloat16), dtype=ttnn.bfloat16,
                              layout=ttnn.TILE_LAYOUT, device=device)
        linear.matmul(tx, tw, None, topk=spec, out=out)
        if write_y:
            assert torch.equal(host(out), y)
        else:
            assert bool((host(out) == -7.0).all())  # never written
        rec = ttnn.to_torch(r).reshape(units + 1, 2, rows, kk).numpy().view(np.uint32)
        assert not rec[0].any()  # slot 0 untouched
        for u in range(units):
            for t in range(rows):
                c0, c1 = u * 2048, min((u + 1) * 2048, n_valid)
                keys, idx = orc.topk_canonical(orc.bf16_bits(y[t, c0:c1]), c1 - c0, kk, base + c0)
                assert np.array_equal(rec[1 + u, 0, t], keys), (u, t)
                assert np.array_equal(rec[1 + u, 1, t], idx), (u, t)
    linear.check_status(device)


@pytest.mark.parametrize("nrec,rows,k,top", [(75, 1, 8, 32), (7, 4, 8, 32), (300, 2, 16, 64), (3, 1, 4, 32)])
def test_topk_merge_exact(device, nrec, rows, k, top):
    """The device merge of records (any rank's, gathered) equals the oracle's: key descending, lower index first among
    the many equal keys, empty slots skipped, fewer candidates than `top` leave empty slots."""
    g = np.random.default_rng(nrec * 31 + rows)
    words = np.zeros((nrec, 2, rows, k), np.uint32)
    words[:, 0] = g.integers(0x8000, 0x8040, size=(nrec, rows, k))  # 64 distinct keys: heavy ties
    words[:, 0][g.random((nrec, rows, k)) < 0.2] = 0                 # empty slots
    words[:, 1] = g.permutation(nrec * rows * k).reshape(nrec, rows, k).astype(np.uint32) + 1000
    words[:, 1][words[:, 0] == 0] = 0xFFFFFFFF
    r = linear.topk_result(device, nrec, rows, k)
    r.t.copy_(torch.from_numpy(words.view(np.int32)).reshape(r.t.shape))
    got = ttnn.to_torch(linear.topk_merge(r, rows, k, top)).numpy().view(np.uint32).reshape(2, rows, top)
    assert np.array_equal(got, orc.topk_merge_ref(words, rows, k, top))
    linear.check_status(device)


def test_packed_weight_cache_round_trip(device, tmp_path):
    """A weight loaded from its cache directory is the packed weight bit for bit (stream, side array, scales), gives
    the same outputs, and a cache of other weights is refused."""
    from dense_reader import cache

    g = torch.Generator().manual_seed(77)
    w = torch.randn(384, 256, generator=g) * 0.02
    for fmt, col_scale in ((ttnn.bfloat8_b, True), (ttnn.bfloat4_b, False), (ttnn.bfloat16, False)):
        path = tmp_path / f"w_{fmt}"
        tw, ts = cache.native_weight_cached(device, w, fmt, path, col_scale=col_scale)   # packs and writes
        tw2, ts2 = cache.native_weight_cached(device, w, fmt, path, col_scale=col_scale)  # loads
        assert torch.equal(tw.t, tw2.t) and (tw.emax is None or torch.equal(tw.emax, tw2.emax))
        assert torch.equal(ts.t, ts2.t)
        tx = dev_x(device, torch.randn(3, 256, generator=g))
        assert torch.equal(host(linear.matmul(tx, tw, ts)), host(linear.matmul(tx, tw2, ts2)))
        other = torch.randn(384, 256, generator=g) * 0.02
        with pytest.raises(cache.PackCacheMismatch):
            cache.native_weight_cached(device, other, fmt, path, col_scale=col_scale)
        tw3, _ = cache.native_weight_cached(device, other, fmt, path, col_scale=col_scale, rebuild=True)
        assert not torch.equal(tw3.t, tw.t)
        tw4, _ = cache.native_weight_cached(device, other, fmt, path, col_scale=col_scale)  # the rebuilt cache, loaded
        assert torch.equal(tw4.t, tw3.t)


def test_full_size_properties(device):
    """At the benchmark configurations' full sizes (the gate weight, 14336 x 4096 bfloat4_b; the down projection's 4096 x 14336 bfloat8_b)
    the oracle is too slow for every column; size-independent properties stand in: linearity in x (power-of-two
    scaling is exact), a zero row of x gives zeros, columns of a sub-matrix equal the same columns computed alone,
    and a sample of columns against the oracle."""
    g = torch.Generator().manual_seed(60)
    for fmt, n, k in (("bfp4", 14336, 4096), ("bfp8", 4096, 14336)):
        w = torch.randn(n, k, generator=g) * 0.02
        tw, _ = linear.native_weight(device, w, DT[fmt])
        x = torch.randn(2, k, generator=g).to(torch.bfloat16).float()
        x[1] = 0
        y = host(linear.matmul(dev_x(device, x), tw, None))
        assert not y[1].any()
        y4 = host(linear.matmul(dev_x(device, x * 4), tw, None))
        assert torch.equal(y4, y * 4)
        cols = torch.randperm(n // 16, generator=g)[:24] * 16
        sub = torch.cat([w[c : c + 16] for c in cols.tolist()])
        ts, _ = linear.native_weight(device, sub, DT[fmt])
        ysub = host(linear.matmul(dev_x(device, x), ts, None))
        pick = torch.cat([y[:, c : c + 16] for c in cols.tolist()], dim=1)
        assert torch.equal(ysub, pick)
        close_bf16(ysub[:1], orc.matmul_f64(x[:1], orc.native_values(sub, fmt)[0]))
    linear.check_status(device)


def test_matmul_host_equals_matmul(device):
    """The host-buffer call (pinned x in, pinned y out, one library call) gives what matmul gives."""
    g = torch.Generator().manual_seed(70)
    k, n, m = 2048, 1024, 3
    tw, _ = linear.native_weight(device, torch.randn(n, k, generator=g) * 0.02, ttnn.bfloat8_b)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    tx = dev_x(device, torch.zeros(m, k))
    out = ttnn.allocate_tensor_on_device([1, 1, m, n], ttnn.bfloat16, ttnn.TILE_LAYOUT, device)
    x_pin, y_pin = x.contiguous().pin_memory(), torch.empty(m, n, dtype=torch.bfloat16).pin_memory()
    for _ in range(2):
        linear.matmul_host(x_pin, y_pin, tx, tw, None, out=out)
        torch.cuda.synchronize()
        want = host(linear.matmul(dev_x(device, x.float()), tw, None))
        assert torch.equal(y_pin.float(), want)
    linear.check_status(device)


def test_launch_cache_survives_freed_weights(device):
    """The launch caches hold raw addresses. A weight is freed, another of the same shape is packed (its stream
    usually lands on the freed one's address) and the same call objects are used again: the result is the new
    weight's, with and without ttnn.deallocate having been told."""
    g = torch.Generator().manual_seed(81)
    k, n = 1024, 512
    x = dev_x(device, torch.randn(2, k, generator=g))
    out = ttnn.allocate_tensor_on_device([1, 1, 2, n], ttnn.bfloat16, ttnn.TILE_LAYOUT, device)
    for told in (False, True):
        w1, w2 = torch.randn(n, k, generator=g) * 0.02, torch.randn(n, k, generator=g) * 0.02
        t1, _ = linear.native_weight(device, w1, ttnn.bfloat8_b)
        y1 = host(linear.matmul(x, t1, None, out=out)).clone()
        y1b = host(linear.matmul(x, t1, None, out=out))  # the replayed call
        assert torch.equal(y1, y1b)
        addr = t1.t.data_ptr()
        if told:
            ttnn.deallocate(t1)
        del t1
        t2, _ = linear.native_weight(device, w2, ttnn.bfloat8_b)
        y2 = host(linear.matmul(x, t2, None, out=out)).clone()
        close_bf16(y2, orc.matmul_f64(ttnn.to_torch(x).reshape(2, k).float(), orc.native_values(w2, "bfp8")[0]))
        assert not torch.equal(y1, y2), addr
    linear.check_status(device)


def test_pack_then_matmul_in_stream_order(device):
    """Through the C-ABI: a weight packed and multiplied by on one stream with no synchronisation in between. The
    matmul's first weight loads may start before the work ahead of it has finished (programmatic dependent launch)
    unless the call says the weights are fresh (TkdMatmul.weights_fresh): with it, the result equals the synchronised
    one bit for bit."""
    import ctypes

    from dense_reader import _tkd

    L = _tkd.lib()
    k, n, m = 4096, 2048, 2
    g = torch.Generator().manual_seed(91)
    npad = L.tkd_padded_cols(n)
    src = [(torch.randn(k, n, generator=g) * 0.02).to(device.torch) for _ in range(2)]
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(device.torch)
    exps = torch.empty(k * npad // 16, dtype=torch.uint8, device=device.torch)
    codes = torch.empty(k * npad, dtype=torch.uint8, device=device.torch)
    packed = torch.zeros(L.tkd_packed_bytes(_tkd.FMT_BFP8, k, n), dtype=torch.uint8, device=device.torch)
    emax = torch.zeros(npad // 16, dtype=torch.uint8, device=device.torch)
    info = torch.zeros(1, dtype=torch.int32, device=device.torch)
    st = torch.cuda.current_stream().cuda_stream

    def pack(w):
        _tkd.check(L.tkd_quantise(_tkd.FMT_BFP8, w.data_ptr(), 1, k, n, None, exps.data_ptr(), codes.data_ptr(), st), "quantise")
        _tkd.check(L.tkd_pack(_tkd.FMT_BFP8, k, n, exps.data_ptr(), codes.data_ptr(), packed.data_ptr(), emax.data_ptr(),
                              info.data_ptr(), st), "pack")

    def describe(out, fresh):
        a = _tkd.TkdMatmul()
        a.fmt, a.m, a.k, a.x, a.ldx = _tkd.FMT_BFP8, m, k, x.data_ptr(), k
        a.nblocks, a.epilogue, a.out_dtype, a.out, a.ldo = 1, _tkd.EPI_PLAIN, _tkd.DT_BF16, out.data_ptr(), n
        a.block[0].w, a.block[0].emax, a.block[0].n = packed.data_ptr(), emax.data_ptr(), n
        a.weights_fresh = fresh
        need = ctypes.c_uint64(0)
        _tkd.check(L.tkd_matmul_workspace(ctypes.byref(a), ctypes.byref(need)), "workspace")
        ws = torch.zeros(need.value, dtype=torch.uint8, device=device.torch)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        return a, ws

    outs = [torch.empty(m, n, dtype=torch.bfloat16, device=device.torch) for _ in range(3)]
    pack(src[0])
    torch.cuda.synchronize()
    a, ws = describe(outs[0], 0)
    _tkd.check(L.tkd_matmul(ctypes.byref(a), st), "tkd_matmul")  # the first weight, packed and synchronised
    torch.cuda.synchronize()
    # the second weight over the same stream, no synchronisation before its matmul
    pack(src[1])
    b, ws2 = describe(outs[1], 1)
    _tkd.check(L.tkd_matmul(ctypes.byref(b), st), "tkd_matmul")
    torch.cuda.synchronize()
    c, ws3 = describe(outs[2], 0)
    _tkd.check(L.tkd_matmul(ctypes.byref(c), st), "tkd_matmul")  # ... and after a synchronisation
    torch.cuda.synchronize()
    assert torch.equal(outs[1], outs[2]) and not torch.equal(outs[0], outs[1])
