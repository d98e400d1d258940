# SPDX-License-Identifier: Apache-2.0
# Copyright 2026 Xylolabs
# Ported from XylolabsInc/tensix-kernels, moe/tests/test_moe.py (Apache-2.0): test_decode, test_rows, test_hifi2, test_route and test_pack_cache, their
# shapes, seeds and bars are that file's; the imports and the device API under them are this package's (test_bias_groups_kblock
# without its check of gu_groups, a Tensix work split that has no counterpart here). The tests after them are this package's own.
"""The reference's MoE checks (moe/tests/test_moe.py) against this package's API on a B200: experts on the bfloat4_b
grid, x with a few outlier channels; gate_up's h and down's y against a float64 reference (relative Frobenius error below
1 %, PCC above 0.9999) for each activation; the inert options and uint32 ids bit for bit; the rows ops with each row's
own experts, rows past R zero. Then parity with the CPU oracle and the edge cases: an id past the experts, repeated
calls on one workspace, a ragged shape."""

import shutil
import tempfile
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

from common import ttnn_like as ttnn  # noqa: E402
from common.testing import check, raises, same  # noqa: E402
from moe import moe8  # noqa: E402
from oracle import oracle as orc  # noqa: E402

E, H, I, K = 16, 1024, 512, 4
BF = torch.bfloat16
REL = 0.01
REL_HIFI2 = 0.016
FID = "hifi4"


def on_grid(w, kblock=False):
    """w's values rounded to BFP4_b as tt-metal rounds them (moe8.bfp4_tiles), as float32 [K, N]."""
    k, n = w.shape
    v = moe8.bfp4_values(moe8.bfp4_tiles(w, kblock=kblock), kblock=kblock)  # [KT, NT, 32, 32]
    return torch.from_numpy(v.transpose(0, 2, 1, 3).reshape(k, n).copy())


def experts(seed, gu_scale=0.02, e=E, h=H, i=I, kblock=False):
    g = torch.Generator().manual_seed(seed)
    gu = torch.stack([on_grid(torch.randn(h, 2 * i, generator=g) * gu_scale, kblock).to(BF) for _ in range(e)])
    dn = torch.stack([on_grid(torch.randn(i, h, generator=g) * 0.02, kblock).to(BF) for _ in range(e)])
    return gu, dn


def make_x(rows, seed, h=H):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, h, generator=g)
    x[:, torch.randperm(h, generator=g)[:8]] *= 20
    return x.to(BF)


def dev(device, t, dtype, layout=ttnn.TILE_LAYOUT, mc=ttnn.DRAM_MEMORY_CONFIG):
    return ttnn.from_torch(t, dtype=dtype, layout=layout, device=device, memory_config=mc)


def decode_inputs(device, seed, ids32=False):
    g = torch.Generator().manual_seed(100 + seed)
    ids = torch.randperm(E, generator=g)[:K]
    wts = torch.softmax(torch.randn(K, generator=g), 0).to(BF)
    x = make_x(1, seed)
    idt, dt = (torch.int32, ttnn.uint32) if ids32 else (torch.int16, ttnn.uint16)
    tid = dev(device, ids.to(idt).reshape(1, 1, 1, K), dt, ttnn.ROW_MAJOR_LAYOUT)
    twt = dev(device, wts.reshape(1, 1, 1, K), ttnn.bfloat16)
    tx = dev(device, x.reshape(1, 1, 1, H), ttnn.bfloat16, mc=ttnn.L1_MEMORY_CONFIG)
    return ids, wts, x, tid, twt, tx


def host(t, cols):
    return ttnn.to_torch(t).float().reshape(-1, t.shape[-1])[:, :cols]


def test_decode(device):
    decode_case(device, FID, REL)


def decode_case(device, fid, rel):
    for act, scale in (("silu", 0.02), ("gelu_tanh", 0.02), ("swiglu_oai", 0.1)):
        gu, dn = experts(1, scale)
        P = moe8.pack(device, gu, dn)
        ids, wts, x, tid, twt, tx = decode_inputs(device, 2)
        ry, rh = moe8.reference(x.float(), gu, dn, ids.tolist(), wts.float(), act)
        outs = {}
        for loaders in (1, 2):
            th = moe8.gate_up(tx, P, tid, twt, K, act=act, loaders=loaders, fidelity=fid)
            ty = moe8.down(th, P, tid, K, loaders=loaders, fidelity=fid)
            outs[loaders] = (host(th, K * I)[:1], host(ty, H)[:1])
            check(f"{act} gate_up h, {fid}, loaders {loaders}", outs[loaders][0], rh, rel=rel)
            check(f"{act} down y, {fid}, loaders {loaders}", outs[loaders][1], ry, rel=rel)
        same(f"{act} h: two loaders against one", outs[2][0], outs[1][0])
        same(f"{act} y: two loaders against one", outs[2][1], outs[1][1])
        if act == "silu" and fid == FID:
            cpb = 2 if P["cpb"] != 2 else 1
            th = moe8.gate_up(tx, P, tid, twt, K, act=act, cpb=cpb, fidelity=fid)
            same(f"h with {cpb} cores a bank against the pack's {P['cpb']}", host(th, K * I)[:1], outs[2][0])
            _, _, _, tid32, twt32, tx32 = decode_inputs(device, 2, ids32=True)
            th = moe8.gate_up(tx32, P, tid32, twt32, K, act=act, ids32=True, fidelity=fid)
            ty = moe8.down(th, P, tid32, K, ids32=True, fidelity=fid)
            same("h with uint32 ids", host(th, K * I)[:1], outs[2][0])
            same("y with uint32 ids", host(ty, H)[:1], outs[2][1])


def test_bias_groups_kblock(device):
    gu, dn = experts(3, 0.1, kblock=True)
    g = torch.Generator().manual_seed(4)
    gb = torch.randn(E, 2 * I, generator=g) * 0.5
    P = moe8.pack(device, gu, dn, banks=2, gu_bias=gb, kblock=True)
    for act in ("swiglu_oai", "silu"):
        ids, wts, x, tid, twt, tx = decode_inputs(device, 5)
        ry, rh = moe8.reference(x.float(), gu, dn, ids.tolist(), wts.float(), act, gb)
        th = moe8.gate_up(tx, P, tid, twt, K, act=act, loaders=2, fidelity=FID)
        ty = moe8.down(th, P, tid, K, loaders=2, fidelity=FID)
        check(f"{act} with a bias, column groups and K blocks, {FID}: h", host(th, K * I)[:1], rh, rel=REL)
        check(f"{act} with a bias, column groups and K blocks, {FID}: y", host(ty, H)[:1], ry, rel=REL)
    rows_case(device, gu, dn, P, 6, act="swiglu_oai", gb=gb, loaders=(1, 2), seed=6)


def test_bias(device):
    """(this package's) the bias on the ordinary layout."""
    gu, dn = experts(3, 0.1)
    g = torch.Generator().manual_seed(4)
    gb = torch.randn(E, 2 * I, generator=g) * 0.5
    P = moe8.pack(device, gu, dn, gu_bias=gb)
    ids, wts, x, tid, twt, tx = decode_inputs(device, 5)
    ry, rh = moe8.reference(x.float(), gu, dn, ids.tolist(), wts.float(), "silu", gb)
    th = moe8.gate_up(tx, P, tid, twt, K, fidelity=FID)
    check(f"silu with a bias, {FID}: h", host(th, K * I)[:1], rh, rel=REL)
    check(f"silu with a bias, {FID}: y", host(moe8.down(th, P, tid, K, fidelity=FID), H)[:1], ry, rel=REL)


def rows_inputs(device, R, seed, ids32=False):
    g = torch.Generator().manual_seed(200 + seed)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(R)])
    wts = torch.softmax(torch.randn(R, K, generator=g), -1).to(BF)
    x = make_x(R, seed)
    idt, dt = (torch.int32, ttnn.uint32) if ids32 else (torch.int16, ttnn.uint16)
    tid = dev(device, ids.to(idt).reshape(1, 1, R, K), dt)
    twt = dev(device, wts.reshape(1, 1, R, K), ttnn.bfloat16)
    tx = dev(device, x.reshape(1, 1, R, H), ttnn.bfloat16)
    return ids, wts, x, tid, twt, tx


def rows_case(device, gu, dn, P, R, act="silu", gb=None, loaders=(1,), seed=0, ids32=False, fid=FID):
    ids, wts, x, tid, twt, tx = rows_inputs(device, R, seed, ids32)
    ref = moe8.reference_rows(x.float(), gu, dn, ids.tolist(), wts.float(), act, gb)
    u = moe8.union(ids, E)
    href = torch.zeros(R, len(u) * I, dtype=torch.float64)
    for r in range(R):
        _, hr = moe8.reference(x[r : r + 1].float(), gu, dn, ids[r].tolist(), wts[r].float(), act, gb)
        for s, e in enumerate(ids[r].tolist()):
            q = u.index(e)
            href[r, q * I : (q + 1) * I] = hr[0, s * I : (s + 1) * I]
    outs = []
    for ld in loaders:
        th = moe8.gate_up_rows(tx, P, tid, twt, K, R, act=act, loaders=ld, ids32=ids32, fidelity=fid)
        ty = moe8.down_rows(th, P, tid, K, R, loaders=ld, ids32=ids32, fidelity=fid)
        hd = host(th, len(u) * I)[:R]
        yall = host(ty, H)
        name = f"rows {R} ({act}{', bias' if gb is not None else ''}{', uint32 ids' if ids32 else ''}), {fid}, loaders {ld}"
        bar = REL if fid == "hifi4" else REL_HIFI2
        check(f"{name}: h", hd, href, rel=bar)
        check(f"{name}: y", yall[:R], ref, rel=bar)
        same(f"{name}: rows past R zero", yall[R:32], torch.zeros(32 - R, H))
        outs.append((hd, yall))
    for (h1, y1), (h2, y2), ld in zip(outs, outs[1:], loaders[1:]):
        same(f"rows {R}: h with {ld} loaders against {loaders[0]}", h2, h1)
        same(f"rows {R}: y with {ld} loaders against {loaders[0]}", y2, y1)
    return outs


def test_rows(device):
    gu, dn = experts(7)
    P = moe8.pack(device, gu, dn)
    rows_case(device, gu, dn, P, 1, seed=1)
    rows_case(device, gu, dn, P, 5, loaders=(1, 2), seed=2)
    rows_case(device, gu, dn, P, 32, act="gelu_tanh", seed=3)
    rows_case(device, gu, dn, P, 5, seed=2, ids32=True)


def test_hifi2(device):
    decode_case(device, "hifi2", REL_HIFI2)
    gu, dn = experts(7)
    P = moe8.pack(device, gu, dn)
    rows_case(device, gu, dn, P, 5, loaders=(1, 2), seed=2, fid="hifi2")
    rows_case(device, gu, dn, P, 32, act="gelu_tanh", seed=3, fid="hifi2")


def ulps(a, b):
    """|a - b| in bf16 ulps of b (bf16 tensors)."""
    return (a.view(torch.int16).to(torch.int32) - b.view(torch.int16).to(torch.int32)).abs()


def edge_rows(e, k, g):
    """32 rows of logits [32, e] that a range or sign error shows in: all equal, near 0, tiny, large, huge, ties at the
    k-th place, two values, signs mixed, the rest random."""
    rows = [
        torch.zeros(e),
        torch.full((e,), 1.5),
        torch.full((e,), -2.0),
        torch.randn(e, generator=g) * 1e-3,
        torch.randn(e, generator=g) * 1e-6,
        torch.randn(e, generator=g) * 40,
        torch.randn(e, generator=g) * 1e3,
    ]
    t = torch.randn(e, generator=g)
    t[: 2 * k] = 2.5  # 2k equal at the top: the pick is the lowest k ids of them
    rows.append(t)
    t = torch.randn(e, generator=g)
    t[torch.randperm(e, generator=g)[: k + 3]] = 1.25  # ties across the k-th place
    rows.append(t)
    rows.append(torch.where(torch.rand(e, generator=g) < 0.5, torch.tensor(-1.0), torch.tensor(1.0)))
    rows.append(torch.randn(e, generator=g).abs())
    rows.append(-torch.randn(e, generator=g).abs())
    while len(rows) < 32:
        rows.append(torch.randn(e, generator=g) * float(2 ** (len(rows) % 7 - 3)))
    return torch.stack(rows)


def route_case(device, g, name, kind, R, k, ids32=False, bias=False, edge=False, **opts):
    e = 128
    lg = edge_rows(e, k, g) if edge else torch.randn(R, e, generator=g) * 3
    if not edge:
        lg[::2] = lg[::2].to(BF).float()  # ties in the even rows
    R = lg.shape[0]
    tl = dev(device, lg.reshape(1, 1, R, e), ttnn.float32)
    kk = k + (opts.get("slot") is not None)
    idt, tdt = (torch.int32, ttnn.uint32) if ids32 else (torch.int16, ttnn.uint16)
    junk = torch.full((1, 1, R, kk), 7)
    ti = dev(device, junk.to(idt), tdt)
    tw = dev(device, junk.to(BF), ttnn.bfloat16)
    b, tb = None, None
    if bias:
        b = torch.randn(e, generator=g) * 0.1
        tb = dev(device, b.reshape(1, 1, 1, e), ttnn.float32)
    moe8.route(tl, ti, tw, k, kind=kind, bias=tb, ids32=ids32, **opts)
    gi = ttnn.to_torch(ti).reshape(R, kk).long() & (0xFFFFFFFF if ids32 else 0xFFFF)
    gw = ttnn.to_torch(tw).reshape(R, kk).to(BF)
    ri, rw = moe8.route_reference(lg, k, kind, b, **opts)
    same(f"route {name}: picks", gi, ri)
    tol = 2.0**-29 * max(1.0, opts.get("scale", 1.0))
    bad = (ulps(gw, rw.to(BF)) > 1) & ((gw.double() - rw).abs() > tol)
    ok = int(bad.sum()) == 0
    print(f"{'ok  ' if ok else 'FAIL'} route {name}: weights within 1 bf16 ulp or {tol:.0e}: {int(bad.sum())} off")
    assert ok, name


def test_route(device):
    g = torch.Generator().manual_seed(3)
    route_case(device, g, "softmax R 1 k 8", "softmax", 1, 8)
    route_case(device, g, "softmax R 4 k 6 uint32", "softmax", 4, 6, ids32=True)
    route_case(device, g, "softmax edge rows k 8", "softmax", 32, 8, edge=True)
    route_case(device, g, "sigmoid + bias R 4 k 8", "sigmoid", 4, 8, bias=True)
    route_case(device, g, "sigmoid + bias edge rows k 6 uint32", "sigmoid", 32, 6, ids32=True, bias=True, edge=True)
    route_case(device, g, "sigmoid, no bias, R 4 k 8", "sigmoid", 4, 8)
    route_case(device, g, "sigmoid, no bias, not normalized, edge rows", "sigmoid", 32, 8, edge=True, norm=False)
    route_case(
        device, g, "sigmoid + bias, groups 8/4, scale 2.5, slot", "sigmoid", 8, 8, bias=True,
        groups=(8, 4), scale=2.5, slot=128,
    )


def test_pack_cache(device):
    gu, dn = experts(9)
    banks = moe8.dram_banks(device)
    tmp = Path(tempfile.mkdtemp(prefix="moe8-cache-"))
    try:
        cache = tmp / "layer0"
        cpb = moe8._clamp_cpb(device, banks, 3)  # (pack's cores a bank on this grid)
        assert moe8.prepack(gu, dn, cache, banks, cpb) is True
        assert moe8.prepack(gu, dn, cache, banks, cpb) is False  # already there
        ids, wts, x, tid, twt, tx = decode_inputs(device, 8)
        P0 = moe8.pack(device, gu, dn)
        P1 = moe8.pack_cached(device, cache)
        h0, h1 = moe8.gate_up(tx, P0, tid, twt, K), moe8.gate_up(tx, P1, tid, twt, K)
        same("pack_cached against pack: h", host(h1, K * I), host(h0, K * I))
        same("pack_cached against pack: y", host(moe8.down(h1, P1, tid, K), H), host(moe8.down(h0, P0, tid, K), H))
        other = experts(10)
        raises("a cache of other weights", moe8.PackCacheMismatch, lambda: moe8.prepack(*other, cache, banks, cpb))
        raises("a cache of another split", moe8.PackCacheMismatch, lambda: moe8.pack_cached(device, cache, cores_per_bank=1))
        assert moe8.repack_down(cache, cores_per_bank=1) is True
        P2 = moe8.pack_cached(device, cache, cores_per_bank=1)
        P3 = moe8.pack(device, gu, dn, cores_per_bank=1)
        same("repack_down against a fresh pack: y", host(moe8.down(h0, P2, tid, K), H), host(moe8.down(h0, P3, tid, K), H))
        # (this package's addition) pack(cache=) takes the directory too, and rebuild=True packs over other weights' cache
        P5 = moe8.pack_upload(device, moe8.pack_host(gu, dn, banks, 1, device=device))
        same("pack_upload of pack_host against pack: y", host(moe8.down(h0, P5, tid, K), H), host(moe8.down(h0, P3, tid, K), H))
        P4 = moe8.pack(device, gu, dn, cores_per_bank=1, cache=cache)
        same("pack(cache=) against pack: y", host(moe8.down(h0, P4, tid, K), H), host(moe8.down(h0, P3, tid, K), H))
        moe8.pack(device, *other, cores_per_bank=1, cache=cache, rebuild=True)
        raises("the cache now holds the other weights", moe8.PackCacheMismatch,
               lambda: moe8.pack(device, gu, dn, cores_per_bank=1, cache=cache))
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


# ---- this package's own checks


def bf16_close(got, want, what, tol=1e-2):
    """got (bf16 values) against the oracle's float64: within a bf16 rounding of the result plus the fp32 sums' error."""
    want = torch.as_tensor(want).float()
    err = (got.float() - want).abs().max().item()
    scale = want.abs().max().item()
    assert err <= tol * scale, (what, err, scale)


def test_decode_against_the_oracle_ragged_and_invalid_ids(device):
    """A shape whose K ends inside a super-atom of 64 (H 96, I 96) and whose columns end inside a panel of 128; an id at or
    past the experts gives zeros in its slot and nothing in y; a second call on the same workspace gives the same bits."""
    e, h, i, k = 5, 96, 96, 3
    gu, dn = experts(11, 0.1, e, h, i)
    P = moe8.pack(device, gu, dn)
    x = make_x(1, 12, h)
    wts = torch.tensor([0.5, 0.25, 0.25]).to(BF)
    for ids in ([4, 0, 2], [1, 7, 3]):
        tid = dev(device, torch.tensor(ids, dtype=torch.int16).reshape(1, 1, 1, k), ttnn.uint16, ttnn.ROW_MAJOR_LAYOUT)
        twt = dev(device, wts.reshape(1, 1, 1, k), ttnn.bfloat16)
        tx = dev(device, x.reshape(1, 1, 1, h), ttnn.bfloat16)
        valid = [(s, v) for s, v in enumerate(ids) if v < e]
        oy, oh = orc.moe_reference(x.float().numpy(), gu.float().numpy(), dn.float().numpy(), [v for _, v in valid],
                                   [float(wts[s]) for s, _ in valid], "silu")
        want_h = torch.zeros(1, k * i, dtype=torch.float64)
        for j, (s, _) in enumerate(valid):
            want_h[0, s * i : (s + 1) * i] = torch.from_numpy(oh[0, j * i : (j + 1) * i])
        th = moe8.gate_up(tx, P, tid, twt, k)
        ty = moe8.down(th, P, tid, k)
        bf16_close(host(th, k * i)[:1], want_h, f"h {ids}")
        # (y against the oracle's y from the device's own bf16 h would be tighter; the float64 chain is within the bar too)
        bf16_close(host(ty, h)[:1], oy, f"y {ids}", tol=2e-2)
        if len(valid) < k:
            s_bad = next(s for s, v in enumerate(ids) if v >= e)
            assert not host(th, k * i)[0, s_bad * i : (s_bad + 1) * i].any()
        ty2 = moe8.down(th, P, tid, k)
        same(f"down twice on one workspace {ids}", host(ty2, h), host(ty, h))


def test_rows_many_inputs_in_passes(device):
    """32 rows of 4096 inputs do not fit in shared memory at once: the kernel takes them in passes of 16 and gives what the
    reference gives."""
    e, h, i, k, R = 4, 4096, 64, 2, 32
    gu, dn = experts(13, 0.02, e, h, i)
    P = moe8.pack(device, gu, dn)
    g = torch.Generator().manual_seed(14)
    ids = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(R)])
    wts = torch.softmax(torch.randn(R, k, generator=g), -1).to(BF)
    x = make_x(R, 15, h)
    tid = dev(device, ids.to(torch.int16).reshape(1, 1, R, k), ttnn.uint16)
    twt = dev(device, wts.reshape(1, 1, R, k), ttnn.bfloat16)
    tx = dev(device, x.reshape(1, 1, R, h), ttnn.bfloat16)
    oy, oh = orc.moe_reference_rows(x.float().numpy(), gu.float().numpy(), dn.float().numpy(), ids.numpy(),
                                    wts.float().numpy(), e)
    th = moe8.gate_up_rows(tx, P, tid, twt, k, R)
    ty = moe8.down_rows(th, P, tid, k, R)
    check("rows in passes: h", host(th, oh.shape[1])[:R], torch.from_numpy(oh), rel=REL)
    check("rows in passes: y", host(ty, h)[:R], torch.from_numpy(oy), rel=REL)


def test_route_against_the_oracle_and_into_the_layer(device):
    """The router's picks and weights against the oracle on the golden logits (ties, equal rows, large and tiny logits), the
    shared expert's gate, and the routed ids and weights driving gate_up and down with nothing read back in between."""
    import numpy as np
    from pathlib import Path

    m = np.load(Path(__file__).resolve().parent / "golden" / "moe.npz")
    lg, rb = torch.from_numpy(m["route_logits"]), torch.from_numpy(m["route_bias"])
    R, e, k = lg.shape[0], lg.shape[1], 6
    wide = torch.cat([lg, torch.linspace(-3, 3, R).reshape(R, 1), torch.zeros(R, 31)], 1)  # column e: a shared expert's gate
    tl = dev(device, wide.reshape(1, 1, R, e + 32), ttnn.float32)
    tb = dev(device, rb.reshape(1, 1, 1, e), ttnn.float32)
    for name, kw in (("softmax", dict(kind="softmax")), ("sigmoid_raw", dict(kind="sigmoid", norm=False)),
                     ("sigmoid_bias", dict(kind="sigmoid", bias=True)),
                     ("groups", dict(kind="sigmoid", bias=True, groups=(8, 3), scale=2.5, slot=64))):
        kk = k + ("slot" in kw)
        ti = dev(device, torch.zeros(1, 1, R, kk, dtype=torch.int16), ttnn.uint16)
        tw = dev(device, torch.zeros(1, 1, R, kk).to(BF), ttnn.bfloat16)
        tsh = dev(device, torch.zeros(1, 1, R, 1).to(BF), ttnn.bfloat16)
        okw = {**kw, "bias": rb.numpy() if kw.get("bias") else None}
        moe8.route(tl, ti, tw, k, experts=e, shared=tsh, **{**kw, "bias": tb if kw.get("bias") else None})
        oi, ow = orc.moe_route_reference(lg.numpy(), k, **okw)
        assert np.array_equal(ttnn.to_torch(ti).reshape(R, kk).long().numpy() & 0xFFFF, oi), name
        got = ttnn.to_torch(tw).reshape(R, kk).float().numpy()
        assert np.allclose(got, ow, rtol=2.0**-8, atol=0), name  # (a bf16 rounding)
        gate = torch.sigmoid(torch.linspace(-3, 3, R).double()).to(BF)
        assert int(ulps(ttnn.to_torch(tsh).reshape(R).to(BF), gate).max()) <= 1, name
    # route -> gate_up -> down on the device, against the oracle given the same picks
    g = torch.Generator().manual_seed(41)
    gu, dn = experts(17, 0.05, 32, 128, 64)
    P = moe8.pack(device, gu, dn)
    x = make_x(1, 18, 128)
    logits = torch.randn(1, 32, generator=g)
    tl = dev(device, logits.reshape(1, 1, 1, 32), ttnn.float32)
    ti = dev(device, torch.zeros(1, 1, 1, 4, dtype=torch.int16), ttnn.uint16)
    tw = dev(device, torch.zeros(1, 1, 1, 4).to(BF), ttnn.bfloat16)
    tx = dev(device, x.reshape(1, 1, 1, 128), ttnn.bfloat16)
    ty = moe8.down(moe8.gate_up(tx, P, ti, moe8.route(tl, ti, tw, 4), 4), P, ti, 4)
    oi, ow = orc.moe_route_reference(logits.numpy(), 4)
    wb = torch.from_numpy(ow[0]).to(BF).float().numpy()
    oy, _ = orc.moe_reference(x.float().numpy(), gu.float().numpy(), dn.float().numpy(), oi[0].tolist(), wb)
    bf16_close(host(ty, 128)[:1], oy, "routed layer y", tol=2e-2)


def test_kblock_pack_holds_the_host_quantisers_values(device):
    """A K-block pack of weights that are NOT on the grid holds exactly what bfp4_tiles(kblock=True) makes of them (pinned
    by the golden vectors), ragged shapes included; and it goes through the cache."""
    import numpy as np
    from dense_reader import _tkd

    L = _tkd.lib()
    e, h, i = 2, 96, 160
    g = torch.Generator().manual_seed(23)
    gu = torch.randn(e, h, 2 * i, generator=g) * torch.exp2(torch.randint(-6, 6, (e, h, 1), generator=g).float())
    dn = torch.randn(e, i, h, generator=g) * 0.05
    P = moe8.pack(device, gu, dn, kblock=True)
    assert P["kblock"] and P["fmt"] == _tkd.FMT_BF16 and P["gu_emax"] is None
    for name, mats, k, n in (("gu", moe8._glu_order(gu, i), h, 2 * i), ("dn", dn, i, h)):
        for x in range(e):
            out = torch.empty(k, L.tkd_padded_cols(n), dtype=torch.float32, device=device.torch)
            _tkd.check(L.tkd_unpack(_tkd.FMT_BF16, k, n, P[name].t[x].data_ptr(), None, out.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream), "tkd_unpack")
            want = on_grid(mats[x], kblock=True)
            assert np.array_equal(out[:, :n].cpu().numpy().view(np.uint32), want.numpy().view(np.uint32)), (name, x)
    tmp = Path(tempfile.mkdtemp(prefix="moe8-kblock-"))
    try:
        P1 = moe8.pack(device, gu, dn, kblock=True, cache=tmp / "l")
        P2 = moe8.pack_cached(device, tmp / "l", kblock=True)
        assert torch.equal(P1["gu"].t, P["gu"].t) and torch.equal(P2["dn"].t, P["dn"].t)
        raises("a K-block cache taken as an ordinary one", moe8.PackCacheMismatch, lambda: moe8.pack_cached(device, tmp / "l"))
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
