"""The mixture-of-experts sibling without a GPU: the package's host functions (moe/moe8.py: bfp4_tiles, bfp4_values,
reference, reference_rows, union) and the oracle's restatement against the golden vectors made by running the
reference (tests/golden/gen_golden.py, section 8, and the quantiser's vectors of section 1-3), and the refusals of what
is not built."""

import hashlib
from pathlib import Path

import numpy as np
import pytest
import torch

from moe import moe8
from oracle import oracle as orc

G = Path(__file__).resolve().parent / "golden"
sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()  # noqa: E731
BF = torch.bfloat16


@pytest.fixture(scope="module")
def m():
    return np.load(G / "moe.npz")


@pytest.fixture(scope="module")
def q():
    return np.load(G / "quantiser_bfp4.npz")


def retile(v):
    kt, nt = v.shape[:2]
    return np.ascontiguousarray(v.transpose(0, 2, 1, 3).reshape(kt * 32, nt * 32))


def test_bfp4_tiles_and_values_match_the_reference(q, m):
    g = torch.Generator().manual_seed(0)
    w1 = torch.randn(256, 512, generator=g) * 0.02
    w1[3, 5], w1[7, 9] = 0.0, -1e-30
    t1 = moe8.bfp4_tiles(w1)
    assert np.array_equal(t1, q["t1"])
    assert sha(retile(moe8.bfp4_values(t1))) == str(q["v1_sha"])
    assert sha(moe8.bfp4_tiles(w1, kblock=True)) == str(m["t1_kblock_sha"])
    # wide exponent spreads, denormals, zeros, huge values; the same tiles with the exponents along K
    assert np.array_equal(moe8.bfp4_tiles(q["w4"]), q["t4"])
    assert np.array_equal(retile(moe8.bfp4_values(q["t4"])), q["v4"])
    assert np.array_equal(moe8.bfp4_tiles(q["w4"], kblock=True), m["t4_kblock"])
    assert np.array_equal(retile(moe8.bfp4_values(m["t4_kblock"], kblock=True)), m["v4_kblock"])
    # the rounding cases of one face row, and the oracle's quantiser on the same inputs
    assert np.array_equal(retile(moe8.bfp4_values(moe8.bfp4_tiles(q["w3"]))), q["v3"])
    e, c = orc.quantise_c(q["w4"], "bfp4")
    assert np.array_equal(orc.tiles(e, c, "bfp4"), moe8.bfp4_tiles(q["w4"]))


def inputs(m):
    x = torch.from_numpy(m["x_bits"]).view(BF)
    w = torch.from_numpy(m["w_bits"]).view(BF)
    return x, w, torch.from_numpy(m["gu"]), torch.from_numpy(m["dn"]), torch.from_numpy(m["gb"]), torch.from_numpy(m["ids"])


def test_references_match_the_reference(m):
    x, w, gu, dn, gb, ids = inputs(m)
    for act in ("silu", "gelu_tanh", "swiglu_oai"):
        for bias, tag in ((None, ""), (gb, "b")):
            y, h = moe8.reference(x[:1].float(), gu, dn, ids[0].tolist(), w[0].float(), act, bias)
            assert np.allclose(y.numpy(), m[f"y{tag}_{act}"], rtol=1e-12, atol=1e-15)
            assert np.allclose(h.numpy(), m[f"h{tag}_{act}"], rtol=1e-12, atol=1e-15)
            oy, oh = orc.moe_reference(x[:1].float().numpy(), gu.numpy(), dn.numpy(), ids[0].tolist(), w[0].float().numpy(),
                                       act, None if bias is None else bias.numpy())
            assert np.allclose(oy, m[f"y{tag}_{act}"], rtol=1e-9, atol=1e-12), act
            assert np.allclose(oh, m[f"h{tag}_{act}"], rtol=1e-9, atol=1e-12), act
    rows = moe8.reference_rows(x.float(), gu, dn, ids.tolist(), w.float(), "silu")
    assert np.allclose(rows.numpy(), m["rows_silu"], rtol=1e-12, atol=1e-15)
    oy, oh = orc.moe_reference_rows(x.float().numpy(), gu.numpy(), dn.numpy(), ids.numpy(), w.float().numpy(), 6,
                                    "swiglu_oai", gb.numpy())
    assert np.allclose(oy, m["rows_oai_bias"], rtol=1e-9, atol=1e-12)
    un = orc.moe_union(ids.numpy(), 6)
    assert oh.shape == (4, len(un) * 32)
    # a row's columns of an expert it did not choose are zero
    for r in range(4):
        for qi, e in enumerate(un):
            assert (e in ids[r].tolist()) == bool(np.any(oh[r, qi * 32 : (qi + 1) * 32] != 0))


def test_union(m):
    ids = torch.from_numpy(m["ids"])
    assert moe8.union(ids, 6) == m["union"].tolist() == orc.moe_union(ids.numpy(), 6)
    clip = torch.tensor([[5, 9, 2], [2, 7, 0]])
    assert moe8.union(clip, 6) == m["union_clip"].tolist() == orc.moe_union(clip.numpy(), 6) == [0, 2, 5]
    assert moe8.u_max({"E": 16}, 5, 4) == 16 and moe8.u_max({"E": 128}, 5, 4) == 20


def test_glu_order():
    assert moe8._glu_order(torch.arange(128.0).reshape(1, 128), 64)[0, :64].tolist() == [
        *range(64, 96), *range(0, 32)]  # gate tile 0 (columns I ..), then up tile 0


ROUTE_CASES = {
    "softmax": dict(kind="softmax"), "sigmoid": dict(kind="sigmoid"), "sigmoid_raw": dict(kind="sigmoid", norm=False),
    "sigmoid_bias": dict(kind="sigmoid", bias=True), "groups": dict(kind="sigmoid", bias=True, groups=(8, 3), scale=2.5, slot=64),
}


def test_route_reference_and_sigmoid_table_match_the_reference(m):
    lg, rb = torch.from_numpy(m["route_logits"]), torch.from_numpy(m["route_bias"])
    for name, kw in ROUTE_CASES.items():
        kw = {**kw, "bias": rb if kw.get("bias") else None}
        ids, w = moe8.route_reference(lg, 6, **kw)
        assert np.array_equal(ids.numpy(), m[f"route_ids_{name}"]), name
        assert np.allclose(w.numpy(), m[f"route_w_{name}"], rtol=1e-13, atol=0), name
        okw = {**kw, "bias": None if kw["bias"] is None else rb.numpy()}
        oi, ow = orc.moe_route_reference(lg.numpy(), 6, **okw)
        assert np.array_equal(oi, m[f"route_ids_{name}"]), name
        assert np.allclose(ow, m[f"route_w_{name}"], rtol=1e-12, atol=0), name
    assert moe8.sigmoid_table() == m["sigmoid_table"].tolist()


class HostDevice:
    """What the cache functions ask of a device, over host memory (no kernel is launched by pack_cached)."""

    torch = torch.device("cpu")

    def dram_grid_size(self):
        from common import ttnn_like as ttnn
        return ttnn.Grid(8, 1)

    def compute_with_storage_grid_size(self):
        from common import ttnn_like as ttnn
        return ttnn.Grid(148, 1)


def test_pack_cache_identity_and_refusals(tmp_path):
    """A cache directory written by the package's own writer, read back through pack_cached: taken when the call matches
    its meta, refused (and left alone) for another split, another layout version, a changed array, a missing bias;
    repack_down renames the split."""
    import json

    from dense_reader import _tkd
    from dense_reader import cache as wcache

    L = _tkd.lib()
    E, H, I = 3, 64, 32
    g = torch.Generator().manual_seed(5)
    gu, dn = torch.randn(E, H, 2 * I, generator=g), torch.randn(E, I, H, generator=g)
    dev = HostDevice()
    meta = moe8._meta(gu, dn, 8, 3, None)
    assert meta["gate_up"] != moe8._meta(gu + 1, dn, 8, 3, None)["gate_up"]
    arrays = {"gu": np.arange(E * L.tkd_packed_bytes(1, H, 2 * I), dtype=np.int64).astype(np.uint8).reshape(E, -1),
              "gu_emax": np.full((E, L.tkd_padded_cols(2 * I) // 16), 120, np.uint8),
              "dn": np.ones((E, L.tkd_packed_bytes(1, I, H)), np.uint8),
              "dn_emax": np.full((E, L.tkd_padded_cols(H) // 16), 121, np.uint8), "bias": None}
    cache = tmp_path / "layer0"
    wcache.write(cache, meta, arrays, names=moe8._CACHE_ARRAYS)
    P = moe8.pack_cached(dev, cache)
    assert (P["E"], P["H"], P["I"], P["cpb"], P["banks"], P["gu_bias"]) == (E, H, I, 3, 8, False)
    assert np.array_equal(P["gu"].t.numpy(), arrays["gu"]) and np.array_equal(P["dn_emax"].numpy(), arrays["dn_emax"])
    before = sorted(p.name for p in cache.iterdir())
    with pytest.raises(moe8.PackCacheMismatch, match="cpb"):
        moe8.pack_cached(dev, cache, cores_per_bank=1)
    with pytest.raises(moe8.PackCacheMismatch, match="a bias"):
        moe8.pack_cached(dev, cache, gu_bias=True)
    assert moe8.repack_down(cache, cores_per_bank=1) is True and moe8.repack_down(cache, cores_per_bank=1) is False
    assert moe8.pack_cached(dev, cache, cores_per_bank=1)["cpb"] == 1
    assert json.loads((cache / "meta.json").read_text()) == moe8._meta(gu, dn, 8, 1, None)  # a fresh pack's meta at that split
    # a changed array is caught by its checksum (and taken unchecked only on request)
    bad = arrays["dn"].copy()
    bad[1, 7] ^= 1
    np.save(cache / "dn.npy", bad)
    with pytest.raises(moe8.PackCacheMismatch, match="dn.npy"):
        moe8.pack_cached(dev, cache, cores_per_bank=1)
    assert moe8.pack_cached(dev, cache, cores_per_bank=1, verify=False)["dn"].t[1, 7] == bad[1, 7]
    # another stream layout
    m2 = json.loads((cache / "meta.json").read_text())
    m2["layout_version"] += 1
    (cache / "meta.json").write_text(json.dumps(m2))
    with pytest.raises(moe8.PackCacheMismatch, match="layout_version"):
        moe8.pack_cached(dev, cache, cores_per_bank=1, verify=False)
    assert sorted(p.name for p in cache.iterdir()) == before
    with pytest.raises(moe8.PackCacheMismatch):
        moe8.pack_cached(dev, tmp_path / "nothing")
    with pytest.raises(moe8.PackCacheMismatch, match="kblock"):
        moe8.pack_cached(dev, cache, cores_per_bank=1, kblock=True, verify=False)


def test_cabi_refuses_bad_requests_before_any_launch():
    """The entry points check their arguments on the host first: these calls return TKD_ERR_BAD_ARG (1) without a GPU."""
    import ctypes

    from dense_reader import _tkd

    L = _tkd.lib()
    buf = (ctypes.c_uint8 * 4096)()
    addr = (ctypes.addressof(buf) + 15) & ~15

    def moe(**kw):
        a = _tkd.TkdMoe()
        a.w, a.emax, a.x, a.ids, a.out, a.route_w = addr, addr, addr, addr, addr, addr
        a.fmt, a.experts, a.k_in, a.n, a.rows, a.k, a.slots = _tkd.FMT_BFP4, 4, 64, 64, 1, 2, 2
        a.expert_bytes = L.tkd_packed_bytes(_tkd.FMT_BFP4, 64, 64)
        a.ldx, a.ldo, a.ld_ids, a.ld_w = 64, 64, 2, 2
        for k, v in kw.items():
            setattr(a, k, v)
        return a

    need = ctypes.c_uint64(0)
    assert L.tkd_moe_workspace(ctypes.byref(moe(rows=3, by_union=1, slots=4)), ctypes.byref(need)) == 0
    assert need.value == 256 + 4 * 3 * 128 * 4  # the units' counters, then slots x rows x padded columns of float32
    for bad in (dict(k=0), dict(k=17), dict(k_in=48), dict(n=48), dict(rows=2), dict(rows=33, by_union=1), dict(fmt=0),
                dict(slots=3), dict(expert_bytes=16), dict(ldx=60), dict(act=3), dict(emax=None), dict(ids=None),
                dict(by_union=1, experts=2048, slots=2), dict(x=addr + 2)):
        assert L.tkd_moe_gate_up(ctypes.byref(moe(**bad)), None) == 1, bad
    assert L.tkd_moe_gate_up(ctypes.byref(moe(route_w=None)), None) == 1
    for bad in (dict(ldx=64), dict(ldo=32), dict(k=0)):  # (down: the row of h holds slots x k_in inputs)
        assert L.tkd_moe_down(ctypes.byref(moe(**bad)), None) == 1, bad

    def route(**kw):
        args = dict(logits=addr, ld=64, rows=2, experts=64, k=4, kind=0, bias=None, scale=1.0, norm=1, ng=1, tg=1, has_slot=0,
                    slot=0, ids=addr, ids32=0, ld_ids=4, w=addr, ld_w=4, shared=None, ld_sh=0)
        args.update(kw)
        return L.tkd_moe_route(*args.values(), None)

    for bad in (dict(rows=33), dict(experts=48), dict(experts=2048, ld=2048), dict(k=17), dict(k=16, has_slot=1, ld_ids=17, ld_w=17),
                dict(kind=1), dict(kind=3), dict(scale=4.0), dict(scale=0.0), dict(norm=0), dict(ld=32), dict(ld_ids=3),
                dict(kind=2, ng=8, tg=2), dict(kind=1, bias=addr, ng=8, tg=9), dict(kind=1, bias=addr, ng=64, tg=1),
                dict(shared=addr, ld=64)):
        assert route(**bad) == 1, bad
