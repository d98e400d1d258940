"""The packed-weight cache's file handling (dense_reader/cache.py), no GPU: whole-or-absent writes, the meta and
checksum checks, rebuild."""

import json

import numpy as np
import pytest

import __graft_entry__ as ge

ge.build_library()
from dense_reader import cache  # noqa: E402


def test_write_read_and_refusals(tmp_path):
    path = tmp_path / "w"
    meta = {"format": "bfloat8_b", "k": 64, "n": 32, "col_scale": False, "layout_version": 2}
    arrays = {"stream": np.arange(2176, dtype=np.uint8), "emax": np.arange(8, dtype=np.uint8), "scale": None}
    assert cache.read(path, meta) is None  # nothing there yet
    path.mkdir()
    assert cache.read(path, meta) is None  # an empty directory is no cache either
    cache.write(path, meta, arrays)
    assert sorted(p.name for p in path.iterdir()) == ["emax.npy", "meta.json", "stream.npy", "sums.json"]
    assert not path.with_name("w.tmp").exists()
    got = cache.read(path, meta)
    assert set(got) == {"stream", "emax"} and np.array_equal(got["stream"], arrays["stream"])
    # another call's meta: refused, the directory untouched; rebuild: treated as absent
    other = dict(meta, n=64)
    with pytest.raises(cache.PackCacheMismatch, match="n: cache 32, call 64"):
        cache.read(path, other)
    assert json.loads((path / "meta.json").read_text()) == meta
    assert cache.read(path, other, rebuild=True) is None
    # a flipped byte fails its checksum
    a = np.load(path / "stream.npy")
    a[5] ^= 1
    np.save(path / "stream.npy", a)
    with pytest.raises(cache.PackCacheMismatch, match="checksum"):
        cache.read(path, meta)
    # an unreadable meta
    (path / "meta.json").write_text("{")
    with pytest.raises(cache.PackCacheMismatch):
        cache.read(path, meta)


def test_layout_version_is_part_of_the_key(tmp_path):
    """A cache written by a library with another stream layout is refused: weight_meta carries tkd_layout_version
    (not the C-ABI version), so a change of the packed stream's bit layout invalidates every cache."""
    from common import ttnn_like as ttnn
    from dense_reader import _tkd

    meta = cache.weight_meta(ttnn.bfloat4_b, 64, 32, False)
    assert meta["layout_version"] == _tkd.lib().tkd_layout_version() >= 3
    path = tmp_path / "w"
    cache.write(path, dict(meta, layout_version=meta["layout_version"] - 1),
                {"stream": np.zeros(16, np.uint8), "emax": np.zeros(2, np.uint8), "scale": None})
    with pytest.raises(cache.PackCacheMismatch, match="layout_version"):
        cache.read(path, meta)
