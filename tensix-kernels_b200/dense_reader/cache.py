"""cache.py: packed weights on disk, so that a model's load does not quantise and pack again.

A packed weight is a directory: meta.json (what was packed: format, K, N, whether columns were scaled, the layout
version of the library that made the stream, and what the caller adds, e.g. a checksum of the source tensor), the
arrays stream.npy, emax.npy (block-float formats) and scale.npy (the per-column scales, bf16 bits), and sums.json with
the sha256 of each array's bytes. It is written whole or not at all (into PATH.tmp, then renamed) and read only if
meta.json equals what the call asks for and every array matches its checksum; anything else raises PackCacheMismatch
and leaves the directory alone, unless rebuild=True, which packs again over it. The pattern is the pack cache of the
reference's expert weights (moe/moe8.py:289-346), applied to dense_reader's weights.

    tw, ts = cache.native_weight_cached(device, w, ttnn.bfloat8_b, "cache/lm_head")      # packs once, then loads
"""

import hashlib
import json
import shutil
from pathlib import Path

import numpy as np
import torch

from common import ttnn_like as ttnn
from dense_reader import _tkd

ARRAYS = ("stream", "emax", "scale")
_NAMES = {ttnn.bfloat8_b: "bfloat8_b", ttnn.bfloat4_b: "bfloat4_b", ttnn.bfloat16: "bfloat16"}


class PackCacheMismatch(RuntimeError):
    """A cache directory that is not the pack the call asks for, or whose arrays fail their checksums."""


def _sha(a):
    h = hashlib.sha256()
    h.update(memoryview(np.ascontiguousarray(a)).cast("B"))
    return h.hexdigest()


def tensor_sum(t):
    """sha256 of a torch tensor's bytes (for meta's `source`: ties a cache to the weights it was packed from)."""
    return _sha(t.detach().contiguous().cpu().view(torch.uint8).numpy())


def write(path, meta, arrays, names=ARRAYS):
    """The cache directory, whole or absent. arrays: {name: numpy array or None} over `names`."""
    path = Path(path)
    tmp = path.with_name(path.name + ".tmp")
    shutil.rmtree(tmp, ignore_errors=True)
    tmp.mkdir(parents=True)
    sums = {}
    for name in names:
        a = arrays.get(name)
        if a is not None:
            np.save(tmp / f"{name}.npy", a)
            sums[name] = _sha(a)
    (tmp / "sums.json").write_text(json.dumps(sums, indent=1))
    (tmp / "meta.json").write_text(json.dumps(meta, indent=1, sort_keys=True))
    shutil.rmtree(path, ignore_errors=True)
    tmp.rename(path)


def read(path, meta, rebuild=False):
    """{name: array} of a cache written with the same meta; None when there is none (no directory, or an empty one) or
    with rebuild. A cache that differs from meta, cannot be read or fails a checksum raises PackCacheMismatch."""
    path = Path(path)
    if not path.exists() or (path.is_dir() and not any(path.iterdir())):
        return None
    if rebuild:
        return None
    try:
        old = json.loads((path / "meta.json").read_text())
        sums = json.loads((path / "sums.json").read_text())
    except (OSError, ValueError) as e:
        raise PackCacheMismatch(f"dense_reader pack cache {path}: its meta.json / sums.json cannot be read "
                                f"({type(e).__name__}); pass rebuild=True to pack over it") from e
    if old != meta:
        keys = sorted(set(old) | set(meta), key=str)
        why = "; ".join(f"{k}: cache {old.get(k)!r}, call {meta.get(k)!r}" for k in keys if old.get(k) != meta.get(k))
        raise PackCacheMismatch(f"dense_reader pack cache {path} does not match this call ({why}); it was neither taken "
                                "nor overwritten. Pass rebuild=True to pack again over it.")
    out = {}
    for name, want in sums.items():
        try:
            a = np.load(path / f"{name}.npy")
        except (OSError, ValueError) as e:
            raise PackCacheMismatch(f"dense_reader pack cache {path}: {name}.npy cannot be read ({type(e).__name__})") from e
        if _sha(a) != want:
            raise PackCacheMismatch(f"dense_reader pack cache {path}: {name}.npy does not match its checksum")
        out[name] = a
    return out


def weight_meta(dtype, k, n, col_scale, extra=None):
    """What a cache directory must say to be taken: the weight asked for and the library's stream layout version
    (tkd_layout_version: it changes with every change of the packed stream's bit layout, which the C-ABI version and
    the checksums would not notice)."""
    return {"format": _NAMES[dtype], "k": int(k), "n": int(n), "col_scale": bool(col_scale),
            "layout_version": int(_tkd.lib().tkd_layout_version()), **(extra or {})}


def save_weight(path, tw, ts=None, col_scale=False, extra=None):
    """A packed weight (native_weight's tw and, optionally, its scales ts) into the directory `path`."""
    assert not tw.wide, "dense_reader: a wide weight (held as a bf16 stream) is not cached"
    arrays = {"stream": tw.t.cpu().numpy(), "emax": tw.emax.cpu().numpy() if tw.emax is not None else None,
              "scale": ts.t.reshape(-1).view(torch.int16).cpu().numpy() if ts is not None else None}
    write(path, weight_meta(tw.dtype, tw.k, tw.n, col_scale, extra), arrays)


def load_weight(device, path, dtype, k, n, col_scale=False, extra=None, memory_config=None, rebuild=False):
    """(tw, ts or None) from the directory `path` if it holds this very pack; None when there is no cache."""
    got = read(path, weight_meta(dtype, k, n, col_scale, extra), rebuild=rebuild)
    if got is None:
        return None
    want = _tkd.lib().tkd_packed_bytes(ttnn.FMT[dtype], k, n)
    if got["stream"].nbytes != want:
        raise PackCacheMismatch(f"dense_reader pack cache {path}: the stream is {got['stream'].nbytes} bytes, this "
                                f"library packs [{k}, {n}] {_NAMES[dtype]} into {want}")
    stream = torch.from_numpy(got["stream"]).to(device.torch)
    emax = torch.from_numpy(got["emax"]).to(device.torch) if "emax" in got else None
    tw = ttnn.Weight(stream, emax, k, n, dtype, device, memory_config or ttnn.DRAM_MEMORY_CONFIG)
    ts = None
    if "scale" in got:
        s = torch.from_numpy(got["scale"]).view(torch.bfloat16).reshape(1, 1, 1, -1)
        ts = ttnn.from_torch(s, dtype=ttnn.bfloat16, layout=ttnn.TILE_LAYOUT, device=device,
                             memory_config=ttnn.DRAM_MEMORY_CONFIG)
    return tw, ts


def native_weight_cached(device, t, dtype, path, col_scale=False, sharded=True, max_banks=None, rebuild=False,
                         check_source=True):
    """linear.native_weight through a cache directory: loaded when `path` holds this pack (same format, shape, column
    scaling, library layout and, with check_source, the same source tensor by sha256), else packed and written."""
    from common.device import sharded_memcfg
    from dense_reader import linear

    n, k = t.shape
    extra = {"source": tensor_sum(t)} if check_source else None
    mc = sharded_memcfg(device, k, n, max_banks=max_banks) if sharded else ttnn.DRAM_MEMORY_CONFIG
    hit = load_weight(device, path, dtype, k, n, col_scale, extra, memory_config=mc, rebuild=rebuild)
    if hit is not None:
        return hit
    tw, ts = linear.native_weight(device, t, dtype, col_scale=col_scale, sharded=sharded, max_banks=max_banks)
    if not tw.wide:
        save_weight(path, tw, ts, col_scale, extra)
    return tw, ts
