"""moe8.py: a mixture-of-experts layer that reads only the chosen experts' weights, on a B200.

Mirrors the reference's moe/moe8.py entry points for the layer's two matmuls: bfp4_tiles :117-154, bfp4_values :157-169,
pack :507-527 (pack_host :435-465, pack_upload :468-499), reference :619-636, reference_rows :639-644, union :647-649, u_max :923-925, gate_up :710-817,
down :820-910, gate_up_rows :928-1037, down_rows :1040-1136. The expert ids are read on the device, as there: every op
is one kernel launch on the current stream and nothing goes to the host, so the ops can be captured in a CUDA graph.

- gate_up(x, P, ids, w, k) -> h [1, 1, 1, k * I]: per chosen expert e (slot s) h_s = w_s * act(x G_e) * (x U_e), act
  "silu", "gelu_tanh" or "swiglu_oai", an optional per-expert gate/up bias added before the activation;
- down(h, P, ids, k) -> y [1, 1, 1, H]: the sum over the slots of h_s @ D_e;
- gate_up_rows / down_rows: R <= 32 rows, each with its own k experts; the work goes by the distinct experts of all
  R x k ids in increasing order (the union), each read once for all rows; h [1, 1, 32, u_max * I] holds union index q's
  I columns at q * I, 0 where a row did not choose the expert.

The packed weights (pack): every expert's gate|up matrix [H, 2I], its 32-column tiles in the GLU's order (gate j, up
j), and its down matrix [I, H], each as one bfloat4_b stream of libtkd (csrc/tkd_layout.h), the experts back to back in
one buffer, so an id finds its expert by a multiplication. The values are rounded to the bfloat4_b grid exactly as
bfp4_tiles rounds them (values already on the grid stay as they are). The K-block layout (kblock=True: each 32 x 32
block held transposed, so the shared exponents run along K in blocks of 16, a GPTQ-along-K export's layout) is rounded
exactly as bfp4_tiles(kblock=True) rounds it, and its values are then held exactly as a bf16 stream, 2 bytes a weight
instead of 0.5625: the bfloat4_b stream shares an exponent among 16 columns of one k, which such values do not fit. The
Tensix options (cores_per_bank, banks, kw, fidelity, cpb, loaders) are accepted and steer nothing; banks and
cores_per_bank are still part of a pack cache's identity, as in the reference.

The pack cache (pack(cache=), prepack, pack_cached, repack_down, PackCacheMismatch; moe8.py:278-465, :530-600): a
directory with meta.json (what was packed), the arrays gu / gu_emax / dn / dn_emax (/ bias) and sums.json (their
sha256), written whole or not at all; taken only when its meta equals the call's, refused and left alone otherwise.
prepack needs the GPU (the packer is the GPU's); repack_down only renames the split, which orders nothing here.

- route(logits, ids, w, k): the router's top k and their weights (softmax or sigmoid scoring, a score bias,
  group-limited routing, a scaling factor, a fixed shared-expert slot) into the ids and weights the other ops read
  (route :1139-1253, route_reference :1256-1286, sigmoid_table :108-111), one warp a row, keys in float64.
"""

import ctypes
import hashlib
import json
import math
from pathlib import Path

import numpy as np
import torch

from common import ttnn_like as ttnn
from common.device import dram_banks
from dense_reader import _tkd
from dense_reader import cache as _cache

TILE = 32
TB = 576  # a bfloat4_b tile: 64 exponent bytes, then 1024 codes of a sign and 3 magnitude bits
ACTS = {"silu": 0, "gelu_tanh": 1, "swiglu_oai": 2}
OAI_ALPHA, OAI_LIMIT = 1.702, 7.0
# The reference's Tensix settings (moe8.py:66-91): module attributes callers may set; they steer nothing here (one work
# split, one loader), so every value gives the same bits.
ROWS_SFPU, GU_CPB, GU_ROWS_CPB, LOADERS, ROWS_LOADERS, SPLIT_SHARE = True, 0, 0, 2, 1, 0.5
PACK_VERSION = 1  # the cache's arrays below; a cache of another version (or of another stream layout) is refused
PackCacheMismatch = _cache.PackCacheMismatch
_CACHE_ARRAYS = ("gu", "gu_emax", "dn", "dn_emax", "bias")


# --- the bfloat4_b grid on the host -----------------------------------------------------------------------------------


def _faces(a):
    """[KT, NT, 32, 32] tile values -> [KT, NT, 64, 16]: the 64 face rows of a tile in storage order (faces (rows 0-15,
    columns 0-15), (0-15, 16-31), (16-31, 0-15), (16-31, 16-31), each row by row)."""
    kt, nt = a.shape[:2]
    return np.ascontiguousarray(a.reshape(kt, nt, 2, 16, 2, 16).transpose(0, 1, 2, 4, 3, 5)).reshape(kt, nt, 64, 16)


def bfp4_tiles(w, kblock=False):
    """float [K, N] (multiples of 32) -> uint8 [K / 32, N / 32, 576], each 32 x 32 tile as bfloat4_b (moe8.py:117-154 of
    the reference, which states it byte-identical to tt-metal's host conversion): the 16 values of a face row share the
    largest of their float32 exponent fields; a value's 24-bit significand is shifted down by its exponent's distance
    from that (dropping the bits shifted out; gone beyond 31), its top 3 bits kept and rounded to nearest, ties to even,
    on the 21 bits below, at most 7; a value whose own exponent field is 0 gives 0; the sign is kept for a non-zero
    result only. 64 exponent bytes, then two codes a byte, the earlier in the low nibble. kblock: the tile holds its
    block transposed (a face row is 16 consecutive K at one N)."""
    w = np.ascontiguousarray(w.detach().float().cpu().numpy() if isinstance(w, torch.Tensor) else w, dtype=np.float32)
    k, n = w.shape
    assert k % TILE == 0 and n % TILE == 0, w.shape
    tiles = w.reshape(k // TILE, TILE, n // TILE, TILE).transpose(0, 2, 1, 3)
    if kblock:
        tiles = tiles.swapaxes(-1, -2)
    u = _faces(tiles).view(np.uint32).astype(np.int64)
    field = (u >> 23) & 0xFF
    top = field.max(axis=-1, keepdims=True)
    gap = top - field
    sig = ((u & 0x7FFFFF) | 0x800000) >> np.minimum(gap, 31)
    sig[gap > 31] = 0
    keep, rest = sig >> 21, sig & 0x1FFFFF
    keep = keep + ((rest > 0x100000) | ((rest == 0x100000) & ((keep & 1) == 1)))
    mag = np.minimum(keep, 7)
    mag[field == 0] = 0
    code = (((u >> 31) & (mag != 0)) << 3 | mag).astype(np.uint8).reshape(k // TILE, n // TILE, 1024)
    out = np.empty((k // TILE, n // TILE, TB), np.uint8)
    out[..., :64] = top[..., 0]
    out[..., 64:] = code[..., 0::2] | (code[..., 1::2] << 4)
    return out


def bfp4_values(tiles, kblock=False):
    """uint8 [..., 576] bfloat4_b tiles -> float32 [..., 32, 32], the tiles' values row-major: (-1)^s * m * 2^(shared -
    129) (moe8.py:157-169). kblock: tiles of bfp4_tiles(kblock=True), turned back to [K, N] order."""
    tiles = np.asarray(tiles)
    lead = tiles.shape[:-1]
    shared = tiles[..., :64].astype(np.int32)
    body = tiles[..., 64:]
    code = np.stack((body & 0xF, body >> 4), axis=-1).reshape(*lead, 64, 16).astype(np.int32)
    val = np.where(code & 8, -1.0, 1.0) * (code & 7) * np.exp2((shared - 129).astype(np.float64))[..., None]
    val = val.astype(np.float32).reshape(*lead, 2, 2, 16, 16).swapaxes(-3, -2).reshape(*lead, TILE, TILE)
    return val.swapaxes(-1, -2) if kblock else val


# --- the packed layer -------------------------------------------------------------------------------------------------


def _glu_order(m, I):
    """[..., 2I] as [up | gate] -> the same columns in the GLU's tile order: gate tile j, then up tile j."""
    up, gate = m[..., :I], m[..., I:]
    lead = m.shape[:-1]
    pairs = torch.stack((gate.reshape(*lead, I // TILE, TILE), up.reshape(*lead, I // TILE, TILE)), dim=-2)
    return pairs.reshape(*lead, 2 * I)


def _pack_experts(device, mats, what):
    """[E, K, N] float -> (streams uint8 [E, bytes], emax uint8 [E, N_pad / 16]) on the device: tkd_quantise and tkd_pack
    of each expert into its slice."""
    L = _tkd.lib()
    E, k, n = mats.shape
    npad = L.tkd_padded_cols(n)
    nbytes = L.tkd_packed_bytes(_tkd.FMT_BFP4, k, n)
    assert nbytes % 16 == 0
    st = torch.cuda.current_stream().cuda_stream
    with torch.cuda.device(device.torch):
        streams = torch.empty(E, nbytes, dtype=torch.uint8, device=device.torch)
        emax = torch.empty(E, npad // 16, dtype=torch.uint8, device=device.torch)
        exps = torch.empty(k * (npad // 16), dtype=torch.uint8, device=device.torch)
        codes = torch.empty(k * npad, dtype=torch.uint8, device=device.torch)
        info = torch.zeros(1, dtype=torch.int32, device=device.torch)
        for e in range(E):
            src = mats[e].to(device.torch, torch.float32).contiguous()
            _tkd.check(L.tkd_quantise(_tkd.FMT_BFP4, src.data_ptr(), 1, k, n, None, exps.data_ptr(), codes.data_ptr(), st),
                       "tkd_quantise")
            _tkd.check(L.tkd_pack(_tkd.FMT_BFP4, k, n, exps.data_ptr(), codes.data_ptr(), streams[e].data_ptr(),
                                  emax[e].data_ptr(), info.data_ptr(), st), "tkd_pack")
        torch.cuda.current_stream().synchronize()  # (the ops read the weights ahead of nothing, but src is a temporary)
        if int(info.item()) & 1:
            raise ValueError(f"moe8: an expert's {what} weight has exponents inside a group of 16 columns more than 48"
                             " binades apart: the packed stream does not hold it")
    return streams, emax


def _pack_experts_kblock(device, mats, what):
    """[E, K, N] float -> streams uint8 [E, bytes] of the K-block layout's values: each expert's TRANSPOSE goes through
    the ordinary quantiser (the 16 values that share an exponent are then 16 consecutive k of one column, as in
    bfp4_tiles(kblock=True)), and the resulting numbers, each a bf16 value exactly, are packed as a bf16 stream."""
    L = _tkd.lib()
    E, k, n = mats.shape
    kp, npad = L.tkd_padded_cols(k), L.tkd_padded_cols(n)
    nbytes = L.tkd_packed_bytes(_tkd.FMT_BF16, k, n)
    st = torch.cuda.current_stream().cuda_stream
    with torch.cuda.device(device.torch):
        streams = torch.empty(E, nbytes, dtype=torch.uint8, device=device.torch)
        exps = torch.empty(n * (kp // 16), dtype=torch.uint8, device=device.torch)
        codes = torch.empty(n * kp, dtype=torch.uint8, device=device.torch)
        vt = torch.empty(n, kp, dtype=torch.int16, device=device.torch)
        vals = torch.zeros(k, npad, dtype=torch.int16, device=device.torch)
        info = torch.zeros(1, dtype=torch.int32, device=device.torch)
        for e in range(E):
            src = mats[e].to(device.torch, torch.float32).T.contiguous()  # [N, K]: a weight of N inputs and K columns
            _tkd.check(L.tkd_quantise(_tkd.FMT_BFP4, src.data_ptr(), 1, n, k, None, exps.data_ptr(), codes.data_ptr(), st),
                       "tkd_quantise")
            _tkd.check(L.tkd_dequantise_bf16(_tkd.FMT_BFP4, n, k, exps.data_ptr(), codes.data_ptr(), vt.data_ptr(), st),
                       "tkd_dequantise_bf16")
            vals[:, :n] = vt[:, :k].T
            _tkd.check(L.tkd_pack(_tkd.FMT_BF16, k, n, None, vals.data_ptr(), streams[e].data_ptr(), None, info.data_ptr(), st),
                       "tkd_pack")
        torch.cuda.current_stream().synchronize()
    return streams, None


def _clamp_cpb(device, banks, cores_per_bank):
    g = device.compute_with_storage_grid_size()
    return max(1, min(cores_per_bank, (g.x * g.y) // banks))


def _fingerprint(t):
    """A cheap identity of a weight tensor for the pack cache: shape, dtype and the sha256 of a strided sample of its
    values as float32 (one in 2039), so that a cache made from other weights is not taken."""
    t = torch.as_tensor(t)
    sample = t.reshape(-1)[::2039].detach().float().cpu().contiguous().numpy()
    return f"{list(t.shape)}/{t.dtype}/{hashlib.sha256(sample.tobytes()).hexdigest()[:40]}"


def _meta(gate_up, down, banks, cpb, gu_bias, kblock=False):
    E, H, I2 = gate_up.shape
    meta = {"version": PACK_VERSION, "layout_version": int(_tkd.lib().tkd_layout_version()), "banks": int(banks),
            "cpb": int(cpb), "E": int(E), "H": int(H), "I": int(I2 // 2), "gate_up": _fingerprint(gate_up),
            "down": _fingerprint(down)}
    if gu_bias is not None:
        meta["gu_bias"] = _fingerprint(gu_bias)
    if kblock:
        meta["kblock"] = True
    return meta


def _pack_arrays(device, gate_up, down, gu_bias, kblock=False):
    """The layer's device arrays: {gu, gu_emax, dn, dn_emax, bias}; the emax arrays are None for a K-block pack (a bf16
    stream), the bias None without one."""
    E, H, I2 = gate_up.shape
    I = I2 // 2
    one = _pack_experts_kblock if kblock else _pack_experts
    gu, gu_emax = one(device, _glu_order(gate_up.float(), I), "gate|up")
    dn, dn_emax = one(device, down.float(), "down")
    bias = None
    if gu_bias is not None:
        b = _glu_order(torch.as_tensor(gu_bias).to(torch.bfloat16), I)
        bias = torch.zeros(E, _tkd.lib().tkd_padded_cols(2 * I), dtype=torch.bfloat16, device=device.torch)
        bias[:, : 2 * I] = b.to(device.torch)
    return {"gu": gu, "gu_emax": gu_emax, "dn": dn, "dn_emax": dn_emax, "bias": bias}


def _to_host(arrays):
    return {n: (None if a is None else (a.view(torch.int16) if a.dtype == torch.bfloat16 else a).cpu().numpy())
            for n, a in arrays.items()}


def _to_device(device, host):
    out = {n: (None if host.get(n) is None else torch.from_numpy(np.ascontiguousarray(host[n])).to(device.torch))
           for n in ("gu", "gu_emax", "dn", "dn_emax")}
    b = host.get("bias")
    out["bias"] = None if b is None else torch.from_numpy(np.ascontiguousarray(b)).to(device.torch).view(torch.bfloat16)
    return out


def _layer(device, E, H, I, banks, cpb, arrays, kblock=False):
    """The dict the ops take."""
    L = _tkd.lib()
    fmt = _tkd.FMT_BF16 if kblock else _tkd.FMT_BFP4
    want = (E, L.tkd_packed_bytes(fmt, H, 2 * I)), (E, L.tkd_packed_bytes(fmt, I, H))
    if (tuple(arrays["gu"].shape), tuple(arrays["dn"].shape)) != want:
        raise PackCacheMismatch(f"moe8: the packed arrays are {tuple(arrays['gu'].shape)}, {tuple(arrays['dn'].shape)}; this"
                                f" library packs {E} experts of [{H}, {2 * I}] and [{I}, {H}] into {want}")
    u8 = lambda t: ttnn.Tensor(t, ttnn.uint8, ttnn.ROW_MAJOR_LAYOUT, device, ttnn.DRAM_MEMORY_CONFIG)  # noqa: E731
    return {
        "E": E, "H": H, "I": I, "banks": banks, "cpb": cpb,
        "gu": u8(arrays["gu"]), "gu_emax": arrays["gu_emax"], "dn": u8(arrays["dn"]), "dn_emax": arrays["dn_emax"],
        "gu_bias": arrays["bias"] is not None, "gu_bias_t": arrays["bias"], "kblock": bool(kblock), "fmt": fmt,
        "bytes": sum(arrays[n].numel() for n in ("gu", "gu_emax", "dn", "dn_emax") if arrays[n] is not None),
        "_device": device, "_ws": {},
    }


def _check_shapes(gate_up, down, gu_bias):
    gate_up, down = torch.as_tensor(gate_up), torch.as_tensor(down)
    E, H, I2 = gate_up.shape
    I = I2 // 2
    assert H % TILE == 0 and I % TILE == 0 and tuple(down.shape) == (E, I, H), (gate_up.shape, down.shape)
    if gu_bias is not None:
        assert tuple(gu_bias.shape) == (E, 2 * I), (tuple(gu_bias.shape), (E, 2 * I))
    return gate_up, down, E, H, I


def _cached_arrays(device, gate_up, down, banks, cpb, cache, gu_bias, rebuild, kblock=False):
    """(the layer's device arrays, whether they were packed now): from the cache when its meta matches; packed and
    written when there is none (or with rebuild); a cache that differs raises PackCacheMismatch and is left alone."""
    if cache is None:
        return _pack_arrays(device, gate_up, down, gu_bias, kblock), True
    meta = _meta(gate_up, down, banks, cpb, gu_bias, kblock)
    host = _cache.read(cache, meta, rebuild=rebuild)
    if host is not None:
        return _to_device(device, host), False
    arrays = _pack_arrays(device, gate_up, down, gu_bias, kblock)
    _cache.write(cache, meta, _to_host(arrays), names=_CACHE_ARRAYS)
    return arrays, True


def pack(device, gate_up, down, cores_per_bank=3, banks=None, cache=None, gu_bias=None, rebuild=False, kblock=False):
    """One MoE layer's experts as the packed weights the ops take (moe8.py:507-527). gate_up: [E, H, 2I] float with up
    in columns 0..I-1 and gate in I..2I-1 ([up | gate]); down: [E, I, H]; gu_bias: [E, 2I] as [up | gate], held in bf16.
    Returns the dict the ops take ("E", "H", "I", "gu", "dn", "gu_bias", "bytes", ...). cores_per_bank and banks are
    recorded only. cache: a directory for this layer's packed arrays: taken when its meta matches (the versions, the
    banks and cores, the shapes and a fingerprint of the weights), made when absent or empty; a cache that differs
    raises PackCacheMismatch and is left as it is, unless rebuild=True, which packs again over it. kblock: each 32 x 32
    block of the weights is rounded with its shared exponents along K (bfp4_tiles(kblock=True)); the values are held
    exactly, as a bf16 stream (2 bytes a weight)."""
    gate_up, down, E, H, I = _check_shapes(gate_up, down, gu_bias)
    banks = banks or dram_banks(device)
    cpb = _clamp_cpb(device, banks, cores_per_bank)
    arrays, _ = _cached_arrays(device, gate_up, down, banks, cpb, cache, gu_bias, rebuild, kblock)
    return _layer(device, E, H, I, banks, cpb, arrays, kblock)


def pack_host(gate_up, down, banks, cores_per_bank=3, cache=None, gu_bias=None, rebuild=False, kblock=False, device=None):
    """pack()'s arrays in host memory (moe8.py:435-465): a dict of numpy arrays and numbers that pack_upload puts on a
    device. Unlike the reference's it needs a GPU to make them (device, default device 0): the packer is the GPU's."""
    gate_up, down, E, H, I = _check_shapes(gate_up, down, gu_bias)
    arrays, _ = _cached_arrays(device or ttnn.open_device(0), gate_up, down, banks, cores_per_bank, cache, gu_bias, rebuild,
                               kblock)
    return {"version": PACK_VERSION, "E": E, "H": H, "I": I, "banks": banks, "cpb": cores_per_bank, "arrays": _to_host(arrays),
            "gu_bias": gu_bias is not None, "kblock": bool(kblock)}


def pack_upload(device, host):
    """pack_host's dict on the device: the dict the ops take (moe8.py:468-499)."""
    assert host["version"] == PACK_VERSION, (host["version"], PACK_VERSION)
    return _layer(device, host["E"], host["H"], host["I"], host["banks"], host["cpb"], _to_device(device, host["arrays"]),
                  host["kblock"])


def prepack(gate_up, down, cache, banks, cores_per_bank=3, gu_bias=None, rebuild=False, kblock=False, device=None):
    """pack()'s arrays into its cache (moe8.py:423-432): the cache pack(..., cache=) or pack_cached then takes. True when it
    was made, False when the cache already held these weights; a cache that differs raises PackCacheMismatch unless
    rebuild=True. Unlike the reference's it needs a GPU (device, default device 0): the packer is the GPU's."""
    gate_up, down, _, _, _ = _check_shapes(gate_up, down, gu_bias)
    device = device or ttnn.open_device(0)
    return _cached_arrays(device, gate_up, down, banks, cores_per_bank, cache, gu_bias, rebuild, kblock)[1]


def pack_cached(device, cache, cores_per_bank=3, banks=None, kblock=False, gu_bias=None, verify=True):
    """pack()'s result from a pack cache alone, without the weights (moe8.py:530-600). The call must match the cache's meta:
    the versions, the banks and cores per bank (clamped to the device as pack() does), and the bias: gu_bias None (the
    cache has none), True (it has one) or the [E, 2I] tensor itself (its fingerprint must equal the cache's). verify:
    every array's sha256 against sums.json. Anything that differs raises PackCacheMismatch, and nothing is changed."""
    path = Path(cache)
    try:
        meta = json.loads((path / "meta.json").read_text())
        sums = json.loads((path / "sums.json").read_text()) if verify else None
    except (OSError, ValueError) as e:
        raise PackCacheMismatch(f"moe8 pack cache {path}: no readable meta.json / sums.json ({type(e).__name__})") from e
    banks = banks or dram_banks(device)
    cpb = _clamp_cpb(device, banks, cores_per_bank)
    want = {"version": PACK_VERSION, "layout_version": int(_tkd.lib().tkd_layout_version()), "banks": banks, "cpb": cpb,
            "kblock": bool(kblock), "a bias": gu_bias is not None}
    have = {"version": meta.get("version"), "layout_version": meta.get("layout_version"), "banks": meta.get("banks"),
            "cpb": meta.get("cpb"), "kblock": bool(meta.get("kblock", False)), "a bias": "gu_bias" in meta}
    diff = [f"{k}: cache {have[k]}, call {want[k]}" for k in want if want[k] != have[k]]
    if gu_bias is not None and gu_bias is not True and "gu_bias" in meta and _fingerprint(gu_bias) != meta["gu_bias"]:
        diff.append("the bias's fingerprint")
    if diff:
        raise PackCacheMismatch(f"moe8 pack cache {path} does not match this call ({'; '.join(diff)}). It was not taken.")
    host = {}
    for n in _CACHE_ARRAYS:
        if (n == "bias" and "gu_bias" not in meta) or (n.endswith("_emax") and kblock):
            continue
        try:
            host[n] = np.load(path / f"{n}.npy")
        except (OSError, ValueError) as e:
            raise PackCacheMismatch(f"moe8 pack cache {path}: {n}.npy cannot be read ({type(e).__name__})") from e
        if verify and sums.get(n) != _cache._sha(host[n]):
            raise PackCacheMismatch(f"moe8 pack cache {path}: {n}.npy differs from sums.json. It was not taken.")
    return _layer(device, meta["E"], meta["H"], meta["I"], banks, cpb, _to_device(device, host), kblock)


def repack_down(cache, cores_per_bank=2):
    """A pack cache moved to another number of cores per bank, without the weights (moe8.py:379-420). There the split
    orders down's tiles; here the arrays do not depend on it, so only the cache's meta changes, and the result equals a
    fresh pack at cores_per_bank, its meta too. True when it was converted, False when the cache already has that split."""
    path = Path(cache) / "meta.json"
    meta = json.loads(path.read_text())
    assert meta["version"] == PACK_VERSION, (cache, meta["version"], PACK_VERSION)
    if meta["cpb"] == cores_per_bank:
        return False
    meta["cpb"] = int(cores_per_bank)
    tmp = path.with_name("meta.json.tmp")
    tmp.write_text(json.dumps(meta, indent=1, sort_keys=True))
    tmp.replace(path)
    return True


# --- references -------------------------------------------------------------------------------------------------------


def _glu(gt, u, act):
    """act(x G) * (x U) for the references (moe8.py:607-616)."""
    assert act in ACTS, f"moe8: act {act!r}"
    if act == "silu":
        return torch.nn.functional.silu(gt) * u
    if act == "gelu_tanh":
        return torch.nn.functional.gelu(gt, approximate="tanh") * u
    g = gt.clamp(max=OAI_LIMIT)
    return g * torch.sigmoid(OAI_ALPHA * g) * (u.clamp(-OAI_LIMIT, OAI_LIMIT) + 1)


def reference(x, gate_up, down, ids, w, act="silu", gu_bias=None):
    """(y [1, H], h [1, k * I]) in float64 for one row (moe8.py:619-636): h_s = w_s * act(x G_e + b) * (x U_e + b) for
    e = ids[s], y the sum of h_s @ D_e; gate_up [E, H, 2I] as [up | gate], gu_bias [E, 2I] likewise, rounded to bf16."""
    x = x.double().reshape(1, -1)
    I = gate_up.shape[-1] // 2
    hs = []
    y = torch.zeros(1, gate_up.shape[1], dtype=torch.float64)
    for s, e in enumerate(ids):
        both = x @ gate_up[e].double()
        if gu_bias is not None:
            both = both + torch.as_tensor(gu_bias[e]).to(torch.bfloat16).double()
        hs.append(_glu(both[:, I:], both[:, :I], act) * float(w[s]))
        y += hs[-1] @ down[e].double()
    return y, torch.cat(hs, dim=1)


def reference_rows(x, gate_up, down, ids, w, act="silu", gu_bias=None):
    """y [R, H] in float64, each row with its own experts (moe8.py:639-644)."""
    return torch.cat([reference(x[r : r + 1], gate_up, down, ids[r], w[r], act, gu_bias)[0] for r in range(len(ids))])


def union(ids, E):
    """The distinct ids below E, increasing: the order the rows ops work in (moe8.py:647-649)."""
    return sorted({int(e) for e in torch.as_tensor(ids).reshape(-1).tolist() if 0 <= int(e) < E})


def u_max(P, rows, k):
    """The most distinct experts rows x k ids can name: h's width is u_max * I (moe8.py:923-925)."""
    return min(P["E"], rows * k)


# --- the ops ----------------------------------------------------------------------------------------------------------


def _ids_args(ids, w, rows, k, ids32):
    want = ttnn.uint32 if ids32 else ttnn.uint16
    assert ids.dtype == want, f"moe8: ids are {ids.dtype}, ids32={ids32} wants {want}"
    assert ids.shape[-1] >= k and ids.shape[-2] >= rows, (ids.shape, rows, k)
    if w is not None:
        assert w.dtype == ttnn.bfloat16 and w.shape[-1] >= k and w.shape[-2] >= rows, (w.dtype, w.shape)


def _fill(a, P, what, x, ids, w, rows, k, ids32, by_union, slots, out):
    H, I = P["H"], P["I"]
    gu = what == "gu"
    em = P["gu_emax"] if gu else P["dn_emax"]
    a.w, a.emax, a.fmt = (P["gu"] if gu else P["dn"]).t.data_ptr(), (None if em is None else em.data_ptr()), P["fmt"]
    a.expert_bytes = (P["gu"] if gu else P["dn"]).t.shape[1]
    a.experts, a.k_in, a.n = P["E"], (H if gu else I), (2 * I if gu else H)
    a.rows, a.x, a.ldx = rows, x.t.data_ptr(), x.t.stride(-2)
    a.ids, a.ids32, a.k, a.ld_ids = ids.t.data_ptr(), int(ids32), k, ids.t.stride(-2)
    if w is not None:
        a.route_w, a.ld_w = w.t.data_ptr(), w.t.stride(-2)
    a.by_union, a.slots = int(by_union), slots
    a.out, a.ldo = out.data_ptr(), out.stride(-2)


def _gate_up(x, P, ids, w, k, rows, ids32, by_union, act, memory_config):
    assert act in ACTS, f"moe8: act {act!r}"
    assert 1 <= k <= 16, k
    device = x.device()
    H, I = P["H"], P["I"]
    assert x.dtype == ttnn.bfloat16 and x.shape[-1] == H and x.shape[-2] >= rows, (x.dtype, x.shape)
    _ids_args(ids, w, rows, k, ids32)
    slots = u_max(P, rows, k) if by_union else k
    with torch.cuda.device(device.torch):
        if by_union:
            out = torch.zeros(1, 1, TILE, slots * I, dtype=torch.bfloat16, device=device.torch)
        else:
            out = torch.empty(1, 1, 1, slots * I, dtype=torch.bfloat16, device=device.torch)
        a = _tkd.TkdMoe()
        _fill(a, P, "gu", x, ids, w, rows, k, ids32, by_union, slots, out)
        a.act = ACTS[act]
        a.bias = P["gu_bias_t"].data_ptr() if P["gu_bias"] else None
        _tkd.check(_tkd.lib().tkd_moe_gate_up(ctypes.byref(a), torch.cuda.current_stream().cuda_stream), "tkd_moe_gate_up")
    return ttnn.Tensor(out, ttnn.bfloat16, ttnn.TILE_LAYOUT, device, memory_config or ttnn.DRAM_MEMORY_CONFIG)


def _down(h, P, ids, k, rows, ids32, by_union, memory_config):
    assert 1 <= k <= 16, k
    device = h.device()
    H, I = P["H"], P["I"]
    slots = u_max(P, rows, k) if by_union else k
    assert h.dtype == ttnn.bfloat16 and h.shape[-1] >= slots * I and h.shape[-2] >= rows, (h.dtype, h.shape)
    _ids_args(ids, None, rows, k, ids32)
    L = _tkd.lib()
    with torch.cuda.device(device.torch):
        if by_union:
            out = torch.zeros(1, 1, TILE, H, dtype=torch.bfloat16, device=device.torch)
        else:
            out = torch.empty(1, 1, 1, H, dtype=torch.bfloat16, device=device.torch)
        a = _tkd.TkdMoe()
        _fill(a, P, "dn", h, ids, None, rows, k, ids32, by_union, slots, out)
        need = ctypes.c_uint64(0)
        _tkd.check(L.tkd_moe_workspace(ctypes.byref(a), ctypes.byref(need)), "tkd_moe_workspace")
        ws = P["_ws"].get("dn")
        if ws is None or ws.numel() < need.value:
            # (zeroed once: the kernel returns its counters to zero; calls on one layer run in stream order)
            ws = P["_ws"]["dn"] = torch.zeros(need.value, dtype=torch.uint8, device=device.torch)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        _tkd.check(L.tkd_moe_down(ctypes.byref(a), torch.cuda.current_stream().cuda_stream), "tkd_moe_down")
    return ttnn.Tensor(out, ttnn.bfloat16, ttnn.TILE_LAYOUT, device, memory_config or ttnn.DRAM_MEMORY_CONFIG)


def gate_up(x, P, ids, w, k, *, ids32=False, kw=8, fidelity="hifi2", memory_config=None, cpb=None, loaders=None, act="silu"):
    """h [1, 1, 1, k * I] bf16: per slot s the routing weight w[s] times act(x G) * (x U) of expert ids[s] (moe8.py:710-817).
    x [1, 1, 1, H] bf16; ids [1, 1, 1, k] uint16 (uint32 with ids32) and w [1, 1, 1, k] bf16, read on the device. A
    pack with a bias adds it before the activation. act: "silu", "gelu_tanh" or "swiglu_oai"."""
    return _gate_up(x, P, ids, w, k, 1, ids32, False, act, memory_config)


def down(h, P, ids, k, *, ids32=False, kw=8, fidelity="hifi2", memory_config=None, loaders=None):
    """y [1, 1, 1, H] bf16 = h @ the chosen experts' down rows, slot s's I rows expert ids[s]'s (moe8.py:820-910). h is
    gate_up's. The slots' sums are added in slot order, each an fp32 sum over its expert's I rows."""
    return _down(h, P, ids, k, 1, ids32, False, memory_config)


def gate_up_rows(x, P, ids, w, k, rows, *, ids32=False, kw=8, fidelity="hifi2", memory_config=None, cpb=None, act="silu",
                 loaders=None):
    """h [1, 1, 32, u_max * I] bf16 for x's first `rows` rows (moe8.py:928-1037): union index q's I columns hold row r's
    routing weight for expert union(ids)[q] times act(x_r G) * (x_r U), 0 where row r did not choose it, 0 past the
    union and in rows past `rows`. ids [1, 1, rows, k], w [1, 1, rows, k]; a row's ids are distinct."""
    assert 1 <= rows <= TILE, rows
    assert P["E"] <= 1024, "moe8 rows: at most 1024 experts"
    return _gate_up(x, P, ids, w, k, rows, ids32, True, act, memory_config)


def down_rows(h, P, ids, k, rows, *, ids32=False, kw=8, fidelity="hifi2", memory_config=None, loaders=None):
    """y [1, 1, 32, H] bf16: row r = the sum over the union of the R x k ids of h's row r (union index q's I columns)
    times expert union(ids)[q]'s down rows (moe8.py:1040-1136); rows past `rows` are 0. h is gate_up_rows' for the same
    ids, rows and k."""
    assert 1 <= rows <= TILE, rows
    assert P["E"] <= 1024, "moe8 rows: at most 1024 experts"
    return _down(h, P, ids, k, rows, ids32, True, memory_config)


# --- the router -------------------------------------------------------------------------------------------------------


def sigmoid_table():
    """sigmoid(i / 16 - 16) for i = 0 .. 512 in Q2.30, rounded: the bounds table of the reference's route kernel
    (moe8.py:108-111, kernels/moe_sigmoid_q30.h). The kernel here computes in float64 and needs no table; kept for callers
    that check it."""
    return [round((1 << 30) / (1.0 + math.exp(16 - i / 16))) for i in range(513)]


def route(logits, ids, w, k, *, kind="softmax", bias=None, ids32=False, experts=None, shared=None, scale=1.0, norm=True,
          groups=None, slot=None):
    """The router's top k and their weights into ids and w, in place of ttnn.topk and the weights' ops (moe8.py:1139-1253).
    logits [1, 1, R, W] float32, R <= 32; experts: the first E columns (default all; a multiple of 32); ids [1, 1, R, k]
    uint16 (uint32 with ids32), w [1, 1, R, k] bf16. Slots in decreasing order of the pick's key, the lower id among equal
    keys. kind "softmax": the top k by logit, weights the softmax over the k. kind "sigmoid": the top k by sigmoid(logit)
    + bias (bias [1, 1, 1, E] float32; None: by logit), weights the picks' sigmoids over their sum (norm=False: each its
    own sigmoid). shared: a [1, 1, R, 1] bf16 that gets sigmoid(logits[:, E]). scale: every weight times it (0 < scale <
    4). groups=(n_group, topk_group): the sigmoid kind with a bias; a group's score the sum of its two largest keys, the
    topk_group best groups kept. slot: that id as slot k of every row at weight 1.0 (ids and w hold k + 1). Returns w."""
    assert kind in ("softmax", "sigmoid"), f"moe8.route: kind {kind!r}"
    R, W = logits.shape[-2], logits.shape[-1]
    E = experts or W
    assert E <= W and (shared is None or E + 1 <= W), (E, W)
    assert logits.dtype == ttnn.float32, logits.dtype
    assert R <= 32 and E % TILE == 0 and 1 <= k <= 16, (R, E, k)
    assert 0 < scale < 4, scale
    assert norm or kind == "sigmoid", "moe8.route: norm=False is for the sigmoid kind"
    assert slot is None or (k + 1 <= 16 and 0 <= int(slot) < (1 << 32 if ids32 else 1 << 16)), (k, slot)
    ng, tg = (1, 1) if groups is None else (int(groups[0]), int(groups[1]))
    if groups is not None:
        assert kind == "sigmoid" and bias is not None, "moe8.route: groups need the sigmoid kind with a bias"
        assert ng <= 32 and E % ng == 0 and E // ng >= 2 and 1 <= tg <= ng and tg * (E // ng) >= k, (E, groups, k)
    assert ids.dtype == (ttnn.uint32 if ids32 else ttnn.uint16), ids.dtype
    assert w.dtype == ttnn.bfloat16, w.dtype
    kk = k + (slot is not None)
    assert ids.shape[-1] >= kk and w.shape[-1] >= kk and ids.shape[-2] >= R and w.shape[-2] >= R, (ids.shape, w.shape)
    sig = kind == "sigmoid" and bias is not None
    if sig:
        assert bias.dtype == ttnn.float32 and bias.shape[-1] == E, (bias.dtype, bias.shape)
    if shared is not None:
        assert shared.dtype == ttnn.bfloat16 and shared.shape[-2] >= R, (shared.dtype, shared.shape)
    kcode = 0 if kind == "softmax" else (1 if sig else 2)
    device = logits.device()
    with torch.cuda.device(device.torch):
        _tkd.check(
            _tkd.lib().tkd_moe_route(
                logits.t.data_ptr(), logits.t.stride(-2), R, E, k, kcode, bias.t.data_ptr() if sig else None, float(scale),
                int(bool(norm)), ng, tg, int(slot is not None), int(slot or 0), ids.t.data_ptr(), int(ids32), ids.t.stride(-2),
                w.t.data_ptr(), w.t.stride(-2), shared.t.data_ptr() if shared is not None else None,
                shared.t.stride(-2) if shared is not None else 0, torch.cuda.current_stream().cuda_stream),
            "tkd_moe_route")
    return w


def route_reference(logits, k, kind="softmax", bias=None, scale=1.0, norm=True, groups=None, slot=None):
    """route's result on the host in float64 (moe8.py:1256-1286): (ids [R, k] long, w [R, k] float64) for float32 logits
    [R, E]. The lower id first among equal keys; groups as route's; slot: an extra column of that id at weight 1."""
    x = logits.float().double()
    sg = torch.sigmoid(x)
    key = x if kind == "softmax" or bias is None else sg + bias.float().double().reshape(1, -1)
    if kind != "softmax" and groups is not None:
        ng, tg = groups
        R, E = key.shape
        score = key.reshape(R, ng, E // ng).topk(2, dim=-1).values.sum(-1)
        best = torch.argsort(-score, dim=-1, stable=True)[:, :tg]
        keep = torch.zeros(R, ng, dtype=torch.bool).scatter_(1, best, True).repeat_interleave(E // ng, dim=1)
        key = key.masked_fill(~keep, float("-inf"))
    picks = torch.argsort(-key, dim=-1, stable=True)[:, :k]
    if kind == "softmax":
        wt = torch.softmax(x.gather(1, picks), dim=-1)
    else:
        wt = sg.gather(1, picks)
        if norm:
            wt = wt / wt.sum(-1, keepdim=True)
    wt = wt * scale
    if slot is not None:
        picks = torch.cat([picks, torch.full_like(picks[:, :1], int(slot))], dim=1)
        wt = torch.cat([wt, torch.ones_like(wt[:, :1])], dim=1)
    return picks, wt
