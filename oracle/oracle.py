"""oracle.py: Python face of the CPU oracle. TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the
benchmark's CPU-baseline leg, never by the product package.

Two independent restatements of the reference's block-float quantiser live here so that they can be checked against
each other and against the golden vectors: the C one (oracle.c, through ctypes) and a vectorised numpy one (this
file). The numpy quantiser follows moe/moe8.py:117-154 of XylolabsInc/tensix-kernels, generalised from 3 mantissa bits
(bfloat4_b, pinned) to 7 (bfloat8_b, PARITY UNPINNED: the reference has no vector for it; its quantiser is inside the
third-party wheel ttnn==0.81.1).
"""

import ctypes
import subprocess
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
MB = {"bfp8": 7, "bfp4": 3}
_LIB = None


def build():
    """Compile oracle.c into liboracle.so beside it (gcc)."""
    subprocess.run(["make", "-s", "-C", str(HERE), "liboracle.so"], check=True)


def lib():
    global _LIB
    if _LIB is None:
        so = HERE / "liboracle.so"
        if not so.exists() or so.stat().st_mtime < (HERE / "oracle.c").stat().st_mtime:
            build()
        L = ctypes.CDLL(str(so))
        L.orc_bf16_ceil.restype = ctypes.c_float
        L.orc_bf16_ceil.argtypes = [ctypes.c_float]
        L.orc_bf16_rne.restype = ctypes.c_uint16
        L.orc_bf16_rne.argtypes = [ctypes.c_float]
        L.orc_key.restype = ctypes.c_uint32
        L.orc_key.argtypes = [ctypes.c_uint16]
        L.orc_key_value.restype = ctypes.c_float
        L.orc_key_value.argtypes = [ctypes.c_uint32]
        _LIB = L
    return _LIB


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _i64(v):
    return ctypes.c_int64(int(v))


# --- quantiser --------------------------------------------------------------------------------------------------------


def quantise_c(w, fmt):
    """w float32 [K, N] -> (exps uint8 [K, N/16], codes uint8 [K, N]) by oracle.c."""
    w = np.ascontiguousarray(w, np.float32)
    k, n = w.shape
    assert n % 16 == 0
    exps = np.zeros((k, n // 16), np.uint8)
    codes = np.zeros((k, n), np.uint8)
    lib().orc_quantise(_p(w), _i64(k), _i64(n), MB[fmt], _p(exps), _p(codes))
    return exps, codes


def quantise_np(w, fmt):
    """The same in numpy (moe8.py:134-150 with mantissa bits mb)."""
    mb = MB[fmt]
    w = np.ascontiguousarray(w, np.float32)
    k, n = w.shape
    bits = w.view(np.uint32).reshape(k, n // 16, 16)
    exp = (bits >> 23) & 0xFF
    sign = bits >> 31
    man = ((bits & 0x7FFFFF) | (1 << 23)).astype(np.int64)
    shared = exp.max(axis=-1, keepdims=True)
    diff = (shared - exp).astype(np.int64)
    m = np.where(diff > 31, 0, man >> np.minimum(diff, 31))
    shift = 24 - mb
    rnd = m & ((1 << shift) - 1)
    m = m >> shift
    guard = m & 1
    tie = 1 << (shift - 1)
    m = m + ((rnd > tie) | ((rnd == tie) & (guard == 1)))
    m = np.minimum(m, (1 << mb) - 1)
    m = np.where(exp == 0, 0, m)
    s = np.where(m == 0, 0, sign)
    codes = ((s << mb) | m).astype(np.uint8).reshape(k, n)
    return shared.reshape(k, n // 16).astype(np.uint8), codes


def dequantise(exps, codes, fmt):
    """(exps, codes) -> float32 [K, N] (moe8.py:157-169: unit exponent 126 + mantissa bits)."""
    mb = MB[fmt]
    mag = (codes & ((1 << mb) - 1)).astype(np.float32)
    sgn = np.where((codes >> mb) & 1, np.float32(-1), np.float32(1))
    e = np.repeat(exps.astype(np.int32), 16, axis=1) - (126 + mb)
    return (sgn * np.ldexp(mag, e)).astype(np.float32)


def dequantise_c(exps, codes, fmt):
    """The same by oracle.c (orc_dequantise): for matrices too large for numpy temporaries."""
    k, n = codes.shape
    out = np.empty((k, n), np.float32)
    lib().orc_dequantise(_p(np.ascontiguousarray(exps)), _p(np.ascontiguousarray(codes)), _i64(k), _i64(n), MB[fmt], _p(out))
    return out


def tiles(exps, codes, fmt):
    """The reference's tile bytes [K/32, N/32, 576 | 1088] (moe8.py:125-154)."""
    mb = MB[fmt]
    k, n = codes.shape
    tb = 64 + (512 if mb == 3 else 1024)
    out = np.zeros((k // 32, n // 32, tb), np.uint8)
    lib().orc_tiles(_p(np.ascontiguousarray(exps)), _p(np.ascontiguousarray(codes)), _i64(k), _i64(n), mb, _p(out))
    return out


def block_float(t, fmt):
    """float [K, N] rounded to fmt's grid, float32: what a weight of that dtype holds (linear.py:159-163). bf16: RNE."""
    if fmt == "bf16":
        return torch.as_tensor(t).float().to(torch.bfloat16).float().numpy()
    e, c = quantise_np(np.asarray(t, np.float32), fmt)
    return dequantise(e, c, fmt)


def native_values(t, fmt, col_scale=False):
    """What linear.native_weight makes of a float [out, in] matrix (linear.py:144-156): (held values float32 [K, N],
    scales float32 [N]). Matrices of more than 2^24 elements go through oracle.c's quantiser and dequantiser (the numpy
    restatement would need several temporaries of the matrix's size); the two are checked against each other and the
    golden vectors in tests/test_oracle.py."""
    t = torch.as_tensor(t).float()
    c = bf16_ceil(t.abs().amax(dim=1).clamp(min=1e-8)) if col_scale else torch.ones(t.shape[0])
    wt = ((t / c[:, None]) if col_scale else t).T.contiguous()
    if fmt != "bf16" and wt.numel() > 1 << 24:
        n = wt.shape[1]
        assert n % 16 == 0, n
        return dequantise_c(*quantise_c(wt.numpy(), fmt), fmt), c.numpy()
    return block_float(wt.numpy(), fmt), c.numpy()


def bf16_ceil(s):
    """linear.py:110-114."""
    b = s.to(torch.bfloat16).float()
    up = (b.view(torch.int32) + 0x10000).view(torch.float32)
    return torch.where(b >= s, b, up)


def interleave_glu(gate, up):
    """linear.py:122-130."""
    o, i = gate.shape
    return torch.stack([gate.reshape(o // 32, 32, i), up.reshape(o // 32, 32, i)], dim=1).reshape(2 * o, i)


# --- matmul and output stages -----------------------------------------------------------------------------------------


def reference(x, w, scale=None):
    """linear.py:166-169, the reference's torch path: bf16(x) @ w (* scale) in float32."""
    y = x.to(torch.bfloat16).float() @ torch.as_tensor(w).float()
    return y * torch.as_tensor(scale).float()[None, :] if scale is not None else y


def ref64(x, wk, scale=None):
    """test_dense_reader.py:56-58: the same in float64, returned as float32."""
    y = x.to(torch.bfloat16).double() @ torch.as_tensor(wk).double()
    return (y * torch.as_tensor(scale).double()[None, :] if scale is not None else y).float()


def matmul_f64(x, w):
    """oracle.c's own loop: x torch [M, K] (rounded to bf16), w float32 [K, N] -> float64 numpy [M, N]."""
    xb = x.to(torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16)
    w = np.ascontiguousarray(w, np.float32)
    m, k = xb.shape
    y = np.zeros((m, w.shape[1]), np.float64)
    lib().orc_matmul_f64(_p(np.ascontiguousarray(xb)), _i64(m), _i64(k), _p(w), _i64(w.shape[1]), _p(y))
    return y


def epilogue(acc, mode, acc2=None, act=0, scale=None, scale2=None, res=None, res32=None):
    """oracle.c's output stages on float64 sums acc [M, N]; mode: 0 plain/scale, 1 GLU interleaved, 2 GLU two sums,
    3 residual (res: torch bf16 [M, N]), 4 fp32 (+ res32). Returns float64."""
    acc = np.ascontiguousarray(acc, np.float64)
    m, n = acc.shape
    out = np.zeros((m, n // 2 if mode == 1 else n), np.float64)
    f = lambda a: None if a is None else np.ascontiguousarray(a, np.float32)  # noqa: E731
    sc, sc2, r32 = f(scale), f(scale2), f(res32)
    a2 = None if acc2 is None else np.ascontiguousarray(acc2, np.float64)
    rb = None if res is None else np.ascontiguousarray(res.to(torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16))
    q = lambda a: None if a is None else _p(a)  # noqa: E731
    lib().orc_epilogue(_p(acc), q(a2), _i64(m), _i64(n), mode, act, q(sc), q(sc2), q(rb), q(r32), _p(out))
    return out


# --- top-k records ----------------------------------------------------------------------------------------------------


def bf16_bits(t):
    return t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16)


def keys_of(bits):
    """dense_writer.cpp:215 on uint16 bf16 bits."""
    b = bits.astype(np.uint32)
    return (b ^ (0x8000 | (0x7FFF & (0 - (b >> 15))))) & 0xFFFF


def topk_canonical(y_row_bits, n, k, base):
    """oracle.c's canonical top-k (key descending, index ascending) of one row: (keys uint32 [k], idx uint32 [k])."""
    y = np.ascontiguousarray(y_row_bits, np.uint16)
    keys, idx = np.zeros(k, np.uint32), np.zeros(k, np.uint32)
    lib().orc_topk_canonical(_p(y), _i64(n), k, ctypes.c_uint32(base), _p(keys), _p(idx))
    return keys, idx


def topk_scan_ref(y_row_bits, c0, c1, n, k, base):
    """The reference writer's running top-k over columns [c0, c1) (dense_writer.cpp:185-232)."""
    y = np.ascontiguousarray(y_row_bits, np.uint16)
    keys, idx = np.zeros(k, np.uint32), np.zeros(k, np.uint32)
    lib().orc_topk_scan_ref(_p(y), _i64(c0), _i64(c1), _i64(n), k, ctypes.c_uint32(base), _p(keys), _p(idx))
    return keys, idx


def topk_merge_ref(words, rows, k, top):
    """The best `top` of every row among the records in `words` (uint32 [records, 2, rows, k]): key descending, index
    ascending among equal keys, empty slots (key 0) never chosen; one record of rows x top, empty beyond the candidates
    (key 0, index 0xFFFFFFFF). The definite-order form of the `vh.topk(top)` of lm_head_topk/lmhead.py:212-239."""
    words = np.asarray(words, np.uint32).reshape(-1, 2, rows, k)
    out = np.zeros((2, rows, top), np.uint32)
    out[1] = 0xFFFFFFFF
    for r in range(rows):
        keys, idx = words[:, 0, r].reshape(-1).astype(np.int64), words[:, 1, r].reshape(-1).astype(np.int64)
        live = keys != 0
        keys, idx = keys[live], idx[live]
        order = np.lexsort((idx, -keys))[:top]
        out[0, r, : order.size], out[1, r, : order.size] = keys[order], idx[order]
    return out


def records_host(t, rows, k):
    """Decode a records tensor as linear.py:753-768 does: (values float32 [rows, records * k], indices int64 [rows,
    records * k]); an empty slot (key 0) gives -inf and -1. Written over numpy words here."""
    words = t.contiguous().view(torch.int32).numpy().view(np.uint32).reshape(-1, 2, rows, k)
    keys = np.transpose(words[:, 0], (1, 0, 2)).reshape(rows, -1)
    idx = np.transpose(words[:, 1], (1, 0, 2)).reshape(rows, -1).astype(np.int64)
    raw = np.where(keys >= 0x8000, keys & 0x7FFF, ~keys & 0xFFFF).astype(np.uint32) << 16
    vals = raw.view(np.float32).copy()
    vals[keys == 0] = -np.inf
    idx[(keys == 0) | (idx == 0xFFFFFFFF)] = -1
    return torch.from_numpy(vals), torch.from_numpy(idx)


# ---- the int4 weight with group scales (int4/w4a16.py of the reference): codes q in -7..7, one bf16 scale per output
# column and 32 consecutive inputs, the weight being q * s exactly. PARITY PINNED for the host forms (nibbles,
# dequantized, reference: golden vectors made by running the reference's own functions, tests/golden/int4.npz).

def int4_nibbles(codes):
    """int codes [K, N] numpy (-7..7) -> uint8 [K / 32, N / 32, 512] (w4a16.py:59-66): per 32 x 32 tile its four 16 x 16
    faces in the order (rows 0-15, cols 0-15), (0-15, 16-31), (16-31, 0-15), (16-31, 16-31), each row-major, a value as
    sign << 3 | magnitude, element 2 i in the low nibble of byte i."""
    q = np.asarray(codes, dtype=np.int16)
    k, n = q.shape
    out = np.zeros((k // 32, n // 32, 512), np.uint8)
    for kt in range(k // 32):
        for nt in range(n // 32):
            tile = q[32 * kt : 32 * kt + 32, 32 * nt : 32 * nt + 32]
            faces = [tile[:16, :16], tile[:16, 16:], tile[16:, :16], tile[16:, 16:]]
            flat = np.concatenate([f.reshape(-1) for f in faces])
            v = (np.abs(flat) | ((flat < 0).astype(np.int16) << 3)).astype(np.uint8)
            out[kt, nt] = v[0::2] | (v[1::2] << 4)
    return out


def int4_dequantized(codes, scales):
    """float32 [N_out, K]: q * s with s rounded to bf16 (w4a16.py:100-102). codes [N_out, K] int, scales [N_out, K / 32]."""
    s = torch.as_tensor(scales).to(torch.bfloat16).float().numpy()
    return np.asarray(codes, dtype=np.float32) * np.repeat(s, 32, axis=1)


def int4_reference(x, codes, scales):
    """x (rounded to bf16) @ (q * s).T, accumulated in float64 (w4a16.py:105-107 states it in float32; the tests' bars
    are relative, test_int4.py:8-12). x torch [M, K]."""
    xb = torch.as_tensor(x).to(torch.bfloat16).double().numpy()
    return xb @ int4_dequantized(codes, scales).astype(np.float64).T


# ---- the ternary weight with group scales and its block Hadamard (ternary_matmul/t2.py of the reference). PARITY PINNED
# for the host forms (tiles, rotate, dequantize, reference: tests/golden/ternary.npz, made by running the reference).

T2_FORMATS = {"bfp2": (320, 127, 2), "bfp2c": (320, 127, 2), "bfp4": (576, 129, 4)}


def t2_tiles(q, fmt="bfp2"):
    """trits [K, N] numpy -> uint8 [K / 32, N / 32, tile bytes] (t2.py:81-99): 64 exponent bytes (127 for the 2-bit
    codes, 129 for the 4-bit ones), then the 1024 codes face by face; 2-bit code = sign << 1 | magnitude, four to a
    byte from the low bits up; 4-bit code = sign << 3 | magnitude, two to a byte."""
    tb, exp, bits = T2_FORMATS[fmt]
    q = np.asarray(q, dtype=np.int16)
    k, n = q.shape
    out = np.zeros((k // 32, n // 32, tb), np.uint8)
    out[..., :64] = exp
    for kt in range(k // 32):
        for nt in range(n // 32):
            tile = q[32 * kt : 32 * kt + 32, 32 * nt : 32 * nt + 32]
            flat = np.concatenate([f.reshape(-1) for f in (tile[:16, :16], tile[:16, 16:], tile[16:, :16], tile[16:, 16:])])
            neg, mag = (flat < 0).astype(np.uint8), (flat != 0).astype(np.uint8)
            if bits == 2:
                c = (neg << 1) | mag
                out[kt, nt, 64:] = c[0::4] | (c[1::4] << 2) | (c[2::4] << 4) | (c[3::4] << 6)
            else:
                c = (neg << 3) | mag
                out[kt, nt, 64:] = c[0::2] | (c[1::2] << 4)
    return out


def t2_rotate(x, signs, block=1024):
    """x' = H_block (signs * x) / sqrt(block) per block of the last dimension, float64 (t2.py:213-217), by butterflies
    (the Sylvester matrix's own recursion) instead of the matrix product."""
    v = (np.asarray(x, dtype=np.float64) * np.asarray(signs, dtype=np.float64)).reshape(-1, block).copy()
    h = 1
    while h < block:
        w = v.reshape(-1, block // (2 * h), 2, h)
        a, b = w[:, :, 0, :].copy(), w[:, :, 1, :].copy()
        w[:, :, 0, :], w[:, :, 1, :] = a + b, a - b
        h *= 2
    return (v / np.sqrt(block)).reshape(np.asarray(x).shape)


def t2_dequantize(trits, scales, g):
    """float32 [N_out, K]: q * s, s as given (t2.py:343-345)."""
    return np.asarray(trits, dtype=np.float32) * np.repeat(torch.as_tensor(scales).float().numpy(), g, axis=1)


def t2_reference(x, trits, scales, g):
    """x (as bf16) @ (q * bf16(s)).T, accumulated in float64 (t2.py:348-350 states it in float32)."""
    xb = torch.as_tensor(x).to(torch.bfloat16).double().numpy()
    return xb @ t2_dequantize(trits, torch.as_tensor(scales).to(torch.bfloat16), g).astype(np.float64).T


# ---- the mixture-of-experts layer (moe/moe8.py of the reference). PARITY PINNED for these host forms
# (tests/golden/moe.npz, made by running the reference's reference / reference_rows / union).


def moe_glu(gt, u, act):
    """act(x G) * (x U) in float64 (moe8.py:607-616): silu; gelu_tanh, 0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3)));
    swiglu_oai, min(g, 7) * sigmoid(1.702 min(g, 7)) * (clamp(u, -7, 7) + 1)."""
    gt, u = np.asarray(gt, np.float64), np.asarray(u, np.float64)
    if act == "silu":
        return gt / (1.0 + np.exp(-gt)) * u
    if act == "gelu_tanh":
        return 0.5 * gt * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (gt + 0.044715 * gt**3))) * u
    assert act == "swiglu_oai", act
    g = np.minimum(gt, 7.0)
    return g / (1.0 + np.exp(-1.702 * g)) * (np.clip(u, -7.0, 7.0) + 1.0)


def moe_reference(x, gate_up, down, ids, w, act="silu", gu_bias=None):
    """(y [1, H], h [1, k * I]) in float64 for one row (moe8.py:619-636): slot s of expert e = ids[s] gives h_s = w_s *
    act(x G_e + b) * (x U_e + b), y = sum of h_s @ D_e. gate_up [E, H, 2I] as [up | gate]; gu_bias [E, 2I] likewise,
    rounded to bf16 first. numpy arrays (x, w already the bf16 values)."""
    x = np.asarray(x, np.float64).reshape(1, -1)
    gate_up, down = np.asarray(gate_up, np.float64), np.asarray(down, np.float64)
    I = gate_up.shape[-1] // 2
    y = np.zeros((1, gate_up.shape[1]))
    hs = []
    for s, e in enumerate(ids):
        both = x @ gate_up[e]
        if gu_bias is not None:
            both = both + torch.as_tensor(np.asarray(gu_bias[e])).to(torch.bfloat16).double().numpy()
        hs.append(moe_glu(both[:, I:], both[:, :I], act) * float(w[s]))
        y += hs[-1] @ down[e]
    return y, np.concatenate(hs, axis=1)


def moe_union(ids, E):
    """The distinct ids below E in increasing order (moe8.py:647-649; kernels/moe8_rows.h builds the same on the device)."""
    return sorted({int(e) for e in np.asarray(ids).reshape(-1).tolist() if 0 <= int(e) < E})


def moe_reference_rows(x, gate_up, down, ids, w, E, act="silu", gu_bias=None):
    """(y [R, H], h [R, U * I]) in float64 for R rows with their own experts (moe8.py:639-644 and gate_up_rows' layout,
    :928-934): union index q's I columns of h hold row r's h for expert union[q], 0 where the row did not choose it."""
    ids = np.asarray(ids)
    un = moe_union(ids, E)
    I = np.asarray(gate_up).shape[-1] // 2
    ys, h = [], np.zeros((len(ids), len(un) * I))
    for r in range(len(ids)):
        y, hr = moe_reference(np.asarray(x)[r : r + 1], gate_up, down, ids[r].tolist(), np.asarray(w)[r], act, gu_bias)
        ys.append(y)
        for s, e in enumerate(ids[r].tolist()):
            h[r, un.index(e) * I : (un.index(e) + 1) * I] = hr[0, s * I : (s + 1) * I]
    return np.concatenate(ys), h


def moe_route_reference(logits, k, kind="softmax", bias=None, scale=1.0, norm=True, groups=None, slot=None):
    """The router's picks and weights in float64 (moe8.py:1256-1286): logits float32 [R, E] numpy -> (ids [R, k] int64, w
    [R, k] float64). softmax: the top k by logit, the softmax over the k. sigmoid: the top k by sigmoid + bias (without a
    bias by logit), the picks' sigmoids over their sum (norm False: as they are). The lower id first among equal keys.
    groups (n_group, topk_group): a group's score the sum of its two largest keys, the topk_group best kept (the lower
    group first among equal scores), the others out. Weights times scale; slot: an extra column, that id at weight 1."""
    x = np.asarray(logits, np.float32).astype(np.float64)
    R, E = x.shape
    sg = 1.0 / (1.0 + np.exp(-x))
    key = x.copy() if kind == "softmax" or bias is None else sg + np.asarray(bias, np.float32).astype(np.float64).reshape(1, -1)
    if kind != "softmax" and groups is not None:
        ng, tg = groups
        per = E // ng
        for r in range(R):
            score = np.sort(key[r].reshape(ng, per), axis=-1)[:, -2:].sum(-1)
            best = np.argsort(-score, kind="stable")[:tg]
            out = np.ones(ng, bool)
            out[best] = False
            key[r, np.repeat(out, per)] = -np.inf
    ids = np.stack([np.argsort(-key[r], kind="stable")[:k] for r in range(R)])
    if kind == "softmax":
        v = np.take_along_axis(x, ids, 1)
        v = np.exp(v - v.max(-1, keepdims=True))
        w = v / v.sum(-1, keepdims=True)
    else:
        w = np.take_along_axis(sg, ids, 1)
        if norm:
            w = w / w.sum(-1, keepdims=True)
    w = w * scale
    if slot is not None:
        ids = np.concatenate([ids, np.full((R, 1), int(slot))], 1)
        w = np.concatenate([w, np.ones((R, 1))], 1)
    return ids, w
