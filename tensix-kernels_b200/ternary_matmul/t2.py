"""t2.py: the ternary-weight matmul with group scales along K (trits -1, 0, +1, one scale per output channel and G
inputs), on a B200: one token (t2_linear), many rows (t2m_linear), linear() choosing by rows, and the block Hadamard
rotation some ternary checkpoints need in front (hadamard, rotate_rows, or fused into t2_linear with hadamard=).

Mirrors the reference's ternary_matmul/t2.py entry points (tiles :81-99, ternary_weight :117-166, group_scales :169-179,
hadamard_signs :185-202, sylvester :205-210, rotate :213-217, rotate_rows :220-259, hadamard :262-340, dequantize
:343-345, reference :348-350, t2_linear :409-495, t2m_linear :649-682, linear :757-800) with the same names, arguments
and results.

What is different underneath. A trit is an int4 code with magnitude 0 or 1, so the one-token kernel is libtkd's int4
stream kernel (TKD_FMT_INT4, include/tkd.h; int4/w4a16.py): the packed stream holds the codes and, per 32 inputs, the
scale of their group (a group of G = 32 * j inputs repeats its scale j times, which changes no sum). The reference's
three storage forms ("bfp2", "bfp2c", "bfp4": tiles() makes each, ternary_weight keeps it as the weight's visible
tensor) therefore run the same stream and give the same bits; the stream is 4.5 bits a weight like the reference's
"bfp4" form. The kernel is bound by instruction issue per weight, not by bytes (profiles/), so a 2-bit stream would
save HBM space, not time. Many rows run the ordinary stream kernels on the weight's values q * s held as bf16 (exact:
a trit times a bf16 scale), as the reference's multi-row kernel dequantizes each tile by its scale row. The Hadamard
is one small kernel (tkd_hadamard: a fast Walsh-Hadamard transform in fp32) for one row or many; with hadamard=
t2_linear has the stream kernel do the same transform on its own copy of x (the same additions in the same order, so
the fused form and the op give the same bits). The Tensix options (cores_per_bank, sbw, kw,
split, budget, fidelity) are accepted and steer nothing. The weight is exactly q * bf16(s); the kernel's error is its
arithmetic alone.
"""

import torch

from common import device as dev
from common import ttnn_like as ttnn
from dense_reader import _tkd
from dense_reader import linear as dense_linear

TILE = 32
# tile bytes, the exponent that reads a code's magnitude m as m, bits per value, tile bytes in DRAM
FORMATS = {"bfp2": (320, 127, 2, 320), "bfp2c": (320, 127, 2, 256), "bfp4": (576, 129, 4, 576)}
HADAMARD = 1024  # the rotation's block
HADAMARD_SCALE = 1 / 32  # the device's transform is 32 times the orthonormal one
MT_MAX = 4  # (the reference's row-slice height in tiles; here a call takes any number of rows)

_SIGNS = {}  # sign mask's address -> its host signs


def tiles(q, fmt="bfp2"):
    """trits q [K, N] (-1, 0, 1) -> uint8 [K / 32, N / 32, tile bytes]: per 32 x 32 tile 64 exponent bytes (the value
    that reads a code's magnitude as itself), then the codes face by face (rows 0-15 x cols 0-15, rows 0-15 x cols
    16-31, rows 16-31 likewise; row-major inside a face): 2 bits a value (sign << 1 | magnitude, four to a byte, the
    first in the low bits) or 4 (sign << 3 | magnitude, two to a byte)."""
    tb, exp, bits, _ = FORMATS[fmt]
    k, n = q.shape
    assert k % TILE == 0 and n % TILE == 0, q.shape
    assert q.abs().max() <= 1, "t2: the weight's values must be -1, 0 or +1"
    v = q.to(torch.int16).reshape(k // 32, 2, 16, n // 32, 2, 16).permute(0, 3, 1, 4, 2, 5).reshape(k // 32, n // 32, 1024)
    neg, mag = (v < 0).to(torch.uint8), (v != 0).to(torch.uint8)
    if bits == 2:
        c = (neg << 1) | mag
        body = c[..., 0::4] | (c[..., 1::4] << 2) | (c[..., 2::4] << 4) | (c[..., 3::4] << 6)
    else:
        c = (neg << 3) | mag
        body = c[..., 0::2] | (c[..., 1::2] << 4)
    out = torch.cat([torch.full((k // 32, n // 32, 64), exp, dtype=torch.uint8), body], dim=-1)
    assert out.shape[-1] == tb
    return out


def ternary_weight(device, trits, *, fmt="bfp2", cores_per_bank=3, sbw=None, banks=None, max_banks=None):
    """trits [N_out, K] (-1, 0, 1) as the weight: a dict with the device tensor "t" (the storage form's tile bytes as
    they lie in DRAM, uint8 [K / 32, N / 32 * bytes]), "k", "n", "fmt", "tb", "db", "banks", "bytes", and the code
    bytes libtkd's packer takes."""
    tb, db = FORMATS[fmt][0], FORMATS[fmt][3]
    q = trits.T.contiguous()
    k, n = q.shape
    assert k % TILE == 0, f"t2: K = {k} must be a multiple of 32"
    assert int(q.abs().max()) <= 1, "t2: the weight's values must be -1, 0 or +1"
    banks = banks or dev.dram_banks(device, max_banks)
    npad = (n + TILE - 1) // TILE * TILE
    qp = torch.zeros(k, npad, dtype=q.dtype)
    qp[:, :n] = q
    body = tiles(qp, fmt)[..., tb - db :]  # ("bfp2c": the codes alone)
    t = ttnn.from_torch(body.reshape(k // 32, -1).contiguous(), dtype=ttnn.uint8, layout=ttnn.ROW_MAJOR_LAYOUT,
                        device=device, memory_config=ttnn.DRAM_MEMORY_CONFIG)
    npk = _tkd.lib().tkd_padded_cols(n)
    canon = torch.zeros(k, npk, dtype=torch.uint8)
    canon[:, :n] = ((q < 0).to(torch.uint8) << 3) | (q != 0).to(torch.uint8)
    return {"t": t, "k": k, "n": n, "fmt": fmt, "tb": tb, "db": db, "banks": banks, "NT": npad // TILE,
            "bytes": (k // 32) * (npad // 32) * db, "_codes": canon.to(device.torch), "_device": device, "_packed": {}}


def group_scales(device, scales, factor=1.0):
    """scales [N_out, K / G] (any float dtype) times factor (a power of two: HADAMARD_SCALE with the Hadamard) as
    [K / G, N] bf16 on the device; the weight is q * bf16(s * factor)."""
    return ttnn.from_torch((scales.float().T * factor).contiguous().to(torch.bfloat16), dtype=ttnn.bfloat16,
                           layout=ttnn.TILE_LAYOUT, device=device, memory_config=ttnn.DRAM_MEMORY_CONFIG)


def hadamard_signs(device, signs):
    """The +-1 signs [K] of the block Hadamard as sign masks on the device: uint8 [1, K / 32 * 64], a 32-bit word per two
    inputs with bit 15 set when the first is negated and bit 31 for the second (an XOR flips a bf16 pair's signs)."""
    k = signs.numel()
    assert k % HADAMARD == 0, f"t2: the Hadamard needs K a multiple of {HADAMARD}, got {k}"
    neg = (signs.reshape(k // 2, 2) < 0).to(torch.int64)
    words = (neg[:, 0] << 15) | (neg[:, 1] << 31)
    b = torch.stack([(words >> s) & 255 for s in (0, 8, 16, 24)], dim=-1).to(torch.uint8)
    mask = ttnn.from_torch(b.reshape(1, k // TILE * 64).contiguous(), dtype=ttnn.uint8, layout=ttnn.ROW_MAJOR_LAYOUT,
                           device=device, memory_config=ttnn.DRAM_MEMORY_CONFIG)
    _SIGNS[mask.buffer_address()] = signs.float().clone()
    return mask


def sylvester(n):
    """The +-1 Sylvester Hadamard matrix of order n (a power of two), float64."""
    h = torch.ones(1, 1, dtype=torch.float64)
    while h.shape[0] < n:
        h = torch.cat([torch.cat([h, h], dim=1), torch.cat([h, -h], dim=1)], dim=0)
    return h


def rotate(x, signs, block=HADAMARD):
    """x' = H_block (signs * x) / sqrt(block) per block of the last dimension, in float64 (the reference)."""
    v = (x.double() * signs.double()).reshape(*x.shape[:-1], -1, block)
    return (v @ sylvester(block).T / block**0.5).reshape(x.shape)


def _rotated(x, mask, memory_config):
    device = x.device()
    m, k = x.shape[-2], x.shape[-1]
    assert x.dtype == ttnn.bfloat16 and k % HADAMARD == 0 and mask.t.numel() == k // TILE * 64, (x.shape, mask.shape)
    y = ttnn.allocate_tensor_on_device([1, 1, m, k], ttnn.bfloat16, ttnn.TILE_LAYOUT, device, memory_config)
    xt = x.t.reshape(m, k)
    with torch.cuda.device(device.torch):
        _tkd.check(_tkd.lib().tkd_hadamard(xt.data_ptr(), xt.stride(0), mask.t.data_ptr(), m, k, y.t.data_ptr(), k,
                                           torch.cuda.current_stream().cuda_stream), "tkd_hadamard")
    return y


def rotate_rows(x, hadamard):
    """x' = 32 H_1024 (s * x) per block for many rows: x [1, 1, M, K] bf16; hadamard: the width's sign mask
    (hadamard_signs). Unnormalized, as the one-token form's (the scales carry the 1 / 32)."""
    return _rotated(x, hadamard, ttnn.DRAM_MEMORY_CONFIG)


def hadamard(x, mask, memory_config=None):
    """x' = 32 H_1024 (s * x) per block for one token, as its own op: x [1, 1, 1, K] bf16; returns x' [1, 1, 1, K] bf16,
    which t2_linear takes without hadamard=. One transform serves every projection of that input."""
    assert x.shape[-2] == 1 and x.shape[-1] % HADAMARD == 0, x.shape
    return _rotated(x, mask, memory_config or ttnn.L1_MEMORY_CONFIG)


def dequantize(trits, scales, g):
    """The float [N_out, K] weight q * s (s as given; s.to(torch.bfloat16) for the kernel's)."""
    return trits.float() * scales.float().repeat_interleave(g, dim=1)


def reference(x, trits, scales, g):
    """x @ (q * s).T in float32, x and s as the device holds them (bf16)."""
    return x.to(torch.bfloat16).float() @ dequantize(trits, scales.to(torch.bfloat16), g).T


def packed(w, scale, g):
    """The TKD_FMT_INT4 stream of (w's trits, scale): made on the first call with this scale tensor, kept with w."""
    key = (id(scale), scale.t.data_ptr(), g)
    hit = w["_packed"].get(key)
    if hit is not None:
        return hit[0]
    device, k, n = w["_device"], w["k"], w["n"]
    assert g % 32 == 0 and k % g == 0, f"t2: G = {g} must be a multiple of 32 that divides K = {k}"
    assert tuple(scale.shape[-2:]) == (k // g, n), (scale.shape, k // g, n)
    L = _tkd.lib()
    npk = L.tkd_padded_cols(n)
    with torch.cuda.device(device.torch):
        sc = torch.zeros(k // 32, npk, dtype=torch.bfloat16, device=device.torch)
        sc[:, :n] = scale.t.reshape(k // g, n).repeat_interleave(g // 32, dim=0)
        stream = torch.empty(L.tkd_packed_bytes(_tkd.FMT_INT4, k, n), dtype=torch.uint8, device=device.torch)
        _tkd.check(L.tkd_pack(_tkd.FMT_INT4, k, n, sc.data_ptr(), w["_codes"].data_ptr(), stream.data_ptr(), None, None,
                              torch.cuda.current_stream().cuda_stream), "tkd_pack")
        torch.cuda.current_stream().synchronize()  # (sc is a temporary; the kernel reads weights ahead of stream order)
    pw = ttnn.Weight(stream, None, k, n, ttnn.bfloat4_b, device, ttnn.DRAM_MEMORY_CONFIG, fmt=_tkd.FMT_INT4)
    w["_packed"] = {key: (pw, scale)}
    w.pop("_rows", None)
    return pw


def _rows_weight(w, scale, g):
    """The weight's values q * s as a bf16 stream (exact), for the kernels that take many rows."""
    pw = packed(w, scale, g)
    hit = w.get("_rows")
    if hit is None or hit[0] is not pw:
        vals = ttnn.held_values(pw)[:, : w["n"]]  # (on the device)
        hit = w["_rows"] = (pw, ttnn.pack_weight(w["_device"], vals, ttnn.bfloat16, 1))
    return hit[1]


def t2_linear(x, w, scale, g=128, *, hadamard=None, memory_config=None, fidelity="hifi2", kw=None, split=True, topk=None,
              out=None, col0=0, gap=None):
    """y = x @ (q * s).T for one token: x [1, 1, 1, K] bf16, w from ternary_weight, scale from group_scales (G inputs
    per scale); with hadamard (hadamard_signs) x is rotated first. Returns [1, 1, 1, N] bf16. topk (the dense reader's
    contract, one row): {"r", "k", "slot0", "base", "n", "write_y"}: the records of the row's best k per unit of output
    columns go to r. out: write into this [1, 1, 1, W] bf16 tensor instead, output column tile c at tile c + col0, and
    with gap = (split, shift) tiles c >= split at c + col0 + shift (the output's columns in two runs). Returns out."""
    assert x.shape[-2] == 1, f"t2: one token, got {x.shape[-2]} rows"
    assert x.dtype == ttnn.bfloat16 and x.layout == ttnn.TILE_LAYOUT
    assert x.shape[-1] == w["k"], (x.shape, w["k"])
    pw = packed(w, scale, g)
    spec = None if topk is None else {**topk, "rows": 1}
    if out is None or gap is None:
        if hadamard is not None:
            # the rotation inside the stream kernel's own copy of x (the same arithmetic as the op's, hence the same bits);
            # a K whose row does not fit in shared memory beside the ring takes the op first
            try:
                return dense_linear.matmul(x, pw, None, memory_config=memory_config, fidelity=fidelity, topk=spec, out=out,
                                           col0=col0, hadamard=hadamard)
            except _tkd.TkdError as e:
                if e.code != _tkd.ERR_UNSUPPORTED:
                    raise
            x = _rotated(x, hadamard, ttnn.L1_MEMORY_CONFIG)
        return dense_linear.matmul(x, pw, None, memory_config=memory_config, fidelity=fidelity, topk=spec, out=out, col0=col0)
    xr = _rotated(x, hadamard, ttnn.L1_MEMORY_CONFIG) if hadamard is not None else x
    # the output's columns in two runs: the plain row, then its two runs copied to their places
    assert topk is None, "t2: gap takes no top-k"
    cut, shift = gap
    y = dense_linear.matmul(xr, pw, None, fidelity=fidelity)
    n, a = w["n"], cut * TILE
    dst = out.t.reshape(-1, out.shape[-1])
    src = y.t.reshape(-1, n)
    dst[:1, col0 * TILE : col0 * TILE + min(a, n)] = src[:1, : min(a, n)]
    if n > a:
        dst[:1, (col0 + shift) * TILE + a : (col0 + shift) * TILE + n] = src[:1, a:]
    return out


def t2m_linear(x, w, scale, g=128, *, memory_config=None, fidelity="hifi2", kw=None, split=True):
    """y = x @ (q * s).T for many rows: x [1, 1, M, K] bf16, already in the weights' basis (rotate_rows for a rotated
    checkpoint). Returns [1, 1, M, N] bf16."""
    assert x.dtype == ttnn.bfloat16 and x.layout == ttnn.TILE_LAYOUT
    assert x.shape[-1] == w["k"], (x.shape, w["k"])
    return dense_linear.matmul(x, _rows_weight(w, scale, g), None, memory_config=memory_config, fidelity=fidelity)


def linear(x, w, scale=None, g=None, memory_config=None, activation=None, rows_kernel=True, **opts):
    """t2_linear / t2m_linear for x of any rank with [..., rows, K] (bf16), w from ternary_weight (a dict may also carry
    "scale", "g" and "had", used unless given), activation "silu" or None, the input's rank back. One row runs the
    one-token kernel. More rows run rotate_rows (with hadamard=) and the multi-row path; rows_kernel=False instead runs
    the one-token kernel per row. With out= (and col0=, gap=) one row is written into out, which is returned."""
    scale = w["scale"] if scale is None else scale
    g = w.get("g", 128) if g is None else g
    opts.setdefault("hadamard", w.get("had"))
    shape = list(x.shape)
    rows, kd = shape[-2], shape[-1]
    if opts.get("out") is not None:
        assert rows == 1 and len(shape) == 4, f"t2.linear: out takes one row of a 4-D x, {shape}"
        assert activation is None, "t2.linear: out takes no activation"
    x4 = x if len(shape) == 4 else ttnn.reshape(x, [1, 1, rows, kd])
    if rows == 1:
        y = t2_linear(x4, w, scale, g, memory_config=memory_config, **opts)
    elif rows_kernel:
        xr = rotate_rows(x4, opts["hadamard"]) if opts.get("hadamard") is not None else x4
        mopts = {k_: v for k_, v in opts.items() if k_ in ("fidelity", "kw", "split")}
        y = t2m_linear(xr, w, scale, g, memory_config=memory_config, **mopts)
    else:
        device = x4.device()
        y = ttnn.allocate_tensor_on_device([1, 1, rows, w["n"]], ttnn.bfloat16, ttnn.TILE_LAYOUT, device, memory_config)
        for r in range(rows):
            xr = ttnn.Tensor(x4.t[:, :, r : r + 1, :].contiguous(), ttnn.bfloat16, ttnn.TILE_LAYOUT, device, None)
            y.t[:, :, r : r + 1, :] = t2_linear(xr, w, scale, g, **opts).t
    if activation is not None:
        assert activation == "silu", f"t2.linear: activation {activation!r}"
        y = ttnn.silu(y)
    if len(shape) != 4 and opts.get("out") is None:
        y = ttnn.reshape(y, [*shape[:-1], w["n"]])
    return y
