"""w4a16.py: the int4-weight matmul with group scales along K (G = 32) for one token, on a B200.

Mirrors the reference's int4/w4a16.py entry points (int4_weight :69-86, group_scales :89-97, dequantized :100-102,
reference :105-107, w4a16_linear :170-252, dequantize :255-337, nibbles :59-66). The weight is q * s exactly: symmetric
codes q in -7..7 (sign-magnitude) and one bf16 scale per output column and 32 consecutive inputs.

Where the reference keeps nibbles in bfloat4_b-shaped tiles and the scales in a tensor of their own, multiplying
32 K tiles of partial products by a scale tile at a time, libtkd streams ONE packed weight (TKD_FMT_INT4,
include/tkd.h): bfloat4_b's super-atoms with the 32 scales of a super-atom (64 k x 16 columns) where bfloat4_b keeps
its exponents, 0.5625 bytes a weight like the reference's nibbles plus scales. The stream kernel multiplies a k32 block
of codes into a fresh accumulator and adds that, times the block's scale, to the running sum, so y = sum over groups of
s * (sum over the group of x * q), each inner sum exact products added in fp32, as in the reference's compute kernel
(kernels/w4a16_compute.cpp).

int4_weight returns a dict like the reference's ("t": the nibbles as a device tensor, "k", "n", ...); the scales arrive
with the call, as there, and the packed stream of (codes, scales) is made on the first call with a given scale tensor
and kept with the weight. The Tensix options (cores_per_bank, kb, kw, sbw, full_sync, split, budget, fidelity) are
accepted and steer nothing: split=False and the default give the same bits trivially.
"""

import torch

from common import device as dev
from common import ttnn_like as ttnn
from dense_reader import _tkd, linear

TILE = 32
G = 32  # inputs per scale
_OPTS = {"cores_per_bank", "kb", "kw", "sbw", "full_sync", "split", "budget"}


def nibbles(codes):
    """int codes [K, N] (-7..7) -> uint8 [K / 32, N / 32, 512]: per 32 x 32 tile its 1024 values face by face (rows 0-15
    x columns 0-15, rows 0-15 x columns 16-31, then rows 16-31 likewise), each sign << 3 | magnitude, two to a byte with
    the even element in the low nibble. (The reference's storage form, w4a16.py:59-66; kept here as the weight's
    host-visible tensor, the kernel reads its own packed stream.)"""
    k, n = codes.shape
    q = codes.to(torch.int16).reshape(k // 32, 2, 16, n // 32, 2, 16)  # [kt, face row, r, nt, face column, c]
    q = q.permute(0, 3, 1, 4, 2, 5).reshape(k // 32, n // 32, 1024)
    v = (q.abs() | ((q < 0).to(torch.int16) << 3)).to(torch.uint8)
    return v[..., 0::2] | (v[..., 1::2] << 4)


def int4_weight(device, codes, banks=None, max_banks=None):
    """codes [N_out, K] int8 in -7..7 -> the weight: a dict with "t" (the nibbles, uint8 [K / 32, N_pad / 32 * 512] on
    the device), "k", "n", "banks", "ns", "pitch" as the reference reports them (N padded to banks * 32 columns; banks:
    the device's HBM stacks or fewer with max_banks), and the canonical code bytes the packer takes."""
    assert int(codes.abs().max()) <= 7, "w4a16: codes are -7..7"
    q = codes.T.contiguous()
    k, n = q.shape
    assert k % TILE == 0, f"w4a16: K = {k} must be a multiple of 32"
    banks = banks or dev.dram_banks(device, max_banks)
    unit = TILE * banks
    npad = (n + unit - 1) // unit * unit
    qp = torch.zeros(k, npad, dtype=q.dtype)
    qp[:, :n] = q
    ns = npad // TILE // banks
    mc = ttnn.MemoryConfig(ttnn.TensorMemoryLayout.WIDTH_SHARDED, ttnn.BufferType.DRAM, ttnn.ShardSpec(banks, (k // 32, ns * 512)))
    t = ttnn.from_torch(nibbles(qp).reshape(k // 32, -1), dtype=ttnn.uint8, layout=ttnn.ROW_MAJOR_LAYOUT, device=device,
                        memory_config=mc)
    # canonical codes for tkd_pack: [K, padded N] bytes sign << 3 | magnitude
    npk = _tkd.lib().tkd_padded_cols(n)
    canon = torch.zeros(k, npk, dtype=torch.uint8)
    canon[:, :n] = (q.abs() | ((q < 0).to(q.dtype) << 3)).to(torch.uint8)
    return {"t": t, "k": k, "n": n, "banks": banks, "ns": ns, "pitch": ns * 512, "_codes": canon.to(device.torch),
            "_device": device, "_packed": {}}


def group_scales(device, scales):
    """scales [N_out, K / 32] -> [K / 32, N] bf16 on the device."""
    return ttnn.from_torch(scales.T.contiguous().to(torch.bfloat16), dtype=ttnn.bfloat16, layout=ttnn.TILE_LAYOUT,
                           device=device, memory_config=ttnn.DRAM_MEMORY_CONFIG)


def dequantized(codes, scales):
    """The float [N_out, K] weight q * s with s as the device holds it (bf16)."""
    s = scales.to(torch.bfloat16).float()
    return codes.float() * s.repeat_interleave(G, dim=1)


def reference(x, codes, scales):
    """x (as bf16) @ (q * s).T in float32."""
    return x.to(torch.bfloat16).float() @ dequantized(codes, scales).T


def packed(wq, scale):
    """The TKD_FMT_INT4 stream of (wq's codes, scale): made on the first call with this scale tensor, kept with wq."""
    key = (id(scale), scale.t.data_ptr())
    hit = wq["_packed"].get(key)
    if hit is not None:
        return hit[0]
    device, k, n = wq["_device"], wq["k"], wq["n"]
    L = _tkd.lib()
    npk = L.tkd_padded_cols(n)
    assert tuple(scale.shape[-2:]) == (k // G, n), (scale.shape, k // G, n)
    with torch.cuda.device(device.torch):
        sc = torch.zeros(k // G, npk, dtype=torch.bfloat16, device=device.torch)
        sc[:, :n] = scale.t.reshape(k // G, n)
        stream = torch.empty(L.tkd_packed_bytes(_tkd.FMT_INT4, k, n), dtype=torch.uint8, device=device.torch)
        _tkd.check(L.tkd_pack(_tkd.FMT_INT4, k, n, sc.data_ptr(), wq["_codes"].data_ptr(), stream.data_ptr(), None, None,
                              torch.cuda.current_stream().cuda_stream), "tkd_pack")
        torch.cuda.current_stream().synchronize()  # (sc is a temporary; the kernel reads weights ahead of stream order)
    w = ttnn.Weight(stream, None, k, n, ttnn.bfloat4_b, device, ttnn.DRAM_MEMORY_CONFIG, fmt=_tkd.FMT_INT4)
    wq["_packed"] = {key: (w, scale)}  # (one entry: the scale tensor is kept alive with it, so its id stays its own)
    return w


def w4a16_linear(x, wq, scale, *, memory_config=None, fidelity="hifi2", **opts):
    """y = x @ (q * s).T for one token: x [1, 1, 1, K] bf16, wq from int4_weight, scale from group_scales. Returns
    [1, 1, 1, N] bf16."""
    assert not set(opts) - _OPTS, f"w4a16: unknown options {sorted(set(opts) - _OPTS)}"
    assert x.shape[-2] == 1, f"w4a16: one token, got {x.shape[-2]} rows"
    assert x.dtype == ttnn.bfloat16 and x.layout == ttnn.TILE_LAYOUT
    assert x.shape[-1] == wq["k"], (x.shape, wq["k"])
    return linear.matmul(x, packed(wq, scale), None, memory_config=memory_config, fidelity=fidelity)


def dequantize(wq, scale, out=None, cores_per_bank=3):
    """The int4 weight times its group scales as a bfloat8_b weight [1, 1, K, N] for an ordinary block-float matmul
    over many rows. out: a weight of that shape to refill (returned, rewritten on every call)."""
    device, k, n = wq["_device"], wq["k"], wq["n"]
    vals = ttnn.held_values(packed(wq, scale))[:, :n]  # q * s, exact in float32, on the device
    w = ttnn.pack_weight(device, vals, ttnn.bfloat8_b, 1, memory_config=dev.sharded_memcfg(device, k, n, wq["banks"]))
    if out is None:
        return w
    assert out.shape == w.shape and out.dtype == w.dtype and out.fmt == w.fmt, "w4a16: out is not this weight's shape"
    out.t.copy_(w.t)
    out.emax.copy_(w.emax)
    torch.cuda.current_stream().synchronize()  # (weights are read ahead of stream order by later launches)
    return out
