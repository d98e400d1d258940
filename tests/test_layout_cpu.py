"""The packed stream's index arithmetic (csrc/tkd_layout.h) and the streaming warp's register decode, walked on the
host (tests/layout_emul.cpp) against the oracle: no GPU needed."""

import ctypes
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle as orc

HERE = Path(__file__).resolve().parent
FMT = {"bfp8": 0, "bfp4": 1, "bf16": 2, "int4": 3}
KSA = {"bfp8": 32, "bfp4": 64, "bf16": 32, "int4": 64}
SAB = {"bfp8": 544, "bfp4": 576, "bf16": 1024, "int4": 576}


@pytest.fixture(scope="module")
def emul(tmp_path_factory):
    so = tmp_path_factory.mktemp("emul") / "liblayout_emul.so"
    subprocess.run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-o", str(so), str(HERE / "layout_emul.cpp")], check=True)
    return ctypes.CDLL(str(so))


def p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def canon(w, fmt):
    if fmt == "bf16":
        bits = torch.from_numpy(w).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
        return np.zeros((w.shape[0], w.shape[1] // 16), np.uint8), np.ascontiguousarray(bits)
    return orc.quantise_c(w, fmt)


def pack(emul, fmt, exps, codes):
    k, n = codes.shape
    nbytes = (n // 16) * (-(-k // KSA[fmt])) * SAB[fmt]
    stream = np.zeros(nbytes, np.uint8)
    emax = np.zeros(n // 16, np.uint8)
    wide = ctypes.c_int(0)
    emul.emul_pack(FMT[fmt], ctypes.c_int64(k), ctypes.c_int64(n), p(exps), p(codes), p(emax), p(stream), ctypes.byref(wide))
    return stream, emax, wide.value


@pytest.mark.parametrize("fmt", ["bfp8", "bfp4", "bf16"])
@pytest.mark.parametrize("k,n", [(64, 128), (96, 128), (288, 256), (544, 128)])
def test_stream_round_trip_and_decode(emul, fmt, k, n):
    g = torch.Generator().manual_seed(k + n)
    w = (torch.randn(k, n, generator=g) * 0.02 * torch.exp2(torch.randint(-3, 4, (k, 1), generator=g).float())).numpy()
    w[1, :16] = 0  # a row of a group with no non-zero code
    exps, codes = canon(w, fmt)
    held = orc.block_float(w, fmt)
    stream, emax, wide = pack(emul, fmt, exps, codes)
    assert wide == 0
    back = np.zeros((k, n), np.float32)
    emul.emul_unpack(FMT[fmt], ctypes.c_int64(k), ctypes.c_int64(n), p(stream), p(emax), p(back))
    assert np.array_equal(back.view(np.uint32), held.view(np.uint32))
    for m in (1, 5):
        x = torch.randn(m, k, generator=g).to(torch.bfloat16)
        y = np.zeros((m, n), np.float64)
        xb = np.ascontiguousarray(x.view(torch.int16).numpy().view(np.uint16))
        emul.emul_matmul(FMT[fmt], ctypes.c_int64(k), ctypes.c_int64(n), p(stream), p(emax), p(xb), m, p(y))
        want = x.double().numpy() @ held.astype(np.float64)
        assert np.allclose(y, want, rtol=1e-12, atol=1e-300), np.abs(y - want).max()


@pytest.mark.parametrize("k,n", [(64, 128), (96, 128), (288, 256)])
def test_int4_stream_round_trip_and_decode(emul, k, n):
    """TKD_INT4: codes in bfloat4_b's words, the group scales (times 2^65) where bfloat4_b keeps its exponents; the
    kernel's per-block sum-then-scale gives x @ (q * s)."""
    g = torch.Generator().manual_seed(k * n)
    q = torch.randint(-7, 8, (k, n), generator=g).numpy()
    kg = k // 32  # (96 and 288 end inside a super-atom of 64 k)
    scales = (torch.rand(kg, n, generator=g) * 0.02 + 1e-3).to(torch.bfloat16)
    codes = np.ascontiguousarray((np.abs(q) | ((q < 0) << 3)).astype(np.uint8))
    sbits = np.ascontiguousarray(scales.view(torch.int16).numpy().view(np.uint16))
    held = orc.int4_dequantized(q.T, scales.float().numpy().T).T
    stream, _, wide = pack(emul, "int4", sbits, codes)
    assert wide == 0
    back = np.zeros((k, n), np.float32)
    emul.emul_unpack(FMT["int4"], ctypes.c_int64(k), ctypes.c_int64(n), p(stream), None, p(back))
    assert np.array_equal(back.view(np.uint32), np.ascontiguousarray(held).view(np.uint32))
    for m in (1, 5):
        x = torch.randn(m, k, generator=g).to(torch.bfloat16)
        y = np.zeros((m, n), np.float64)
        xb = np.ascontiguousarray(x.view(torch.int16).numpy().view(np.uint16))
        emul.emul_matmul(FMT["int4"], ctypes.c_int64(k), ctypes.c_int64(n), p(stream), None, p(xb), m, p(y))
        want = x.double().numpy() @ held.astype(np.float64)
        assert np.allclose(y, want, rtol=1e-11, atol=1e-300), np.abs(y - want).max()


def test_every_stream_bit_is_owned_once(emul):
    """Packing all-ones codes and exponents fills the stream's code words completely: the layout is a bijection."""
    k, n = 320, 128
    for fmt, code in (("bfp8", 0xFF), ("bfp4", 0x0F)):
        exps = np.full((k, n // 16), 100, np.uint8)
        codes = np.full((k, n), code, np.uint8)
        stream, emax, _ = pack(emul, fmt, exps, codes)
        sa = stream.reshape(-1, SAB[fmt])
        eb = SAB[fmt] - 512
        assert np.all(sa[:, eb:] == 0xFF)
        words = sa[:, :eb].copy().view(np.uint32)
        # bfloat8_b: four exponent fields of 196 = 0xC4 << 7, rotated: all bits owned; bfloat4_b: four 6-bit fields of 63
        assert np.all(words == np.uint32(0x62626262 if fmt == "bfp8" else 0x1FBF1FBF))


def test_wide_weight_is_flagged(emul):
    w = np.full((64, 128), 1.0, np.float32)
    w[3] = 1e-20
    exps, codes = orc.quantise_c(w, "bfp8")
    assert pack(emul, "bfp8", exps, codes)[2] == 1
