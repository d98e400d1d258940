"""Without a GPU: the oracle's restatement of the reference's int4 host forms and the product's own (int4/w4a16.py:
nibbles, dequantized, reference) against golden vectors made by running the reference (tests/golden/int4.npz,
gen_golden.py), and what the C-ABI says of TKD_FMT_INT4 without launching anything."""

import ctypes
import hashlib
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle as orc

GOLDEN = Path(__file__).resolve().parent / "golden"
sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()  # noqa: E731


def case(n, k, seed):
    """The reference tests' generator (int4/tests/test_int4.py:27-31)."""
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(-7, 8, (n, k), generator=g).to(torch.int8)
    scales = (torch.rand(n, k // 32, generator=g) * 0.01 + 0.001).to(torch.bfloat16)
    return codes, scales


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLDEN / "int4.npz")


def test_oracle_against_golden(gold):
    codes, sbits, x = gold["codes1"], gold["scales1_bits"], torch.from_numpy(gold["x1"])
    scales = torch.from_numpy(sbits).view(torch.bfloat16)
    assert np.array_equal(orc.int4_nibbles(codes.T), gold["nib1"])
    assert np.array_equal(orc.int4_dequantized(codes, scales), gold["deq1"])
    np.testing.assert_allclose(orc.int4_reference(x, codes, scales), gold["ref1"], rtol=1e-5, atol=1e-6)
    c2, s2 = case(1152, 1024, 1024 + 1152)
    assert sha(c2.numpy()) == str(gold["codes2_sha"]), "torch's generator gives other codes here than where the vectors were made"
    assert sha(orc.int4_nibbles(c2.numpy().T)) == str(gold["nib2_sha"])
    assert sha(orc.int4_dequantized(c2.numpy(), s2)) == str(gold["deq2_sha"])
    g = torch.Generator().manual_seed(1152)
    x2 = torch.randn(1, 1024, generator=g)
    x2[:, torch.randperm(1024, generator=g)[:8]] *= 20
    np.testing.assert_allclose(orc.int4_reference(x2, c2.numpy(), s2), gold["ref2"], rtol=2e-5, atol=1e-5)


def test_host_mirror_against_golden(gold):
    from int4 import w4a16

    codes, sbits, x = torch.from_numpy(gold["codes1"]), gold["scales1_bits"], torch.from_numpy(gold["x1"])
    scales = torch.from_numpy(sbits).view(torch.bfloat16)
    assert np.array_equal(w4a16.nibbles(codes.T.contiguous()).numpy(), gold["nib1"])
    assert np.array_equal(w4a16.dequantized(codes, scales).numpy(), gold["deq1"])
    assert np.array_equal(w4a16.reference(x, codes, scales).numpy(), gold["ref1"])
    c2, s2 = case(1152, 1024, 1024 + 1152)
    assert sha(w4a16.nibbles(c2.T.contiguous()).numpy()) == str(gold["nib2_sha"])
    assert sha(w4a16.dequantized(c2, s2).numpy()) == str(gold["deq2_sha"])


def test_cabi_int4_without_a_launch():
    from dense_reader import _tkd

    L = _tkd.lib()
    # the stream: bfloat4_b's geometry, 0.5625 bytes a weight (the reference's 512 nibble bytes + 32 scales per tile)
    assert L.tkd_packed_bytes(_tkd.FMT_INT4, 4096, 14336) == L.tkd_packed_bytes(_tkd.FMT_BFP4, 4096, 14336) == 4096 * 14336 * 576 // 1024
    a = _tkd.TkdMatmul()
    a.fmt, a.m, a.k, a.nblocks, a.epilogue, a.out_dtype = _tkd.FMT_INT4, 1, 4096, 1, _tkd.EPI_PLAIN, _tkd.DT_BF16
    a.block[0].n = 14336
    plan = _tkd.TkdPlan()
    assert L.tkd_matmul_plan(ctypes.byref(a), ctypes.byref(plan)) == 0
    assert plan.chunk_k == 512 and plan.panels == 112
    a.m = 9  # more than eight rows: the dequantised bfloat8_b form's job
    assert L.tkd_matmul_plan(ctypes.byref(a), ctypes.byref(plan)) != 0
