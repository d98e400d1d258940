"""Without a GPU: the oracle's restatement of the reference's ternary host forms and the product's own
(ternary_matmul/t2.py: tiles, sylvester, rotate, dequantize, reference) against golden vectors made by running the
reference (tests/golden/ternary.npz, gen_golden.py)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle as orc

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def gold():
    g = np.load(GOLDEN / "ternary.npz")
    return {k: g[k] for k in g.files}


def test_oracle_against_golden(gold):
    trits, signs = gold["trits"], gold["signs"]
    scales = torch.from_numpy(gold["scales_bits"]).view(torch.float16)
    x = torch.from_numpy(gold["x_bits"]).view(torch.bfloat16)
    for fmt in ("bfp2", "bfp4"):
        assert np.array_equal(orc.t2_tiles(trits.T, fmt), gold[f"tiles_{fmt}"]), fmt
    assert np.array_equal(orc.t2_tiles(trits.T, "bfp2c"), gold["tiles_bfp2c"])
    np.testing.assert_allclose(orc.t2_rotate(x.double().numpy(), signs), gold["rotated"], rtol=0, atol=1e-11)
    assert np.array_equal(orc.t2_dequantize(trits, scales.to(torch.bfloat16), 128), gold["deq"])
    np.testing.assert_allclose(orc.t2_reference(x, trits, scales, 128), gold["ref"], rtol=2e-5, atol=2e-5)


def test_host_mirror_against_golden(gold):
    from ternary_matmul import t2

    trits, signs = torch.from_numpy(gold["trits"]), torch.from_numpy(gold["signs"])
    scales = torch.from_numpy(gold["scales_bits"]).view(torch.float16)
    x = torch.from_numpy(gold["x_bits"]).view(torch.bfloat16)
    for fmt in ("bfp2", "bfp2c", "bfp4"):
        assert np.array_equal(t2.tiles(trits.T.contiguous(), fmt).numpy(), gold[f"tiles_{fmt}"]), fmt
    assert np.array_equal(t2.sylvester(8).numpy(), gold["sylvester8"])
    assert np.array_equal(t2.rotate(x.double(), signs).numpy(), gold["rotated"])
    assert np.array_equal(t2.dequantize(trits, scales.to(torch.bfloat16), 128).numpy(), gold["deq"])
    assert np.array_equal(t2.reference(x, trits, scales, 128).numpy(), gold["ref"])
