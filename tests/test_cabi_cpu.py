"""Without a GPU: libtkd.so loads, exports every symbol include/tkd.h declares, its struct layout matches the ctypes
mirror, and the launch plan (pure host arithmetic) gives the numbers the design states. No compute call is made."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def tkd():
    import sys

    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as ge

    ge.build_library()
    from dense_reader import _tkd

    return _tkd


def test_exports_match_header(tkd):
    header = (ROOT / "include" / "tkd.h").read_text()
    declared = set(re.findall(r"^\s*(?:int|int64_t|const char\*)\s+(tkd_\w+)\(", header, re.M))
    assert declared == set(tkd.SYMBOLS), declared ^ set(tkd.SYMBOLS)
    lib = ctypes.CDLL(str(tkd.LIB_PATH))
    for name in declared:
        assert hasattr(lib, name), name
    assert tkd.lib().tkd_version() == 3 and tkd.lib().tkd_layout_version() >= 3
    assert tkd.lib().tkd_error_string(3).decode().startswith("a kernel")


def test_stream_sizes(tkd):
    L = tkd.lib()
    # bytes per weight: 1.0625, 0.5625, 2 (the reference's 1088 / 576 / 2048 bytes per 1024 values)
    assert L.tkd_packed_bytes(tkd.FMT_BFP8, 2048, 4096) == 2048 * 4096 * 1088 // 1024 == 8912896
    assert L.tkd_packed_bytes(tkd.FMT_BFP4, 4096, 14336) * 2 == 66060288
    assert L.tkd_packed_bytes(tkd.FMT_BFP8, 14336, 4096) == 62390272
    assert L.tkd_packed_bytes(tkd.FMT_BFP8, 4096, 151936) == 661225472
    assert L.tkd_packed_bytes(tkd.FMT_BF16, 1024, 48) == 1024 * 128 * 2  # N padded to a panel of 128 columns
    assert L.tkd_padded_cols(33) == 128


def plan(tkd, **kw):
    a = tkd.TkdMatmul()
    a.nblocks, a.epilogue, a.out_dtype = 1, tkd.EPI_PLAIN, tkd.DT_BF16
    ns = kw.pop("ns", None)
    for k, v in kw.items():
        setattr(a, k, v)
    for i, n in enumerate(ns):
        a.block[i].n = n
    a.nblocks = len(ns)
    p = tkd.TkdPlan()
    rc = tkd.lib().tkd_matmul_plan(ctypes.byref(a), ctypes.byref(p))
    return rc, p


def test_plans(tkd):
    rc, p = plan(tkd, fmt=tkd.FMT_BFP4, m=1, k=4096, ns=[14336], epilogue=tkd.EPI_GLU2)
    assert rc == 0 and p.ks == 1024 and p.nslices == 4 and p.panels == 224 and p.items == 896
    assert p.weight_bytes == 66060288 and p.smem_bytes <= 227 * 1024 and p.stages >= 4
    rc, p = plan(tkd, fmt=tkd.FMT_BFP8, m=32, k=14336, ns=[4096], epilogue=tkd.EPI_OUT32, out_dtype=tkd.DT_F32)
    assert rc == 0 and p.ks == 3584 and p.nslices == 4 and p.panels == 32 and p.stages >= 3 and p.stream_warps == 16  # (32 rows: the tensor-memory kernel, 16 decode warps)
    rc, p = plan(tkd, fmt=tkd.FMT_BFP8, m=4, k=4096, ns=[4096, 1024, 1024, 4096])
    assert rc == 0 and p.panels == 32 + 8 + 8 + 32
    # refusals
    assert plan(tkd, fmt=tkd.FMT_BFP8, m=33, k=4096, ns=[64])[0] == 1
    assert plan(tkd, fmt=tkd.FMT_BFP8, m=1, k=4016, ns=[64])[0] == 1
    assert plan(tkd, fmt=7, m=1, k=4096, ns=[64])[0] == 1
    assert plan(tkd, fmt=tkd.FMT_BFP8, m=1, k=4096, ns=[64], ks=100)[0] == 1
    assert plan(tkd, fmt=tkd.FMT_BFP8, m=1, k=2048, ns=[4096])[1].ks == 512 and plan(tkd, fmt=tkd.FMT_BFP8, m=1, k=1024, ns=[64])[1].ks == 256
    assert plan(tkd, fmt=tkd.FMT_BFP8, m=1, k=4096, ns=[96], epilogue=tkd.EPI_GLU_IL)[0] == 1


def test_host_logic_without_gpu(tkd):
    """The host-side mirror of the reference's helpers needs no GPU."""
    import numpy as np
    import torch

    from common import device as cdev
    from dense_reader import linear

    h = np.load(ROOT / "tests" / "golden" / "host_helpers.npz")
    gate = torch.arange(128.0).reshape(64, 2)
    assert np.array_equal(linear.interleave_glu(gate, -gate).numpy(), h["il"])
    assert np.array_equal(linear.bf16_ceil(torch.from_numpy(h["ceil_in"])).numpy(), h["ceil_out"])
    assert [cdev.split_arg(True, v) for v in (0.5, 0.6, 2 / 3, 0.75)] + [cdev.split_arg(False)] == h["split"].tolist()
    vals, idx = linear.records_host(torch.from_numpy(h["rec"]), 2, 4)
    assert np.array_equal(vals.numpy().view(np.uint32), h["rec_vals"].view(np.uint32))
    assert np.array_equal(idx.numpy(), h["rec_idx"])
    x, wk, sc = torch.from_numpy(h["x"]), torch.from_numpy(h["wk"]), torch.from_numpy(h["sc"])
    assert np.array_equal(linear.reference(x, wk).numpy(), h["ref"])
    assert np.array_equal(linear.reference(x, wk, sc).numpy(), h["ref_sc"])
    assert linear.is_block_list([(object(), 0), (object(), 3)]) and not linear.is_block_list((object(), object()))
    assert linear.topk_units(151936) == 75 and linear.topk_units(2048) == 1


def test_no_cpu_fallback(tkd):
    """Without a CUDA device the product path refuses instead of computing on the host."""
    import torch

    from common import ttnn_like as ttnn

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError):
        ttnn.open_device(0)
