"""tkd_matmul_noalloc, the entry point for hosts that cannot allocate device memory (a plugin inside another
framework's pool, a fixed-arena replay): called through the C-ABI, its output must equal tkd_matmul's bit for bit,
call after call, because it is the same kernel with its workspace in the library's built-in array.

Collected last on purpose (the file name): a run that stops at the first failure has then run every other test."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

from common import ttnn_like as ttnn  # noqa: E402
from dense_reader import _tkd, linear  # noqa: E402


def describe(tw, x, out, m, k, n):
    a = _tkd.TkdMatmul()
    a.fmt, a.m, a.k = tw.fmt, m, k
    a.x, a.ldx = x.data_ptr(), k
    a.nblocks, a.epilogue = 1, _tkd.EPI_PLAIN
    a.block[0].w, a.block[0].emax, a.block[0].n = tw.t.data_ptr(), tw.emax.data_ptr(), n
    a.out, a.out_dtype, a.ldo = out.data_ptr(), _tkd.DT_BF16, n
    return a


@pytest.mark.parametrize("dtype,m", [(ttnn.bfloat8_b, 1), (ttnn.bfloat4_b, 3)])
def test_noalloc_equals_matmul_twice(device, dtype, m):
    L = _tkd.lib()
    k, n = 4096, 4096 + 128  # 33 panels of 4 slices on 132 CTAs: every panel's slices are spread over four CTAs (scratch in use)
    g = torch.Generator().manual_seed(71)
    tw, _ = linear.native_weight(device, torch.randn(n, k, generator=g) * 0.02, dtype)
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(device.torch)
        want = torch.full((m, n), 7.0, dtype=torch.bfloat16, device=device.torch)
        got = torch.full((m, n), -7.0, dtype=torch.bfloat16, device=device.torch)
        a = describe(tw, x, want, m, k, n)
        need = ctypes.c_uint64(0)
        _tkd.check(L.tkd_matmul_workspace(ctypes.byref(a), ctypes.byref(need)), "workspace")
        assert need.value <= 8 << 20
        ws = torch.zeros(need.value, dtype=torch.uint8, device=device.torch)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        _tkd.check(L.tkd_matmul(ctypes.byref(a), stream), "tkd_matmul")
        b = describe(tw, x, got, m, k, n)  # no workspace given
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0] if call else None  # (the first call is where the array is resolved)
        _tkd.check(L.tkd_matmul_noalloc(ctypes.byref(b), stream), "tkd_matmul_noalloc")
        torch.cuda.synchronize()
        if call:
            assert torch.cuda.mem_get_info()[0] == free_before  # nothing was allocated or freed
        assert torch.equal(got, want), f"call {call}"
        ref = x.float() @ ttnn.to_torch(tw)[0, 0, :, :n].to(device.torch)
        assert ((got.float() - ref).norm() / ref.norm()).item() < 0.01


def test_noalloc_refuses_what_does_not_fit(device):
    """Eight rows against the LM head (1187 panels of 4 slices, 8 KB of slice sums each) need more scratch than the
    built-in array: refused, nothing launched."""
    L = _tkd.lib()
    a = _tkd.TkdMatmul()
    a.fmt, a.m, a.k, a.nblocks, a.epilogue, a.out_dtype = _tkd.FMT_BFP8, 8, 4096, 1, _tkd.EPI_PLAIN, _tkd.DT_BF16
    a.block[0].n = 151936
    assert L.tkd_matmul_noalloc(ctypes.byref(a), None) == _tkd.ERR_FIXED_SCRATCH
    assert b"built-in" in L.tkd_error_string(_tkd.ERR_FIXED_SCRATCH)


def test_noalloc_reset_recovers_from_dirty_counters(device):
    """A kernel that gave up a bounded wait can leave the built-in array's panel counters mid-count, and the next call
    would then add a panel up early, or never. The counters are dirtied here from the host side (a merge
    record written over them: no kernel is made to time out): a call then leaves its output unwritten, and after
    tkd_matmul_noalloc_reset the calls are right again."""
    L = _tkd.lib()
    m, k, n = 1, 4096, 4096 + 128
    g = torch.Generator().manual_seed(72)
    tw, _ = linear.native_weight(device, torch.randn(n, k, generator=g) * 0.02, ttnn.bfloat8_b)
    stream = torch.cuda.current_stream().cuda_stream
    xs = [torch.randn(m, k, generator=g).to(torch.bfloat16).to(device.torch) for _ in range(2)]
    wants = []
    for x in xs:  # what tkd_matmul gives, with a workspace of its own
        want = torch.empty((m, n), dtype=torch.bfloat16, device=device.torch)
        a = describe(tw, x, want, m, k, n)
        need = ctypes.c_uint64(0)
        _tkd.check(L.tkd_matmul_workspace(ctypes.byref(a), ctypes.byref(need)), "workspace")
        ws = torch.zeros(need.value, dtype=torch.uint8, device=device.torch)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        _tkd.check(L.tkd_matmul(ctypes.byref(a), stream), "tkd_matmul")
        wants.append(want)
    got = torch.full((m, n), -7.0, dtype=torch.bfloat16, device=device.torch)
    b0, b1 = describe(tw, xs[0], got, m, k, n), describe(tw, xs[1], got, m, k, n)
    _tkd.check(L.tkd_matmul_noalloc(ctypes.byref(b0), stream), "tkd_matmul_noalloc")
    torch.cuda.synchronize()
    assert torch.equal(got, wants[0])
    # dirty: a record of hundreds over the first 66 words, the panel counters (no panel's count then ever equals its
    # number of slices: no panel is added up and nothing is written)
    addr = ctypes.c_void_p()
    _tkd.check(L.tkd_noalloc_scratch_address(ctypes.byref(addr)), "tkd_noalloc_scratch_address")
    rec = torch.full((2 * 33,), 100, dtype=torch.int32, device=device.torch)
    _tkd.check(L.tkd_topk_merge(rec.data_ptr(), 1, 1, 33, 33, addr.value, stream), "tkd_topk_merge")
    _tkd.check(L.tkd_matmul_noalloc(ctypes.byref(b1), stream), "tkd_matmul_noalloc")
    torch.cuda.synchronize()
    assert not torch.equal(got, wants[1])  # the dirt shows
    _tkd.check(L.tkd_matmul_noalloc_reset(stream), "tkd_matmul_noalloc_reset")
    for b, want in ((b1, wants[1]), (b0, wants[0]), (b1, wants[1])):
        got.fill_(-7.0)
        _tkd.check(L.tkd_matmul_noalloc(ctypes.byref(b), stream), "tkd_matmul_noalloc")
        torch.cuda.synchronize()
        assert torch.equal(got, want)
