"""_tkd.py: ctypes binding of libtkd.so (include/tkd.h), the only way the Python layer reaches the GPU kernels.

There is no fallback: if the library is missing the import fails with the build command, and every call that returns a
non-zero code raises.
"""

import ctypes
from pathlib import Path

PKG = Path(__file__).resolve().parents[1]
LIB_PATH = PKG / "csrc" / "libtkd.so"

FMT_BFP8, FMT_BFP4, FMT_BF16, FMT_INT4 = 0, 1, 2, 3
EPI_PLAIN, EPI_GLU_IL, EPI_GLU2, EPI_RESIDUAL, EPI_OUT32 = range(5)
DT_NONE, DT_BF16, DT_F32 = 0, 1, 2
ERR_UNSUPPORTED, ERR_TIMEOUT, ERR_WIDE, ERR_FIXED_SCRATCH = 2, 3, 5, 6

c_i32, c_i64, c_u32, c_u64, c_vp = ctypes.c_int32, ctypes.c_int64, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_void_p


class TkdBlock(ctypes.Structure):
    _fields_ = [("w", c_vp), ("w_up", c_vp), ("emax", c_vp), ("emax_up", c_vp), ("n", c_i64), ("out_col0", c_i64)]


class TkdMatmul(ctypes.Structure):
    _fields_ = [
        ("fmt", c_i32), ("m", c_i32), ("k", c_i64), ("x", c_vp), ("ldx", c_i64), ("nblocks", c_i32), ("epilogue", c_i32),
        ("block", TkdBlock * 4), ("act", c_i32), ("scale_dtype", c_i32), ("scale", c_vp), ("scale_up", c_vp),
        ("residual", c_vp), ("ldr", c_i64), ("residual_dtype", c_i32), ("out_dtype", c_i32), ("out", c_vp), ("ldo", c_i64),
        ("records", c_vp), ("topk_k", c_i32), ("topk_rows", c_i32), ("topk_unit", c_i32), ("topk_slot0", c_i32),
        ("topk_write_y", c_i32), ("topk_base", c_u32), ("topk_n", c_i64), ("workspace", c_vp), ("workspace_bytes", c_u64),
        ("status", c_vp), ("ks", c_i32), ("max_ctas", c_i32),
        ("nranks", c_i32), ("rank", c_i32), ("peer_out", c_vp * 7), ("peer_records", c_vp * 7), ("peer_flags", c_vp * 7),
        ("flags", c_vp), ("exchange_wait", c_i32), ("weights_fresh", c_i32), ("hadamard", c_vp),
    ]


MAX_RANKS, FLAG_SEQ, FLAG_WORDS = 8, 8, 16


class TkdMoe(ctypes.Structure):
    _fields_ = [
        ("w", c_vp), ("emax", c_vp), ("expert_bytes", c_i64), ("experts", c_i32), ("k_in", c_i32), ("n", c_i32),
        ("rows", c_i32), ("x", c_vp), ("ldx", c_i64), ("ids", c_vp), ("ids32", c_i32), ("k", c_i32), ("ld_ids", c_i64),
        ("route_w", c_vp), ("ld_w", c_i64), ("by_union", c_i32), ("slots", c_i32), ("act", c_i32), ("bias", c_vp),
        ("out", c_vp), ("ldo", c_i64), ("workspace", c_vp), ("workspace_bytes", c_u64), ("fmt", c_i32),
    ]


class TkdPlan(ctypes.Structure):
    _fields_ = [
        ("ks", c_i32), ("nslices", c_i32), ("panels", c_i32), ("grid", c_i32), ("stages", c_i32), ("stream_warps", c_i32),
        ("chunk_k", c_i32), ("smem_bytes", c_i32), ("items", c_i64), ("weight_bytes", c_i64),
    ]


SYMBOLS = {
    "tkd_version": (c_i32, []),
    "tkd_struct_bytes": (c_i32, [c_i32]),
    "tkd_error_string": (ctypes.c_char_p, [c_i32]),
    "tkd_padded_cols": (c_i64, [c_i64]),
    "tkd_packed_bytes": (c_i64, [c_i32, c_i64, c_i64]),
    "tkd_quantise": (c_i32, [c_i32, c_vp, c_i32, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp]),
    "tkd_pack": (c_i32, [c_i32, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "tkd_layout_version": (c_i32, []),
    "tkd_dequantise_bf16": (c_i32, [c_i32, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp]),
    "tkd_unpack": (c_i32, [c_i32, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp]),
    "tkd_matmul_plan": (c_i32, [ctypes.POINTER(TkdMatmul), ctypes.POINTER(TkdPlan)]),
    "tkd_matmul_workspace": (c_i32, [ctypes.POINTER(TkdMatmul), ctypes.POINTER(c_u64)]),
    "tkd_matmul": (c_i32, [ctypes.POINTER(TkdMatmul), c_vp]),
    "tkd_matmul_host": (c_i32, [ctypes.POINTER(TkdMatmul), c_vp, c_vp, c_vp]),
    "tkd_matmul_noalloc": (c_i32, [ctypes.POINTER(TkdMatmul), c_vp]),
    "tkd_matmul_noalloc_reset": (c_i32, [c_vp]),
    "tkd_noalloc_scratch_address": (c_i32, [ctypes.POINTER(c_vp)]),
    "tkd_hadamard": (c_i32, [c_vp, c_i64, c_vp, c_i32, c_i32, c_vp, c_i64, c_vp]),
    "tkd_moe_workspace": (c_i32, [ctypes.POINTER(TkdMoe), ctypes.POINTER(c_u64)]),
    "tkd_moe_gate_up": (c_i32, [ctypes.POINTER(TkdMoe), c_vp]),
    "tkd_moe_down": (c_i32, [ctypes.POINTER(TkdMoe), c_vp]),
    "tkd_moe_route": (c_i32, [c_vp, c_i64, c_i32, c_i32, c_i32, c_i32, c_vp, ctypes.c_double, c_i32, c_i32, c_i32, c_i32, c_u32,
                              c_vp, c_i32, c_i64, c_vp, c_i64, c_vp, c_i64, c_vp]),
    "tkd_topk_merge": (c_i32, [c_vp, c_i32, c_i32, c_i32, c_i32, c_vp, c_vp]),
    "tkd_head_pick": (c_i32, [c_vp, c_i32, c_i32, c_i32, c_i32, c_u32, c_vp, c_i64, c_i32, c_vp, c_i64, c_i32, c_vp, c_vp, c_vp]),
    "tkd_head_pick_records": (c_i32, [c_vp, c_i32, c_i32, c_i32, c_u32, c_vp, c_vp, c_vp, c_vp]),
    "tkd_exchange_wait": (c_i32, [c_vp, c_i32, c_vp, c_vp]),
    "tkd_exchange_publish": (c_i32, [c_vp, ctypes.POINTER(c_vp), c_i32, c_i32, c_i32, c_vp, c_vp]),
    "tkd_peer_alloc": (c_i32, [c_u64, ctypes.POINTER(c_vp), c_vp]),
    "tkd_peer_free": (c_i32, [c_vp]),
    "tkd_peer_open": (c_i32, [c_vp, ctypes.POINTER(c_vp)]),
    "tkd_peer_close": (c_i32, [c_vp]),
}

_lib = None


def lib():
    """The loaded library; a RuntimeError naming the build step when it is not there."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"dense_reader: {LIB_PATH} is missing; build it with `python {PKG / 'build.py'}` (nvcc, sm_100a). There is"
                " no CPU path."
            )
        L = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        for which, mirror in enumerate((TkdMatmul, TkdPlan, TkdBlock, TkdMoe)):
            if L.tkd_struct_bytes(which) != ctypes.sizeof(mirror):
                raise RuntimeError(f"dense_reader: {LIB_PATH} was built from another include/tkd.h ({mirror.__name__}"
                                   f" is {L.tkd_struct_bytes(which)} bytes there, {ctypes.sizeof(mirror)} here): rebuild")
        _lib = L
    return _lib


class TkdError(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        super().__init__(f"dense_reader: {what}: {lib().tkd_error_string(code).decode()} (code {code})")


def check(code, what):
    if code:
        raise TkdError(code, what)
