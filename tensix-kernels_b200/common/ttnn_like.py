"""ttnn_like.py: the few names of ttnn the dense_reader path's callers use, over torch CUDA tensors.

The reference's API takes and returns ttnn tensors (dense_reader/linear.py:568-624). On a B200 there is no ttnn; this
module is the naming glue that lets callers and the ported tests read the same: dtype and layout tokens, memory-config
tokens (accepted and recorded, they select nothing here), a Tensor that wraps a torch CUDA tensor and answers the
attribute queries linear.py makes (.shape, .padded_shape, .dtype, .layout, .memory_config(), .device(),
.buffer_address()), and from_torch / to_torch / allocate_tensor_on_device / deallocate / reshape / silu. It is not a
backend switch: every tensor lives in the GPU's memory and every op is this package's CUDA code or a torch copy.

Block-float weights (bfloat8_b, bfloat4_b) made by from_torch are Weight objects: the packed HBM stream the kernels
read (csrc/tkd_layout.h), made on the GPU by libtkd's packer.
"""

import enum
import itertools
import math

import torch

from dense_reader import _tkd

TILE = 32


class DataType(enum.Enum):
    bfloat16 = "bfloat16"
    float32 = "float32"
    uint32 = "uint32"
    int32 = "int32"
    uint16 = "uint16"
    uint8 = "uint8"
    bfloat8_b = "bfloat8_b"
    bfloat4_b = "bfloat4_b"


bfloat16, float32, uint32, int32 = DataType.bfloat16, DataType.float32, DataType.uint32, DataType.int32
uint16, uint8 = DataType.uint16, DataType.uint8
bfloat8_b, bfloat4_b = DataType.bfloat8_b, DataType.bfloat4_b

_TORCH = {
    bfloat16: torch.bfloat16, float32: torch.float32, uint32: torch.int32, int32: torch.int32, uint16: torch.int16,
    uint8: torch.uint8,
}
_FROM_TORCH = {torch.bfloat16: bfloat16, torch.float32: float32, torch.int32: int32, torch.uint8: uint8, torch.int16: uint16}
FMT = {bfloat8_b: _tkd.FMT_BFP8, bfloat4_b: _tkd.FMT_BFP4, bfloat16: _tkd.FMT_BF16}


class Layout(enum.Enum):
    TILE = "tile"
    ROW_MAJOR = "row_major"


TILE_LAYOUT, ROW_MAJOR_LAYOUT = Layout.TILE, Layout.ROW_MAJOR


class TensorMemoryLayout(enum.Enum):
    INTERLEAVED = "interleaved"
    WIDTH_SHARDED = "width_sharded"


class BufferType(enum.Enum):
    DRAM = "dram"
    L1 = "l1"


class ShardSpec:
    """A width-sharded weight's shard: (K, columns per bank) over `banks` banks (HBM stacks here)."""

    def __init__(self, banks, shape):
        self.banks, self.shape = banks, tuple(shape)
        self.grid, self.orientation = f"banks[0..{banks - 1}]", "row_major"

    def num_cores(self):
        return self.banks


class MemoryConfig:
    def __init__(self, memory_layout=TensorMemoryLayout.INTERLEAVED, buffer_type=BufferType.DRAM, shard_spec=None):
        self.memory_layout, self.buffer_type, self.shard_spec = memory_layout, buffer_type, shard_spec

    def __str__(self):
        sp = self.shard_spec
        return f"MemoryConfig({self.memory_layout.value},{self.buffer_type.value},{(sp.banks, sp.shape) if sp else None})"


DRAM_MEMORY_CONFIG = MemoryConfig()
L1_MEMORY_CONFIG = MemoryConfig(buffer_type=BufferType.L1)


class Grid:
    def __init__(self, x, y):
        self.x, self.y = x, y


class Device:
    """One CUDA device. The "compute grid" is its SMs, the "DRAM grid" its HBM stacks."""

    HBM_STACKS = 8

    def __init__(self, device_id=0):
        if not torch.cuda.is_available():
            raise RuntimeError("dense_reader: no CUDA device (this package has no CPU path)")
        self.id = device_id
        self.torch = torch.device("cuda", device_id)
        self.sms = torch.cuda.get_device_properties(device_id).multi_processor_count
        _tkd.lib()

    def compute_with_storage_grid_size(self):
        return Grid(self.sms, 1)

    def dram_grid_size(self):
        return Grid(self.HBM_STACKS, 1)

    def __repr__(self):
        return f"Device(cuda:{self.id})"


_DEVICES = {}


def open_device(device_id=0):
    if device_id not in _DEVICES:
        _DEVICES[device_id] = Device(device_id)
    return _DEVICES[device_id]


def close_device(device):
    torch.cuda.synchronize(device.torch)


def _pad(n):
    return -(-n // TILE) * TILE


class Tensor:
    """A torch CUDA tensor of the logical shape with ttnn's attribute surface. TILE layout only changes what
    padded_shape reports (ttnn pads the last two dimensions to 32); the storage stays row-major."""

    def __init__(self, t, dtype, layout, device, memory_config):
        self.t, self.dtype, self.layout, self._device = t, dtype, layout, device
        self._mc = memory_config or DRAM_MEMORY_CONFIG

    @property
    def shape(self):
        return list(self.t.shape)

    @property
    def padded_shape(self):
        s = list(self.t.shape)
        if self.layout == TILE_LAYOUT and len(s) >= 2:
            s[-1], s[-2] = _pad(s[-1]), _pad(s[-2])
        return s

    def memory_config(self):
        return self._mc

    def device(self):
        return self._device

    def buffer_address(self):
        return self.t.data_ptr()


class Weight(Tensor):
    """A [1, 1, K, N] weight as the packed stream the kernels read. `t` is the stream (uint8), `emax` the per-group
    side array (None for a bfloat16 stream), `fmt` the stream's format: the dtype's own, or bfloat16 for a "wide"
    block-float weight (one whose exponents inside a group of 16 columns spread further than the block-float stream
    encodes: its values, all exact in bf16, are then streamed as bf16). `serial` numbers the weights of a process."""

    _serials = itertools.count(1)

    def __init__(self, stream, emax, k, n, dtype, device, memory_config, fmt=None):
        super().__init__(stream, dtype, TILE_LAYOUT, device, memory_config)
        self.emax, self.k, self.n = emax, k, n
        self.fmt = FMT[dtype] if fmt is None else fmt
        self.wide = self.fmt != FMT[dtype]
        self.serial = next(Weight._serials)
        sp = memory_config.shard_spec
        self._npad = sp.shape[1] * sp.banks if sp else _pad(n)

    @property
    def shape(self):
        return [1, 1, self.k, self.n]

    @property
    def padded_shape(self):
        return [1, 1, self.k, self._npad]


def _stream_ptr():
    return torch.cuda.current_stream().cuda_stream


def pack_weight(device, wt, dtype, orient, col_div=None, memory_config=None):
    """A float32 matrix (orient 0: [N, K] as torch's [out, in]; 1: [K, N]) -> Weight, on the GPU (libtkd: tkd_quantise,
    tkd_pack)."""
    L = _tkd.lib()
    fmt = FMT[dtype]
    src = wt.to(device.torch, torch.float32).contiguous()
    n, k = (src.shape[0], src.shape[1]) if orient == 0 else (src.shape[1], src.shape[0])
    assert k % TILE == 0, f"K {k} is not a multiple of 32"
    npad = L.tkd_padded_cols(n)
    with torch.cuda.device(device.torch):
        exps = torch.empty(max(1, k * (npad // 16)), dtype=torch.uint8, device=device.torch)
        codes = torch.empty(k * npad * (2 if fmt == _tkd.FMT_BF16 else 1), dtype=torch.uint8, device=device.torch)
        div = None if col_div is None else col_div.to(device.torch, torch.float32).contiguous()
        _tkd.check(
            L.tkd_quantise(fmt, src.data_ptr(), orient, k, n, div.data_ptr() if div is not None else None,
                           exps.data_ptr(), codes.data_ptr(), _stream_ptr()),
            "tkd_quantise",
        )
        stream = torch.empty(L.tkd_packed_bytes(fmt, k, n), dtype=torch.uint8, device=device.torch)
        emax = None if fmt == _tkd.FMT_BF16 else torch.empty(npad // 16, dtype=torch.uint8, device=device.torch)
        info = torch.zeros(1, dtype=torch.int32, device=device.torch)
        _tkd.check(
            L.tkd_pack(fmt, k, n, exps.data_ptr(), codes.data_ptr(), stream.data_ptr(),
                       emax.data_ptr() if emax is not None else None, info.data_ptr(), _stream_ptr()),
            "tkd_pack",
        )
        if int(info.item()) & 1:
            # a wide weight: the same numbers as a bf16 stream (twice to four times the bytes, and exact)
            vals = torch.empty(k * npad, dtype=torch.int16, device=device.torch)
            _tkd.check(L.tkd_dequantise_bf16(fmt, k, n, exps.data_ptr(), codes.data_ptr(), vals.data_ptr(), _stream_ptr()),
                       "tkd_dequantise_bf16")
            fmt, emax = _tkd.FMT_BF16, None
            stream = torch.empty(L.tkd_packed_bytes(fmt, k, n), dtype=torch.uint8, device=device.torch)
            _tkd.check(L.tkd_pack(fmt, k, n, None, vals.data_ptr(), stream.data_ptr(), None, info.data_ptr(), _stream_ptr()),
                       "tkd_pack")
            torch.cuda.current_stream().synchronize()
    return Weight(stream, emax, k, n, dtype, device, memory_config or DRAM_MEMORY_CONFIG, fmt=fmt)


def as_bf16_stream(w):
    """The weight `w` with its values streamed as bf16 (itself when it already is): what a block list does with its
    other weights when one of them is wide, since one launch streams one format."""
    if w.fmt == _tkd.FMT_BF16:
        return w
    twin = getattr(w, "_bf16_twin", None)
    if twin is None:
        vals = to_torch(w)[0, 0, :, : w.n]
        twin = pack_weight(w._device, vals, bfloat16, 1, memory_config=w._mc)
        twin.dtype = w.dtype
        twin.wide = True
        w._bf16_twin = twin
    return twin


def from_torch(t, dtype=None, layout=ROW_MAJOR_LAYOUT, device=None, memory_config=None):
    """ttnn.from_torch: a host (or device) torch tensor onto the device. Block-float dtypes take [..., K, N] float
    values and give a Weight."""
    device = device or open_device(0)
    if dtype in (bfloat8_b, bfloat4_b):
        k, n = t.shape[-2], t.shape[-1]
        return pack_weight(device, t.reshape(k, n).float(), dtype, 1, memory_config=memory_config)
    if dtype is None:
        dtype = _FROM_TORCH[t.dtype]
    return Tensor(t.to(device.torch, _TORCH[dtype]).contiguous(), dtype, layout, device, memory_config)


def held_values(t):
    """The float32 values a Weight holds, [K, N padded to a panel], on its device (tkd_unpack)."""
    L = _tkd.lib()
    with torch.cuda.device(t._device.torch):
        out = torch.empty(t.k, L.tkd_padded_cols(t.n), dtype=torch.float32, device=t._device.torch)
        _tkd.check(
            L.tkd_unpack(t.fmt, t.k, t.n, t.t.data_ptr(), t.emax.data_ptr() if t.emax is not None else None,
                         out.data_ptr(), _stream_ptr()),
            "tkd_unpack",
        )
    return out


def to_torch(t):
    """ttnn.to_torch: the tensor on the host. A Weight comes back as the float32 values it holds, [1, 1, K, padded N]."""
    if isinstance(t, Weight):
        out = held_values(t)
        full = torch.zeros(1, 1, t.k, max(t.padded_shape[-1], out.shape[1]), dtype=torch.float32)
        full[0, 0, :, : out.shape[1]] = out.cpu()
        return full
    return t.t.cpu()


def allocate_tensor_on_device(shape, dtype, layout, device, memory_config=None):
    return Tensor(torch.empty(list(shape), dtype=_TORCH[dtype], device=device.torch), dtype, layout, device, memory_config)


def Shape(dims):
    return list(dims)


# Counts deallocations: caches of launch descriptors (which hold raw addresses) key on it, so that nothing described
# before a tensor was freed is launched after.
EPOCH = 0


def deallocate(t):
    global EPOCH
    EPOCH += 1
    t.t = None
    if isinstance(t, Weight):
        t.emax = None
        t._bf16_twin = None


def reshape(t, shape):
    return Tensor(t.t.reshape(list(shape)), t.dtype, t.layout, t._device, t._mc)


def to_memory_config(t, memory_config):
    """A copy of t carrying another memory config (there is one kind of device memory here: the copy is what a caller
    that deallocates the result expects)."""
    return Tensor(t.t.clone(), t.dtype, t.layout, t._device, memory_config)


def sharded_to_interleaved(t, memory_config=None):
    return Tensor(t.t, t.dtype, t.layout, t._device, memory_config or DRAM_MEMORY_CONFIG)


def silu(t):
    """ttnn.silu on a bf16 tensor (linear.linear's activation="silu", applied after the matmul as the reference does)."""
    return Tensor(torch.nn.functional.silu(t.t.float()).to(t.t.dtype), t.dtype, t.layout, t._device, t._mc)


def padded_cols(n, banks):
    return math.ceil(n / (TILE * banks)) * TILE * banks
