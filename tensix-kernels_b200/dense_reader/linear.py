"""linear.py: the weight-streaming decode matmul of XylolabsInc/tensix-kernels' dense_reader, on a B200.

y = x @ w (* scale), x bf16 activations, w block-float (bfloat8_b, bfloat4_b) or bfloat16 weights, fp32 accumulation,
bf16 out (or float32), with the fused output stages (per-column scales, act(gate) * up, a residual add, the fp32
accumulator as it is), a top-k of each output row kept as records, and block lists (one launch over several weights).

The module keeps the reference's names, signatures and argument meaning (its dense_reader/linear.py; file:line in the
docstrings below are that file's), so a caller switches by importing this one instead. Underneath there is no ttnn
program: native_weight packs the weight into the HBM stream of csrc/tkd_layout.h on the GPU, and matmul makes one
launch of the sm_100a kernel of csrc/tkd_stream.cu through libtkd's C-ABI (include/tkd.h). Tensors are the thin
wrappers of common/ttnn_like.py around torch CUDA tensors. There is no CPU path: without libtkd.so or without a GPU the
calls raise.

What differs from the reference, by necessity or on purpose:
- Tensix work-split options (cores_per_bank, split, rows, xs, kb, kw, sbw, full_sync, fidelity, memory_config) are
  accepted, checked as the reference checks them, and steer nothing: the kernel's split is plan()'s.
- Top-k records: one record per TOPK_UNIT (2048) output columns instead of one per Tensix core, and inside a record
  the order is key descending, index ascending among equal keys (the reference keeps the same values; which of several
  equal values' indices it keeps depends on its cores' column split).
- Extensions, off unless asked for: col_scales= (float32 per-column scales with a GLU), a float32 residual with out32.
"""

import ctypes
import itertools
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from common import device as dev  # noqa: E402
from common import ttnn_like as ttnn  # noqa: E402
from common.device import (  # noqa: E402,F401  (re-exported, as the reference does)
    FIDELITY,
    TILE,
    bank_grid,
    check_banks,
    dram_banks,
    is_dram_sharded,
    place,
    read_vcs,
    sharded_memcfg,
    split_arg,
)
from dense_reader import _tkd  # noqa: E402

BFP8_TILE = 1088
NATIVE_TILES = {ttnn.bfloat8_b: BFP8_TILE, ttnn.bfloat4_b: 576, ttnn.bfloat16: 2048}

# --- settings. The first group are the reference's (linear.py:52-82): Tensix buffer budgets and split knobs, kept so
# that code which sets them keeps working; they change nothing here. ---
L1_BUDGET = None
L1_MARGIN = 32 * 1024
X_BUDGET = 600_000
XS_DEPTH = 3
MIN_CHUNKS = 0
MIN_CHUNKS_SHAPES = None
NARROW_N = 0
SPLIT_SHARE = 0.5
REQ_TILES = 0
GLU_ROWS = True
CONFIGS = ({"cores_per_bank": 2, "split": True, "rows": True},)
# the top-k result tensor as bfloat16 (the same bytes as the uint32 words; False: uint32)  (linear.py:77-78)
RECORDS_BF16 = False
# launch descriptors cached by everything that shapes them (a hit only rewrites the tensors' addresses)  (:79-80)
CACHE = True
# a line per planned shape on stdout  (:81-82)
LOG = False
# --- B200 settings ---
# output columns per top-k record (a multiple of 128, at most 2048)
TOPK_UNIT = 2048
# k per slice of the kernel's work items (None: the library's default for the row count); CTAs per launch (None: all SMs)
KS = None
MAX_CTAS = None

_TENSIX_OPTS = {"cores_per_bank", "split", "rows", "xs", "kb", "kw", "sbw", "noscale", "glu2", "budget", "mt"}
_OPTS = _TENSIX_OPTS | {"glu", "glu_act", "residual", "residual_mode", "out32", "blocks", "max_banks", "col_scales", "ks",
                        "max_ctas", "exchange", "hadamard"}

_CALLS = {}      # whole calls by the identity of their arguments (a hit goes straight to the library)
_CALLS_MAX = 256
_LAUNCHES = {}   # the launch cache: key -> (TkdMatmul, keep-alive)
_CHOICE = {}     # the plan cache
_WORKSPACE = {}  # device id -> zeroed uint8 tensor
_STATUS = {}     # device id -> int32 status word


# --- host side --------------------------------------------------------------------------------------------------------


def bf16_ceil(s):
    """The smallest bf16 value >= s (s > 0, float32). (linear.py:110-114)"""
    down = s.to(torch.bfloat16).float()
    return torch.where(down >= s, down, (down.view(torch.int32) + (1 << 16)).view(torch.float32))


def native_tile(w):
    """Tile bytes of a weight this matmul reads (bfloat8_b, bfloat4_b, bfloat16), else 0. (linear.py:117-119)"""
    return NATIVE_TILES.get(w.dtype, 0)


def interleave_glu(gate, up):
    """[gate | up] for the fused GLU stage: two float [out, in] matrices as one [2 * out, in] whose 32-row tiles
    alternate, tile 2j the gate's rows 32j .. 32j + 31 and tile 2j + 1 the up's. (linear.py:122-130)"""
    assert gate.shape == up.shape and gate.shape[0] % TILE == 0, (gate.shape, up.shape)
    rows, cols = gate.shape
    both = torch.empty(rows // TILE, 2, TILE, cols, dtype=gate.dtype)
    both[:, 0] = gate.reshape(rows // TILE, TILE, cols)
    both[:, 1] = up.reshape(rows // TILE, TILE, cols)
    return both.reshape(2 * rows, cols)


def scale_tensor(device, s):
    """Per-output-column scales s [N] as [1, 1, 1, N] bf16 on the device. (linear.py:133-141)"""
    return ttnn.from_torch(s.reshape(1, 1, 1, -1).to(torch.bfloat16), dtype=ttnn.bfloat16, layout=ttnn.TILE_LAYOUT,
                           device=device, memory_config=ttnn.DRAM_MEMORY_CONFIG)


def native_weight(device, t, dtype, col_scale=False, sharded=True, max_banks=None):
    """A float [out, in] matrix as a weight [1, 1, in, out] of dtype (bfloat8_b, bfloat4_b or bfloat16) and its
    [1, 1, 1, out] scales: ones, or with col_scale each output column divided by c = max |w| (rounded up to bf16)
    before the block-float rounding and multiplied back after the matmul. (linear.py:144-156)

    The weight is quantised and packed on the GPU (libtkd); `sharded` / `max_banks` only set what its memory config
    reports (width-sharded over the device's banks, or interleaved)."""
    assert dtype in NATIVE_TILES, f"dense_reader: weights are bfloat8_b, bfloat4_b or bfloat16, not {dtype}"
    t = t.float()
    c = bf16_ceil(t.abs().amax(dim=1).clamp(min=1e-8)) if col_scale else torch.ones(t.shape[0])
    n, k = t.shape
    mc = sharded_memcfg(device, k, n, max_banks=max_banks) if sharded else ttnn.DRAM_MEMORY_CONFIG
    w = ttnn.pack_weight(device, t, dtype, 0, col_div=c if col_scale else None, memory_config=mc)
    return w, scale_tensor(device, c)


def block_float(t, dtype):
    """t (float [..., rows, cols]) rounded to dtype's grid, as float32: the values a weight of that dtype holds.
    (linear.py:159-163; the rounding runs on the GPU, through the same packer as native_weight)"""
    lead = t.shape[:-2]
    k, n = t.shape[-2], t.shape[-1]
    out = []
    for m in t.reshape(-1, k, n):
        w = ttnn.pack_weight(ttnn.open_device(0), m.float(), dtype, 1)
        out.append(ttnn.to_torch(w)[0, 0, :, :n])
    return torch.stack(out).reshape(*lead, k, n)


def reference(x, w, scale=None):
    """x @ w (* scale) in float32 on the host, x as the device sees it (bf16); w [K, N] as the weight holds it.
    (linear.py:166-169)"""
    y = x.to(torch.bfloat16).float() @ w.float()
    return y if scale is None else y * scale.float()[None, :]


# --- the plan ---------------------------------------------------------------------------------------------------------


class BlockListMismatch(ValueError):
    """A block list refused before its launch because its one call would not equal one call per block bit for bit
    (linear.py:498-501). The B200 kernel cuts K the same way for every weight of one K, format and row count, so this
    is never raised for lists that pass block_entries; the class stays for callers that catch it."""


def row_slices(x, full_sync=False):
    """[(first row, rows)] of x's rows, at most 32 each: one launch per slice, each reading all the weights once.
    (linear.py:179-184, whose slices are up to 4 tile rows)"""
    m = x.shape[-2]
    return [(m0, min(32, m - m0)) for m0 in range(0, m, 32)]


def _raw(t):
    return t.t if isinstance(t, ttnn.Tensor) else t


# Calls that may overlap on the GPU (different streams) must not share a workspace: the one in use is picked by slot.
WORKSPACE_SLOT = 0


def _ws_key(device):
    return (device.id, WORKSPACE_SLOT)


def _workspace(device, nbytes):
    ws = _WORKSPACE.get(_ws_key(device))
    if ws is None or ws.numel() < nbytes:
        # (zeroed once: the kernel leaves its counters at zero)
        ws = _WORKSPACE[_ws_key(device)] = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device.torch)
    return ws


def status_word(device):
    """The int32 the kernels write an error code to (0: none)."""
    st = _STATUS.get(device.id)
    if st is None:
        st = _STATUS[device.id] = torch.zeros(1, dtype=torch.int32, device=device.torch)
    return st


def check_status(device):
    """Synchronise and raise if a kernel of this device reported an error (a bounded wait that gave up)."""
    code = int(status_word(device).item())
    if code:
        status_word(device).zero_()
        for key in [k for k in _WORKSPACE if k[0] == device.id]:
            _WORKSPACE.pop(key)  # their counters may be mid-count
        raise _tkd.TkdError(code, "a kernel reported")


def _describe(x, m, entries, epi, act, scale, scale_up, scale_dt, residual, res_dt, y, topk, ks, max_ctas):
    """The TkdMatmul of one row slice, without the activation, output and residual addresses."""
    a = _tkd.TkdMatmul()
    w0 = entries[0][0]
    a.fmt, a.m, a.k = w0.fmt, m, w0.k
    a.ldx = x.shape[-1]
    a.nblocks, a.epilogue, a.act = len(entries), epi, act
    for i, (g, u, c0) in enumerate(entries):
        b = a.block[i]
        b.w, b.emax = g.t.data_ptr(), (g.emax.data_ptr() if g.emax is not None else None)
        if u is not None:
            b.w_up, b.emax_up = u.t.data_ptr(), (u.emax.data_ptr() if u.emax is not None else None)
        b.n, b.out_col0 = g.n, c0
    a.scale_dtype = scale_dt
    a.scale = scale.data_ptr() if scale is not None else None
    a.scale_up = scale_up.data_ptr() if scale_up is not None else None
    a.residual_dtype = res_dt
    a.ldr = residual.shape[-1] if residual is not None else 0
    a.out_dtype = _tkd.DT_F32 if epi == _tkd.EPI_OUT32 else _tkd.DT_BF16
    a.ldo = y.shape[-1]
    if topk is not None:
        a.records = _raw(topk["r"]).data_ptr()
        a.topk_k, a.topk_rows, a.topk_unit = topk["k"], topk["rows"], TOPK_UNIT
        a.topk_slot0, a.topk_write_y = topk["slot0"], int(bool(topk.get("write_y", False)))
        a.topk_base, a.topk_n = topk["base"], topk["n"]
    a.ks, a.max_ctas = ks, max_ctas
    return a


def _plan_of(a):
    p = _tkd.TkdPlan()
    _tkd.check(_tkd.lib().tkd_matmul_plan(ctypes.byref(a), ctypes.byref(p)), "tkd_matmul_plan")
    return p


def plan(device, x, w, cores_per_bank=3, full_sync=False, kb=None, kw=None, sbw=None, split=False, mt=None, rows=False,
         budget=None, xs=False, noscale=False, glu=False, glu2=False, out32=False, blocks=None, max_banks=None, m=None,
         ks=None, max_ctas=None):
    """The work split of one row slice (at most 32 rows; default: x's first slice), as a dict: the reference's keys
    where they mean something here (MT, KT, NT, KW, SEGS, glu, glu2, out32, noscale, work, l1) and the kernel's own
    (KS: k per slice, SLICES, PANELS of 128 columns, ITEMS = PANELS x SLICES, GRID: CTAs, STAGES of the shared-memory
    ring, BYTES: the weight stream read). work: [(cta, (first item, items))], the contiguous run of items each CTA
    takes. (linear.py:187-382; the Tensix options are accepted and ignored)"""
    blocks = tuple(blocks) if blocks else (w,)
    if len(blocks) > 1:
        assert 2 <= len(blocks) <= 4, f"dense_reader: {len(blocks)} blocks (at most 4)"
        assert noscale and not out32 and (glu2 or not glu), (
            "dense_reader: a block list streams x (up to 32 rows) with unit-scale weights, plain or (gate, up) pairs"
        )
        assert len({(b.k, b.dtype) for b in blocks}) == 1, "dense_reader: blocks of one K, dtype and bank count"
    assert not glu2 or glu, "dense_reader: glu2 needs glu"
    assert not (out32 and (glu or not noscale)), "dense_reader: out32 needs unit scales, no GLU stage"
    assert native_tile(w), f"dense_reader: weights are bfloat8_b, bfloat4_b or bfloat16, not {w.dtype}"
    K, N = w.shape[-2], w.shape[-1]
    assert K % TILE == 0 and x.shape[-1] == K, (x.shape, w.shape)
    if kb is not None and (K // TILE) % kb:
        raise ValueError(f"dense_reader: kb {kb} does not divide K's {K // TILE} tiles")
    rows_ = m or min(32, x.shape[-2])
    a = _tkd.TkdMatmul()
    a.fmt, a.m, a.k, a.nblocks = w.fmt, rows_, K, len(blocks)
    a.epilogue = _tkd.EPI_GLU2 if glu2 else (_tkd.EPI_GLU_IL if glu else (_tkd.EPI_OUT32 if out32 else _tkd.EPI_PLAIN))
    a.out_dtype = _tkd.DT_F32 if out32 else _tkd.DT_BF16
    for i, b in enumerate(blocks):
        a.block[i].n = b.n
    a.ks, a.max_ctas = ks or KS or 0, max_ctas or MAX_CTAS or 0
    p = _plan_of(a)
    work = [(c, (p.items * c // p.grid, p.items * (c + 1) // p.grid - p.items * c // p.grid)) for c in range(p.grid)]
    return {
        "MT": -(-rows_ // TILE), "KT": K // TILE, "NT": -(-N // TILE), "KW": p.chunk_k // TILE, "KS": p.ks,
        "SLICES": p.nslices, "PANELS": p.panels, "ITEMS": p.items, "GRID": p.grid, "STAGES": p.stages,
        "BYTES": p.weight_bytes, "SEGS": len(blocks), "glu": glu, "glu2": glu2, "out32": out32, "noscale": noscale,
        "native": native_tile(w), "work": work, "l1": p.smem_bytes,
    }


_PLAN_ARGS = set(plan.__code__.co_varnames[: plan.__code__.co_argcount])


def choose(device, x, w, full_sync=False, **forced):
    """[(first row, plan)] for x's rows, cached by shapes and settings. (linear.py:455-495)"""
    blocks = forced.get("blocks")
    shapes = tuple((b.k, b.n, b.dtype, b.fmt) for b in (blocks or (w,)))
    key = (shapes, tuple(x.shape), tuple(sorted((k, v) for k, v in forced.items() if k != "blocks")), KS, MAX_CTAS)
    got = _CHOICE.get(key)
    if got is None:
        known = {k: v for k, v in forced.items() if k in _PLAN_ARGS}
        got = _CHOICE[key] = [(m0, plan(device, x, w, full_sync=full_sync, m=mr, **known)) for m0, mr in row_slices(x)]
        if LOG:
            p0 = got[0][1]
            print(f"dense_reader: K {w.shape[-2]} N {'+'.join(str(s[1]) for s in shapes)} rows {x.shape[-2]}: plan ctas"
                  f" {p0['GRID']} SEGS {p0['SEGS']} KS {p0['KS']} slices {p0['SLICES']} items {p0['ITEMS']} stages"
                  f" {p0['STAGES']} smem {p0['l1']}", flush=True)
    return got


def is_block_list(w):
    """True for matmul's block list [(w | (gate, up), col0_tiles), ...]: a list or tuple of 2 to 4 entries, each a
    (weight or (gate, up), int col0_tiles) pair; False for one weight and for linear's (gate, up) pair.
    (linear.py:520-530)"""
    if not isinstance(w, (list, tuple)) or not 2 <= len(w) <= 4:
        return False
    return all(isinstance(e, (list, tuple)) and len(e) == 2 and type(e[1]) is int for e in w)


def block_entries(w):
    """A block list as [(gate, up or None, col0_tiles)], checked: two to four entries, all plain weights or all
    pairs, of one K, dtype and bank count. (linear.py:533-556)"""
    def split(entry):
        ok = isinstance(entry, (list, tuple)) and len(entry) == 2
        assert ok, f"dense_reader: a block is (weight, col0_tiles): {entry!r}"
        weight, col0_tiles = entry
        assert type(col0_tiles) is int and col0_tiles >= 0, f"dense_reader: col0_tiles {col0_tiles!r}"
        if not isinstance(weight, (list, tuple)):
            return weight, None, col0_tiles
        gate, up = weight
        alike = (up.dtype, tuple(up.padded_shape), str(up.memory_config())) == (
            gate.dtype, tuple(gate.padded_shape), str(gate.memory_config()))
        assert alike, "dense_reader: gate and up differ"
        return gate, up, col0_tiles

    entries = [split(e) for e in w]
    assert len(entries) in (2, 3, 4), f"dense_reader: {len(entries)} blocks (2 to 4; one weight goes in on its own)"
    pairs = [up is not None for _, up, _ in entries]
    assert all(pairs) or not any(pairs), "dense_reader: blocks all plain or all (gate, up) pairs"
    for gate, _, _ in entries:
        assert is_dram_sharded(gate), "dense_reader: blocks are DRAM-sharded"
    first = entries[0][0]
    same = all((g.shape[-2], g.dtype, g.memory_config().shard_spec.num_cores())
               == (first.shape[-2], first.dtype, first.memory_config().shard_spec.num_cores()) for g, _, _ in entries)
    assert same, "dense_reader: blocks of one K, dtype, bank count, shard grid and orientation"
    return entries


def _one_stream_format(entries):
    """The entries of one launch with all their weights in one stream format. They are (one dtype), unless some are
    "wide" (held as a bf16 stream, see ttnn_like.Weight): then the others' values are streamed as bf16 too (a twin kept
    with the weight). Such a list's sums are those of bf16 weights, not bit for bit the block-float kernels'."""
    ws = [t for g, u, _ in entries for t in (g, u) if t is not None]
    if len({t.fmt for t in ws}) == 1:
        return entries
    return [(ttnn.as_bf16_stream(g), None if u is None else ttnn.as_bf16_stream(u), c0) for g, u, c0 in entries]


def choose_blocks(device, x, w, full_sync=False, **forced):
    """choose for a block list: the plan of its one call. (linear.py:559-562)"""
    entries = _one_stream_format(block_entries(w))
    return choose(device, x, entries[0][0], full_sync, blocks=tuple(g for g, _, _ in entries), noscale=True,
                  glu=entries[0][1] is not None, glu2=entries[0][1] is not None, **forced)


def _block_kw_check(device, x, entries, full_sync, opts, slices):
    """BlockListMismatch unless every block's own call cuts K as the list's one call does. (linear.py:504-517)"""
    single = {k: v for k, v in opts.items() if k != "blocks"}
    own = [choose(device, x, g, full_sync, **single)[0][1]["KS"] for g, _, _ in entries]
    ks = slices[0][1]["KS"]
    if any(k != ks for k in own):
        raise BlockListMismatch(f"dense_reader: block list refused: its KS {ks}, the blocks' own calls' KS {own}")


# --- the op -----------------------------------------------------------------------------------------------------------


def matmul(x, w, scale, *, memory_config=None, fidelity="hifi2", full_sync=False, topk=None, out=None, col0=0, w_up=None,
           max_banks=None, **opts):
    """y = x @ w (* scale) on the device: x [1, 1, M, K] bf16, w a [1, 1, K, N] bfloat8_b, bfloat4_b or bfloat16 weight
    (native_weight), scale [1, 1, 1, N] bf16 (scale_tensor) or None. Returns [1, 1, M, N] bf16. (linear.py:568-744)

    topk (M <= 32): {"r": result tensor (topk_result), "k", "rows" (<= 16, rows * k <= 64), "slot0": first record,
    "base": index of output element 0, "n": valid output elements, "write_y": bool}: one record per TOPK_UNIT output
    columns, record slot0 + unit, holds the best k (key, index) of each of the first `rows` rows among the unit's
    columns below n: keys[rows][k] then indices[rows][k], uint32, key descending and index ascending among equal keys;
    y is written only with write_y. out: a tensor to write into instead of a new one; col0 (with out, no topk): output
    column tile c goes to tile c + col0 of a wider out.

    opts: glu (scale None): w is interleave_glu's [gate | up], the output act(gate) * up, N / 2 wide; glu_act 0 silu, 1
    gelu_tanh; w_up: the up weight apart (w the gate's), the output N wide; residual ([1, 1, M, N] bf16, scale None, no
    GLU or top-k): y = bf16(x @ w + residual), out may be the residual itself; residual_mode "epilogue" | "preload" (one
    sum here: the residual is added to the finished K sum in fp32); out32: y in float32. The Tensix options
    (cores_per_bank, split, rows, xs, kb, kw, sbw, full_sync, fidelity, memory_config) are accepted and steer nothing.
    Extensions: exchange= (a sharded.Exchange): the output and the records, where they lie inside the exchange's
    buffer, are also written to every other rank's buffer, and the call completes when all ranks' have arrived.
    col_scales=(gate scales, up scales) float32 [N] each with w_up (or one float32 vector in the
    interleaved weight's column order with glu); a float32 residual with out32 (y = x @ w + residual in float32);
    hadamard= (the sign words of ternary_matmul.t2.hadamard_signs; int4-stream weights only): x is rotated by the block
    Hadamard inside the kernel first.

    A block list in place of w, [(w | (gate, up), col0_tiles), ...]: one launch over two to four weights of one K and
    dtype, each written at its col0_tiles (in 32-column tiles); bit for bit one call per block. More than 32 rows run
    as slices of 32, each reading the weights once."""
    call_key = None
    if CACHE:
        # The same call again (the same tensor objects and options): everything was checked and described the first
        # time; only the addresses are looked at again. The entry keeps its arguments alive, so their ids stay theirs.
        call_key = _call_key(x, w, scale, topk, out, col0, w_up, max_banks, opts)
        hit = _CALLS.get(call_key)
        if hit is not None and hit["ws_key"][1] != WORKSPACE_SLOT:
            hit = None
        if hit is not None and _replay(hit):
            return hit["y"]
    launched = []
    device = x.device()
    unknown = set(opts) - _OPTS
    if unknown:
        raise TypeError(f"dense_reader.matmul: unknown options {sorted(unknown)}")
    opts_in = dict(opts)
    if not isinstance(w, (list, tuple)):
        check_banks(w, max_banks)
    elif is_block_list(w):
        for wt, _ in w:
            for u in wt if isinstance(wt, (list, tuple)) else (wt,):
                check_banks(u, max_banks)
    check_banks(w_up, max_banks)
    assert fidelity in FIDELITY, fidelity
    segs = ()
    if isinstance(w, (list, tuple)):
        assert is_block_list(w), "dense_reader: w is one weight or a block list [(w | (gate, up), col0_tiles), ...]"
        entries = _one_stream_format(block_entries(w))
        for what, given in (("scale", scale is not None), ("topk", topk is not None), ("col0", col0 != 0),
                            ("w_up", w_up is not None), ("residual", "residual" in opts), ("out32", bool(opts.get("out32")))):
            assert not given, (f"dense_reader: a block list takes no {what} (no scale, topk, col0, w_up, residual or out32:"
                               " each block carries its own col0_tiles)")
        assert x.shape[-2] <= 32, "dense_reader: a block list is a decode call: up to 32 rows"
        (w, w_up, col0), segs = entries[0], tuple(entries[1:])
        opts = {**opts, "blocks": tuple(g for g, _, _ in entries), **({"glu": True} if w_up is not None else {})}
    res_mode = opts.pop("residual_mode", "epilogue")
    assert res_mode in ("epilogue", "preload"), res_mode
    residual = opts.pop("residual", None)
    col_scales = opts.pop("col_scales", None)
    exchange = opts.pop("exchange", None)
    hadamard = opts.pop("hadamard", None)
    out32 = bool(opts.get("out32"))
    assert not (out32 and topk is not None), "dense_reader: out32 without top-k"
    assert not (out32 and out is not None and out.dtype != ttnn.float32), out.dtype
    assert x.dtype == ttnn.bfloat16, x.dtype
    assert x.memory_config().memory_layout == ttnn.TensorMemoryLayout.INTERLEAVED, x.memory_config()
    assert native_tile(w), f"dense_reader: weights are bfloat8_b, bfloat4_b or bfloat16, not {w.dtype}"
    glu = bool(opts.get("glu", False))
    act = opts.pop("glu_act", 0)
    assert act in (0, 1) and (act == 0 or glu), "dense_reader: glu_act (0 silu, 1 gelu_tanh) needs glu"
    assert not (glu and scale is not None), "dense_reader: glu takes weights without scales"
    assert col_scales is None or (glu and not segs), "dense_reader: col_scales go with a GLU over one weight or pair"
    if scale is not None:
        assert scale.dtype == ttnn.bfloat16 and scale.memory_config().memory_layout == ttnn.TensorMemoryLayout.INTERLEAVED
    extra = {"noscale": True} if scale is None else {}
    if max_banks is not None:
        extra["max_banks"] = max_banks
    N = w.shape[-1]
    if w_up is None:
        N = N // 2 if glu else N
    else:
        assert glu, "dense_reader: w_up is the GLU's up weight (glu=True)"
        assert (w_up.dtype, tuple(w_up.padded_shape)) == (w.dtype, tuple(w.padded_shape)), "dense_reader: gate and up differ"
        assert str(w_up.memory_config()) == str(w.memory_config()), "dense_reader: gate and up differ"
        extra["glu2"] = True
    opts = {**opts, **extra}
    M = x.shape[-2]
    if residual is not None:
        ext = out32 and residual.dtype == ttnn.float32  # (extension: a float32 residual into the float32 output)
        assert scale is None and not glu and topk is None and (ext or not out32), (
            "dense_reader: residual: unit-scale matmul only"
        )
        assert ext or residual.dtype == ttnn.bfloat16, residual.dtype
        assert residual.memory_config().memory_layout == ttnn.TensorMemoryLayout.INTERLEAVED
        wide = out is not None and tuple(residual.padded_shape) == tuple(out.padded_shape)
        assert wide or tuple(residual.padded_shape) == (1, 1, -(-M // TILE) * TILE, -(-N // TILE) * TILE), (residual.shape, N)
        # (the reference takes a fresh output or the residual itself; any other preallocated out is as safe here, and
        # with col0 the residual is as wide as out: it is read at the output's own columns)
        assert col0 == 0 or wide, "dense_reader: residual with a fresh output or in place"
    blocks_all = ((w, w_up, col0), *segs)
    ends = [(c0, -(-(g.shape[-1] // 2 if glu and u is None else g.shape[-1]) // TILE)) for g, u, c0 in blocks_all]
    if segs:
        N = max(TILE * c0 + nt * TILE for c0, nt in ends)  # the furthest block's end
    y = out
    if y is None:
        y = ttnn.allocate_tensor_on_device(ttnn.Shape([1, 1, M, N]), ttnn.float32 if out32 else ttnn.bfloat16,
                                           ttnn.TILE_LAYOUT, device, memory_config or ttnn.DRAM_MEMORY_CONFIG)
    assert segs or col0 == 0 or (out is not None and topk is None), "dense_reader: col0 needs out, no top-k"
    for c0, nt_ in ends:
        assert nt_ + c0 <= -(-y.shape[-1] // TILE), (nt_, c0, y.shape)
    if segs:
        spans = sorted(ends)
        assert all(a0 + an <= b0 for (a0, an), (b0, _) in itertools.pairwise(spans)), (
            f"dense_reader: block output spans overlap (col0_tiles, tiles): {spans}"
        )
    if topk is not None:
        assert M <= 32, "dense_reader: top-k needs one row slice"
        assert 1 <= topk["rows"] <= 16 and topk["rows"] * topk["k"] <= 64 and topk["rows"] <= M, topk
    if w_up is not None and w_up.fmt != w.fmt:
        ((w, w_up, _),) = _one_stream_format([(w, w_up, 0)])
    slices = choose(device, x, w, full_sync, **opts)
    if segs:
        _block_kw_check(device, x, blocks_all, full_sync, opts, slices)
    for m0, _ in slices:
        launched.append(_launch(x, blocks_all, scale, col_scales, y, m0, min(32, M - m0), topk, act, residual, glu,
                                out32, opts.get("ks") or KS or 0, opts.get("max_ctas") or MAX_CTAS or 0, exchange, hadamard))
    if call_key is not None and out is not None:
        # (only calls that write into a given output: a fresh output per call cannot be replayed)
        if len(_CALLS) >= _CALLS_MAX:
            _CALLS.clear()
        ws = _WORKSPACE.get(_ws_key(device))
        _CALLS[call_key] = {
            "y": y, "launches": launched, "device": device, "ws": ws, "ws_key": _ws_key(device), "exchange": exchange,
            "keep": (x, w, scale, out, w_up, topk, opts_in),
            "ptrs": (_raw(x).data_ptr(), _raw(y).data_ptr()),
            "topk": None if topk is None else tuple(sorted((k, id(v)) for k, v in topk.items())),
        }
    return y


def _call_key(x, w, scale, topk, out, col0, w_up, max_banks, opts):
    # (the entry keeps its arguments alive, so their ids stay theirs; ttnn.deallocate starts a new epoch, which retires
    # every entry made before it)
    return (ttnn.EPOCH, id(x), id(w), id(scale), id(out), id(w_up), id(topk), col0, max_banks, KS, MAX_CTAS, TOPK_UNIT, WORKSPACE_SLOT,
            tuple((k, tuple(map(id, v)) if type(v) is tuple else id(v)) for k, v in opts.items()))


def matmul_host(x_host, out_host, x, w, scale, *, topk=None, out=None, col0=0, w_up=None, max_banks=None, stream=None,
                **opts):
    """matmul for a caller whose activations and result live in host memory: x_host (pinned torch bf16 [M, K]) is
    copied into the device tensor x, the op runs, and its output `out` (required) is copied to out_host (pinned), all
    on the current stream (or `stream`, a torch.cuda.Stream) and without synchronising: one call into the library
    (tkd_matmul_host) instead of three framework calls. The other arguments are matmul's; up to 32 rows. The first call with a given set of tensors goes
    through matmul itself (which checks everything and also launches once)."""
    assert out is not None and CACHE, "dense_reader.matmul_host: needs out= and the launch cache"
    key = _call_key(x, w, scale, topk, out, col0, w_up, max_banks, opts)
    hit = _CALLS.get(key)
    if hit is None:
        if stream is None:
            matmul(x, w, scale, topk=topk, out=out, col0=col0, w_up=w_up, max_banks=max_banks, **opts)
        else:
            with torch.cuda.stream(stream):
                matmul(x, w, scale, topk=topk, out=out, col0=col0, w_up=w_up, max_banks=max_banks, **opts)
        hit = _CALLS[key]
    assert len(hit["launches"]) == 1, "dense_reader.matmul_host: one launch (up to 32 rows)"
    assert hit["exchange"] is None or hit["exchange"].side is None, (
        "dense_reader.matmul_host: the result is copied out by the same call, so an exchange must complete inside the kernel")
    sp = torch.cuda.current_stream().cuda_stream if stream is None else stream.cuda_stream
    rc = _tkd.lib().tkd_matmul_host(ctypes.byref(hit["launches"][0]), x_host.data_ptr(), out_host.data_ptr(), sp)
    if rc:
        _tkd.check(rc, "tkd_matmul_host")
    return out


def _replay(hit):
    """Launch a cached call again; False when something under it has moved (then the full path runs)."""
    x, _, _, _, _, topk, _ = hit["keep"]
    device = hit["device"]
    if (_raw(x).data_ptr(), _raw(hit["y"]).data_ptr()) != hit["ptrs"] or _WORKSPACE.get(hit["ws_key"]) is not hit["ws"]:
        return False
    if torch.cuda.current_device() != device.id:
        return False
    if topk is not None and tuple(sorted((k, id(v)) for k, v in topk.items())) != hit["topk"]:
        return False
    fn = _tkd.lib().tkd_matmul
    stream = torch.cuda.current_stream().cuda_stream
    for a in hit["launches"]:
        rc = fn(ctypes.byref(a), stream)
        if rc:
            _tkd.check(rc, "tkd_matmul")
        if hit["exchange"] is not None:
            hit["exchange"].after_launch(status_word(device))
    return True


def _launch(x, entries, scale, col_scales, y, m0, m, topk, act, residual, glu, out32, ks=0, max_ctas=0, exchange=None,
            hadamard=None):
    """One launch of the stream kernel: rows m0 .. m0 + m of x into the same rows of y. The descriptor is cached by
    everything that shapes it; a hit only rewrites the activation, output and residual addresses.
    (linear.py:828-1070)"""
    device = x.device()
    w, w_up, _ = entries[0]
    two = w_up is not None
    if glu:
        epi = _tkd.EPI_GLU2 if two else _tkd.EPI_GLU_IL
    elif residual is not None and not out32:
        epi = _tkd.EPI_RESIDUAL
    else:
        epi = _tkd.EPI_OUT32 if out32 else _tkd.EPI_PLAIN
    sc = sc_up = None
    scale_dt = _tkd.DT_NONE
    if scale is not None:
        sc, scale_dt = _raw(scale).reshape(-1), _tkd.DT_BF16
    elif col_scales is not None:
        parts = col_scales if two else (col_scales, None)
        sc = _raw(parts[0]).reshape(-1)
        sc_up = _raw(parts[1]).reshape(-1) if two else None
        assert sc.dtype == torch.float32 and sc.is_cuda and sc.numel() >= w.n, "dense_reader: col_scales: float32 [N] on the device"
        scale_dt = _tkd.DT_F32
    res_dt = _tkd.DT_NONE if residual is None else (_tkd.DT_F32 if residual.dtype == ttnn.float32 else _tkd.DT_BF16)
    xt, yt = _raw(x), _raw(y)
    rt = _raw(residual) if residual is not None else None
    key = None
    if CACHE:
        tk = None if topk is None else (_raw(topk["r"]).data_ptr(), topk["k"], topk["rows"], topk["slot0"], topk["base"],
                                        topk["n"], bool(topk.get("write_y", False)), TOPK_UNIT)
        key = (
            # (weights by their serial numbers, never by address: a freed weight's memory may come back as another
            # weight's stream, a serial does not come back)
            ttnn.EPOCH, tuple((g.serial, u.serial if u is not None else 0, c0) for g, u, c0 in entries),
            m, tuple(xt.shape), tuple(yt.shape), epi, act, sc.data_ptr() if sc is not None else 0,
            sc_up.data_ptr() if sc_up is not None else 0, scale_dt, res_dt, tk, ks, max_ctas, device.id, id(exchange),
            _raw(hadamard).data_ptr() if hadamard is not None else 0,
        )
    hit = _LAUNCHES.get(key) if key is not None else None
    if hit is None:
        blocks = [(g, u, c0 * TILE) for g, u, c0 in entries]
        a = _describe(xt, m, blocks, epi, act, sc, sc_up, scale_dt, rt, res_dt, yt, topk, ks, max_ctas)
        need = ctypes.c_uint64(0)
        _tkd.check(_tkd.lib().tkd_matmul_workspace(ctypes.byref(a), ctypes.byref(need)), "tkd_matmul_workspace")
        a.hadamard = _raw(hadamard).data_ptr() if hadamard is not None else None
        hit = (a, need.value, (sc, sc_up, exchange, hadamard))
        if key is not None:
            _LAUNCHES[key] = hit
    a, need, _ = hit
    ws = _workspace(device, need)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.status = status_word(device).data_ptr()
    esz_x, esz_y = xt.element_size(), yt.element_size()
    a.x = xt.data_ptr() + m0 * xt.shape[-1] * esz_x
    a.out = yt.data_ptr() + m0 * yt.shape[-1] * esz_y
    a.residual = rt.data_ptr() + m0 * rt.shape[-1] * rt.element_size() if rt is not None else None
    if exchange is not None:
        exchange.fill(a, a.out, a.records)
    with torch.cuda.device(device.torch):
        _tkd.check(_tkd.lib().tkd_matmul(ctypes.byref(a), torch.cuda.current_stream().cuda_stream), "tkd_matmul")
        if exchange is not None:
            exchange.after_launch(status_word(device))
    done = _tkd.TkdMatmul()
    ctypes.pointer(done)[0] = a  # (a copy: the cached descriptor is rewritten by the next row slice or call)
    return done


# --- top-k records ----------------------------------------------------------------------------------------------------


def topk_records(r, rows, k):
    """The records of a top-k result tensor on the host: (values [rows, records * k] float32, indices [rows,
    records * k] int64); empty slots hold -inf and -1. (linear.py:747-750)"""
    return records_host(ttnn.to_torch(r), rows, k)


def records_host(t, rows, k):
    """topk_records on a host copy of the result tensor (int32 words, or the same bytes as bfloat16). A key is a bf16
    as a monotone 16-bit code (positive: bits | 0x8000; negative: ~bits), 0 an empty slot. (linear.py:753-768)"""
    words = t.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    words = words.reshape(-1, 2, rows, k)
    keys = words[:, 0].transpose(0, 1).reshape(rows, -1)
    idx = words[:, 1].transpose(0, 1).reshape(rows, -1)
    positive = keys >= 0x8000
    bits = torch.where(positive, keys - 0x8000, 0xFFFF - keys)
    vals = bits << 16
    vals = torch.where(vals >= 1 << 31, vals - (1 << 32), vals).to(torch.int32).view(torch.float32)
    empty = keys == 0
    vals = vals.masked_fill(empty, float("-inf"))
    idx = idx.masked_fill(empty | (idx == 0xFFFFFFFF), -1)
    return vals, idx


def topk_result(device, records, rows, k):
    """A result tensor for `records` top-k records of rows x k, zeroed (every slot empty): [1, 1, records, 2 * rows * k]
    uint32, or with RECORDS_BF16 the same bytes as [1, 1, records, 4 * rows * k] bfloat16. (linear.py:771-785)"""
    if RECORDS_BF16:
        return ttnn.from_torch(torch.zeros(1, 1, records, 4 * rows * k, dtype=torch.bfloat16), dtype=ttnn.bfloat16,
                               layout=ttnn.ROW_MAJOR_LAYOUT, device=device, memory_config=ttnn.DRAM_MEMORY_CONFIG)
    return ttnn.from_torch(torch.zeros(1, 1, records, 2 * rows * k, dtype=torch.int32), dtype=ttnn.uint32,
                           layout=ttnn.ROW_MAJOR_LAYOUT, device=device, memory_config=ttnn.DRAM_MEMORY_CONFIG)


def topk_merge(records, rows, k, top, out=None):
    """The best `top` candidates of every row among all the records of a result tensor (topk_result's layout; any
    number of records, e.g. every rank's after an exchange), on the device: value descending, lower index first among
    equal values. Returns a result tensor of one record of rows x top (topk_records / records_host decode it); out: a
    tensor to write into. The counterpart of `vh.topk(top)` in the reference's collect (lm_head_topk/lmhead.py:212-239),
    with the tie order made definite."""
    device = records.device()
    nrec = _raw(records).numel() * _raw(records).element_size() // (8 * rows * k)
    if out is None:
        out = topk_result(device, 1, rows, top)
    with torch.cuda.device(device.torch):
        _tkd.check(_tkd.lib().tkd_topk_merge(_raw(records).data_ptr(), nrec, rows, k, top, _raw(out).data_ptr(),
                                             torch.cuda.current_stream().cuda_stream), "tkd_topk_merge")
    return out


def topk_units(n):
    """Records a call over n output columns writes: one per TOPK_UNIT columns."""
    return -(-(-(-n // 128) * 128) // TOPK_UNIT)


# --- any rank ---------------------------------------------------------------------------------------------------------


def linear(x, w, scale, memory_config=None, activation=None, out_dtype=None, **opts):
    """matmul for x of any rank: x [..., rows, K] bf16, the output's rank the input's. activation: None, "silu"
    (applied after the matmul), "swiglu" or "geglu" (w is interleave_glu's weight with scale None, the output N / 2
    wide; or w is (gate, up), the output N wide). out_dtype ttnn.float32: out32. A block list for w: plain weights with
    activation None, (gate, up) pairs with "swiglu" or "geglu". opts go to matmul. (linear.py:1073-1124)"""
    shape = list(x.shape)
    glu_kinds = {"swiglu": 0, "geglu": 1}
    if out_dtype not in (None, ttnn.bfloat16):
        assert out_dtype == ttnn.float32, f"dense_reader.linear: out_dtype {out_dtype}"
        opts = {**opts, "out32": True}
    blocks = is_block_list(w)
    if blocks:
        pairs = isinstance(w[0][0], (tuple, list))
        assert activation != "silu", "dense_reader.linear: no silu after a block list"
        allowed = tuple(glu_kinds) if pairs else (None,)
        assert activation in allowed, (
            f"dense_reader.linear: a block list of {'(gate, up) pairs' if pairs else 'plain weights'} takes activation"
            f" {' or '.join(map(repr, allowed))}, not {activation!r}"
        )
        if glu_kinds.get(activation):
            opts = {**opts, "glu_act": 1}
        n = max(TILE * c0 + (wt[0] if pairs else wt).shape[-1] for wt, c0 in w)
    else:
        if isinstance(w, (tuple, list)):
            assert activation in glu_kinds, "dense_reader.linear: two weights are the GLU's gate and up"
            w, opts = w[0], {**opts, "w_up": w[1]}
        n = w.shape[-1]
        if activation in glu_kinds:
            opts = {**opts, "glu": True, **({"glu_act": 1} if glu_kinds[activation] else {})}
            if opts.get("w_up") is None:
                n //= 2
    x4 = x if len(shape) == 4 else ttnn.reshape(x, [1, 1, shape[-2], shape[-1]])
    if x4.memory_config().memory_layout != ttnn.TensorMemoryLayout.INTERLEAVED:
        x4 = ttnn.sharded_to_interleaved(x4, ttnn.L1_MEMORY_CONFIG)
    y = matmul(x4, w, scale, memory_config=memory_config, **opts)
    if activation is not None and activation not in ("swiglu", "geglu"):
        assert activation == "silu", f"dense_reader.linear: activation {activation!r}"
        y = ttnn.silu(y)
    if len(shape) != 4 and opts.get("out") is None:
        y = ttnn.reshape(y, [*shape[:-1], n])
    return y
