"""head_pick.py: the top-k LM head's exact rescore and pick on the GPU (the reference's lm_head_topk/head_pick.py, same
names and arguments).

lmhead.DeviceHead's device part leaves, per row, every block's top-k candidates in a result tensor (linear.matmul's
topk records). pick() takes the best `top` of them by the device's logit, recomputes their logits from the bf16 head
rows (bf16 x times bf16 rows, float32 sums, rounded to bf16 unless logits="float32") and picks the largest (lowest id on
ties, a NaN counting as the largest), one CTA a row in one launch (tkd_head_pick). pick_records() is the pick without a
rescore, for a draft head, with an optional token map (tkd_head_pick_records). Both write a [1, 1, 32, 32] uint32 page:
row r = [token, the device's own best candidate, the count, 0 ...]; tokens() reads it.

The reference's four Tensix kernels (kernels/head_pick_reader.cpp, _compute.cpp, _writer.cpp, _records.cpp) are the two
instantiations of one CUDA kernel here (csrc/tkd_topk.cu).
"""

import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from common import ttnn_like as ttnn  # noqa: E402
from dense_reader import _tkd  # noqa: E402

TILE = 32


def _stream():
    return torch.cuda.current_stream().cuda_stream


def head_rows(device, weight):
    """The bf16 head [vocab, dim] (torch) as a row-major device tensor [1, 1, vocab, dim]. (head_pick.py:44-54)"""
    table = weight.to(torch.bfloat16)[None, None]
    return ttnn.from_torch(table, dtype=ttnn.bfloat16, layout=ttnn.ROW_MAJOR_LAYOUT, device=device,
                           memory_config=ttnn.DRAM_MEMORY_CONFIG)


def check_rows(rows_t, dim, vocab=None):
    """A bf16 head table pick can gather from: row-major bf16 [rows, dim] or [1, 1, rows, dim] in device memory, with at
    least `vocab` rows when that is given. (head_pick.py:57-73)"""
    *lead, nrows, width = tuple(rows_t.shape)
    mc = rows_t.memory_config()
    problems = [
        what for what, bad in (
            ("dtype bfloat16", rows_t.dtype != ttnn.bfloat16),
            ("row-major layout", rows_t.layout != ttnn.ROW_MAJOR_LAYOUT),
            ("interleaved device memory", mc.memory_layout != ttnn.TensorMemoryLayout.INTERLEAVED
             or mc.buffer_type != ttnn.BufferType.DRAM),
            ("leading dimensions of 1", any(d != 1 for d in lead)),
            (f"rows of {dim}", width != dim),
            (f"at least {vocab} rows", vocab is not None and nrows < vocab),
        ) if bad
    ]
    assert not problems, f"head_pick: the head table needs {', '.join(problems)}: {tuple(rows_t.shape)} {rows_t.dtype} {mc}"


def check_ids_out(t):
    """ids_out: a one-element uint32 row-major device tensor (an embedding's index for a draft's next step).
    (head_pick.py:76-91)"""
    n = 1
    for d in t.shape:
        n *= d
    mc = t.memory_config()
    assert (t.dtype == ttnn.uint32 and t.layout == ttnn.ROW_MAJOR_LAYOUT and n == 1
            and mc.memory_layout == ttnn.TensorMemoryLayout.INTERLEAVED and mc.buffer_type == ttnn.BufferType.DRAM), (
        tuple(t.shape), t.dtype, t.layout, str(mc))


def _out_page(device):
    return ttnn.allocate_tensor_on_device(ttnn.Shape([1, 1, TILE, TILE]), ttnn.uint32, ttnn.ROW_MAJOR_LAYOUT, device,
                                          ttnn.DRAM_MEMORY_CONFIG)


def _record_count(records, nrows, k):
    page = 2 * nrows * k * 4
    assert page % 32 == 0, (nrows, k)  # (the reference's 32-byte record alignment, kept as an argument check)
    assert records.shape[-1] * (2 if records.dtype == ttnn.bfloat16 else 4) == page, (records.shape, nrows, k)
    return records.shape[-2]


def pick(records, x, rows_t, nrows, k, top=16, logits="bf16", out=None, valid=None, ids_out=None):
    """Token ids for the first nrows rows of x [1, 1, >= nrows, dim] bf16: per row the best `top` candidates of the top-k
    result `records` (linear.topk_result's, made for nrows rows and k), rescored with the bf16 rows of rows_t and picked.
    out: [1, 1, 32, 32] uint32 row-major (made here unless given); row r = [token, the device's own best candidate, the
    valid count, 0 ...]. valid: a padded head's real vocabulary (ids at or past it are empty slots; default the table's
    rows). A row with no valid candidate gets token 0 and count 0. ids_out: also row 0's token into this one-element
    uint32 tensor. (head_pick.py:101-220)"""
    assert logits in ("bf16", "float32"), logits
    assert 1 <= top <= 32 and 1 <= nrows <= TILE, (top, nrows)
    device = x.device()
    dim = x.shape[-1]
    assert dim % TILE == 0, dim
    assert x.dtype == ttnn.bfloat16 and nrows <= x.shape[-2], (x.dtype, x.shape, nrows)
    check_rows(rows_t, dim)
    nrec = _record_count(records, nrows, k)
    vocab = rows_t.shape[-2] if valid is None else int(valid)
    assert 1 <= vocab <= rows_t.shape[-2], (valid, rows_t.shape)
    if out is None:
        out = _out_page(device)
    if ids_out is not None:
        check_ids_out(ids_out)
    with torch.cuda.device(device.torch):
        _tkd.check(_tkd.lib().tkd_head_pick(
            records.t.data_ptr(), nrec, nrows, k, top, vocab, x.t.data_ptr(), x.t.shape[-1], dim, rows_t.t.data_ptr(),
            rows_t.t.shape[-1], int(logits == "bf16"), out.t.data_ptr(), ids_out.t.data_ptr() if ids_out is not None else None,
            _stream()), "tkd_head_pick")
    return out


def token_map(device, ids):
    """A sub-head's token map for pick_records: row i of the sub-head is token ids[i] (below 2**31). [1, 1, ceil(n / 32),
    32] uint32 row-major, the tail past n zero. (head_pick.py:223-240)"""
    ids = torch.as_tensor(ids, dtype=torch.int64).reshape(-1)
    n = ids.numel()
    assert n >= 1 and int(ids.min()) >= 0 and int(ids.max()) < 1 << 31, (n, ids.min(), ids.max())
    pages = -(-n // TILE)
    t = torch.zeros(pages * TILE, dtype=torch.int32)
    t[:n] = ids.to(torch.int32)
    return ttnn.from_torch(t.reshape(1, 1, pages, TILE), dtype=ttnn.uint32, layout=ttnn.ROW_MAJOR_LAYOUT, device=device,
                           memory_config=ttnn.DRAM_MEMORY_CONFIG)


def pick_records(records, nrows, k, vocab, tmap=None, out=None, ids_out=None):
    """Token ids for the first nrows rows of a top-k result with no rescore: per row the best record slot by the device's
    logit (the first of equal keys, record by record and slot by slot; a NaN counts as the largest), its id mapped
    through tmap (token_map's; None: the id itself). vocab: the head's rows that count (a slot of id at or past it is
    empty). out row r = [token, the best id, the valid slots' count, 0 ...]; no valid slot: token 0, id 0xFFFFFFFF, count
    0. (head_pick.py:243-335)"""
    assert 1 <= nrows <= TILE and k >= 1, (nrows, k)
    device = records.device()
    nrec = _record_count(records, nrows, k)
    vocab = int(vocab)
    assert 1 <= vocab < 1 << 32, vocab
    if tmap is not None:
        mc = tmap.memory_config()
        assert (tmap.dtype == ttnn.uint32 and tmap.layout == ttnn.ROW_MAJOR_LAYOUT and tmap.shape[-1] == TILE
                and mc.memory_layout == ttnn.TensorMemoryLayout.INTERLEAVED and mc.buffer_type == ttnn.BufferType.DRAM
                and tmap.shape[-2] * TILE >= vocab), (tuple(tmap.shape), tmap.dtype, tmap.layout, str(mc), vocab)
    if out is None:
        out = _out_page(device)
    if ids_out is not None:
        check_ids_out(ids_out)
    with torch.cuda.device(device.torch):
        _tkd.check(_tkd.lib().tkd_head_pick_records(
            records.t.data_ptr(), nrec, nrows, k, vocab, tmap.t.data_ptr() if tmap is not None else None, out.t.data_ptr(),
            ids_out.t.data_ptr() if ids_out is not None else None, _stream()), "tkd_head_pick_records")
    return out


def tokens(out, nrows):
    """The host's read of pick's output: (tokens [nrows], the device's own best [nrows], valid counts [nrows]).
    (head_pick.py:331-335)"""
    t = ttnn.to_torch(out).reshape(32, 32)[:nrows].to(torch.int64) & 0xFFFFFFFF
    return t[:, 0], t[:, 1], t[:, 2]
