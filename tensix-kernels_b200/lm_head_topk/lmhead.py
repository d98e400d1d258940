"""lmhead.py: an LM head on the GPU that returns token ids, not logits (the reference's lm_head_topk/lmhead.py, same
names, arguments and results).

The vocabulary is cut into `chunks` column blocks of the [dim, vocab] weight; each block is one dense-reader call
(linear.matmul with block-float weights) for up to 16 rows at a time that writes no logits: the kernel's output warps
keep the best `k` of each row per 2048-column unit (linear.matmul's topk) as one small record, so one small tensor
holds every block's candidates. With `rescore` (the default) the candidates' logits are recomputed exactly from the bf16
weight rows and the largest is picked, the lowest token id first on ties and a NaN counting as the largest
(pick_token): on the host (collect), or with device_pick=True on the GPU (head_pick.py), which then reads back only the
token ids. Without a rescore, device_pick=True is the records-only pick with an optional token map (a draft head).

  head = DeviceHead(device, lm_head_weight, fmt="bfp4")                     # [vocab, dim] torch
  ids = head(x, rows)                                                       # x [1, 1, >= rows, dim] on the device
  head = DeviceHead(device, lm_head_weight, device_pick=True)               # rescore and pick on the device
  head = DeviceHead(device, sub_weight, rescore=False, device_pick=True, token_map=ids)   # a draft sub-head
"""

import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from common import ttnn_like as ttnn  # noqa: E402
from dense_reader import linear  # noqa: E402
from lm_head_topk import head_pick  # noqa: E402

FORMATS = {"bfp8": ttnn.bfloat8_b, "bfp4": ttnn.bfloat4_b, "bf16": ttnn.bfloat16}


def pick_token(exact, ids, vocab):
    """The argmax over the rescored candidates: per row the lowest token id among the largest exact logits, a NaN
    counting as the largest. exact: [rows, c] float with -inf for empty slots, ids: [rows, c]. (lmhead.py:40-46)"""
    rank = torch.nan_to_num(exact, nan=float("inf"), posinf=torch.finfo(exact.dtype).max)  # NaN above +inf above the rest
    winners = rank == rank.amax(dim=1, keepdim=True)
    return ids.masked_fill(~winners, vocab).amin(dim=1)


class DeviceHead:
    """The LM head as `chunks` device matmuls with top-k records. (lmhead.py:49-263)"""

    def __init__(self, device, weight, fmt="bfp4", chunks=16, k=8, rescore=True, top=16, blocks=None, logits="bf16",
                 device_pick=False, rows=None, valid=None, token_map=None, l1x=True, **opts):
        """weight: the head [vocab, dim] (torch; kept on the host in bf16 for a host rescore). chunks: vocabulary blocks,
        one dense-reader call each (vocab / chunks a multiple of 32). blocks: device weights already made, [(w, scale or
        None)] in vocabulary order; else made here in fmt. k: candidates per record; top: of all candidates the best
        `top` by device logit are rescored. logits: "bf16" (rounded) or "float32". device_pick: the rescore and the pick
        on the device with a bf16 copy of the head in device memory (`top` at most 32); rows: that copy when the caller
        already has it (a tied embedding table); valid: a padded head's real vocabulary. Without a rescore,
        device_pick=True is the records-only pick and token_map (a list, a tensor of ids, or head_pick.token_map's device
        tensor) maps the head's rows to token ids. l1x: accepted (the reference copies x into L1 once a call; the GPU
        reads x through its caches). opts go to linear.matmul."""
        if fmt not in FORMATS:
            raise AssertionError(f"lmhead: fmt {fmt!r} (one of {sorted(FORMATS)})")
        if logits not in ("bf16", "float32"):
            raise AssertionError(f"lmhead: logits {logits!r}")
        self.device, self.fmt, self.k, self.top, self.opts = device, fmt, k, top, opts
        self.vocab, self.dim = weight.shape
        nblocks = chunks if blocks is None else len(blocks)
        self.step, left = divmod(self.vocab, nblocks)
        assert left == 0 and self.step % 32 == 0, (self.vocab, nblocks)
        self.slots = linear.topk_units(self.step)  # records a block writes: one per unit of output columns
        self.logits, self.round, self.l1x, self.valid = logits, logits == "bf16", l1x, valid
        self.device_pick = bool(device_pick)
        self.records_pick = self.device_pick and not rescore
        # what calls keep from one to the next: result tensors and pick pages by row count, the placeholder output
        self.results, self.picks, self.y = {}, {}, None
        self.miss = 0  # rows whose best candidate by the device's logit lost the rescore
        # the three ways to turn candidates into tokens
        self.host = None                          # host rescore: the head in bf16 on the host
        self.rows_t, self.own_rows = None, False  # device rescore: the bf16 head on the device (ours to free?)
        self.tmap, self.own_tmap = None, False    # records-only pick: the optional token map (ours to free?)
        if token_map is not None:
            assert self.records_pick, "lmhead: token_map is for rescore=False, device_pick=True"
            self._take_token_map(token_map)
        if rescore:
            if self.device_pick:
                self._take_head_rows(weight, rows)
            else:
                self.host = weight.to(torch.bfloat16)
        self.blocks = list(blocks) if blocks is not None else self._pack(weight)

    def _take_token_map(self, token_map):
        if isinstance(token_map, ttnn.Tensor):
            self.tmap = token_map
            return
        assert len(token_map) == self.vocab, (len(token_map), self.vocab)
        self.tmap, self.own_tmap = head_pick.token_map(self.device, token_map), True

    def _take_head_rows(self, weight, rows):
        assert 1 <= self.top <= 32, f"lmhead: the device pick rescores at most 32 candidates, top {self.top}"
        if rows is None:
            self.rows_t, self.own_rows = head_pick.head_rows(self.device, weight), True
        else:
            head_pick.check_rows(rows, self.dim, self.valid if self.valid is not None else self.vocab)
            self.rows_t = rows

    def _pack(self, weight):
        """The head's blocks as device weights with unit scales, in vocabulary order."""
        made = []
        for first in range(0, self.vocab, self.step):
            tw, ts = linear.native_weight(self.device, weight[first : first + self.step], FORMATS[self.fmt])
            ttnn.deallocate(ts)
            made.append((tw, None))
        return made

    def _result(self, rows):
        if rows not in self.results:
            self.results[rows] = linear.topk_result(self.device, len(self.blocks) * self.slots, rows, self.k)
        return self.results[rows]

    def _placeholder(self, x):
        """The matmuls' output tensor: never written (write_y False), as tall as x."""
        if self.y is not None and self.y.shape[-2] == x.shape[-2]:
            return self.y
        if self.y is not None:
            ttnn.deallocate(self.y)
        self.y = ttnn.allocate_tensor_on_device(ttnn.Shape([1, 1, x.shape[-2], self.step]), ttnn.bfloat16, ttnn.TILE_LAYOUT,
                                                self.device, ttnn.DRAM_MEMORY_CONFIG)
        return self.y

    def logits_topk(self, x, rows=1, ids_out=None):
        """The device part: per block the matmul that keeps each unit's best k of the first `rows` rows (no logits are
        written), then with device_pick the rescore and the pick. Returns the result tensor (block b's records at
        b * slots ..). Nothing is read back and the tensors are kept from call to call, so a CUDA graph can hold it.
        (lmhead.py:135-197)"""
        assert 1 <= rows <= min(16, x.shape[-2]), f"lmhead: 1 to 16 rows, at most x's ({rows})"
        assert ids_out is None or self.rows_t is not None or self.records_pick, "lmhead: ids_out needs the device pick"
        r, y = self._result(rows), self._placeholder(x)
        for b, (tw, ts) in enumerate(self.blocks):
            linear.matmul(x, tw, ts, out=y, **self.opts,
                          topk={"r": r, "k": self.k, "rows": rows, "slot0": b * self.slots, "base": b * self.step,
                                "n": self.step, "write_y": False})
        page = self.picks.get(rows)
        if self.rows_t is not None:
            self.picks[rows] = head_pick.pick(r, x, self.rows_t, rows, self.k, top=self.top, logits=self.logits, out=page,
                                              valid=self.valid, ids_out=ids_out)
        elif self.records_pick:
            self.picks[rows] = head_pick.pick_records(r, rows, self.k, self.valid if self.valid is not None else self.vocab,
                                                      tmap=self.tmap, out=page, ids_out=ids_out)
        return r

    def candidates(self, x, rows):
        """(values [rows, c] float, global ids [rows, c] long) of the device's candidates. (lmhead.py:199-202)"""
        return linear.topk_records(self.logits_topk(x, rows), rows, self.k)

    def rescore(self, xh, ids):
        """Exact logits of the candidates: x (bf16) times the bf16 weight rows, float32 sums, rounded to bf16 unless
        logits="float32". (lmhead.py:204-209)"""
        nrows, ncand = ids.shape
        picked = self.host.index_select(0, ids.reshape(-1)).float().reshape(nrows, ncand, self.dim)
        exact = torch.bmm(picked, xh.float().reshape(nrows, self.dim, 1)).reshape(nrows, ncand)
        return exact.to(torch.bfloat16).float() if self.round else exact

    def __call__(self, x, rows=1):
        """Token ids [rows] (long) for the first `rows` rows of x [1, 1, >= rows, dim] bf16."""
        self.logits_topk(x, rows)
        return self.collect(x, rows)

    def collect(self, x, rows=1, xh=None):
        """The host part, after logits_topk ran: with a device pick the token ids read back; else the records' read-back,
        x's (or xh, a host copy of x's first rows) and the rescore. Token ids [rows] (long). (lmhead.py:216-243)"""
        if self.rows_t is not None or self.records_pick:
            tok, device_best, _ = head_pick.tokens(self.picks[rows], rows)
            if self.rows_t is not None:
                self.miss += int((device_best != tok).sum())
            return tok
        vals, ids = linear.topk_records(self.results[rows], rows, self.k)
        row = torch.arange(rows)
        if self.host is None:  # no rescore: the device's own best
            return ids[row, vals.argmax(dim=1)]
        if xh is None:
            xh = ttnn.to_torch(x)
        xh = xh.reshape(-1, self.dim)[:rows].to(torch.bfloat16)
        if self.top and self.top < ids.shape[1]:  # only the best `top` by device logit are rescored
            keep = vals.topk(self.top, dim=1).indices
            vals, ids = vals.gather(1, keep), ids.gather(1, keep)
        device_best = ids[row, vals.argmax(dim=1)]
        empty = ids < 0
        ids = ids.clamp(min=0)
        exact = self.rescore(xh, ids).masked_fill(empty, float("-inf"))
        tok = pick_token(exact, ids, self.vocab)
        self.miss += int((device_best != tok).sum())
        return tok

    def deallocate(self):
        """Free what the head holds on the device (the caller's own `rows` table and token map stay)."""
        owned = list(self.picks.values()) + list(self.results.values())
        owned += [t for pair in self.blocks for t in pair if t is not None]
        owned += [t for t, mine in ((self.tmap, self.own_tmap), (self.rows_t, self.own_rows), (self.y, True)) if t is not None and mine]
        for t in owned:
            ttnn.deallocate(t)
        self.picks, self.results, self.blocks = {}, {}, []
        self.tmap = self.rows_t = self.y = None
