# SPDX-License-Identifier: Apache-2.0
# Copyright 2026 Xylolabs
# Ported from XylolabsInc/tensix-kernels, lm_head_topk/tests/test_lm_head.py (Apache-2.0): the test cases, shapes, seeds and bars are that
# file's; the imports and the device API under them are this package's.
"""The top-k LM head (lm_head_topk/lmhead.py, head_pick.py) against torch, case for case the reference's
lm_head_topk/tests/test_lm_head.py: a random bf16 head [8192, 1024] as four bfloat4_b blocks and random x rows;
- the records hold the block matmul's own bf16 logits at their ids, and each row's best k over the records are its best
  k over all logits, bit for bit;
- the host rescore's tokens against a bf16 host head, token for token;
- the device pick against the host rescore on the same records in bf16 and float32 logits (token for token, or, where
  the sum orders part a near tie, exact logits equal to 1e-6 / one bf16 step), also on a head whose rows
  repeat in pairs (exact ties: the lowest id wins) and on a padded head (valid=), its table also the valid rows only;
- the records-only pick with and without a token map against the host's argmax over the same records;
- both picks with k 4 at 1 and 3 rows.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

from common import ttnn_like as ttnn  # noqa: E402
from common.testing import same  # noqa: E402
from dense_reader import linear  # noqa: E402
from lm_head_topk import head_pick, lmhead  # noqa: E402

VOCAB, DIM, CHUNKS = 8192, 1024, 4


def head(seed, pairs=False):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(VOCAB, DIM, generator=g) * 0.05).to(torch.bfloat16)
    if pairs:
        w[1::2] = w[0::2]  # rows 2i and 2i + 1 equal: every logit ties with its pair
    return w


def x_rows(device, rows, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, DIM, generator=g).to(torch.bfloat16)
    return x, ttnn.from_torch(x.reshape(1, 1, rows, DIM), dtype=ttnn.bfloat16, layout=ttnn.TILE_LAYOUT, device=device)


def host_tokens(x, w, logits="bf16"):
    z = x.float() @ w.float().T
    if logits == "bf16":
        z = z.to(torch.bfloat16).float()
    return lmhead.pick_token(z, torch.arange(VOCAB).expand(x.shape[0], -1), VOCAB)


def agree(what, got, want, x, w, tol=2.0 ** -7, pairs=False):
    """Tokens equal, or, where they differ, a near tie: the float32 sums behind two logits come out in another order on
    the device than in torch (whose own order varies with the host's thread count), so two candidates whose exact
    logits are within `tol` (relative; one bf16 step for rounded logits) may be picked either way. pairs: rows 2i and
    2i + 1 of the head are equal, an exact tie, and of those the lower id must have won."""
    if torch.equal(got, want):
        print(f"ok   {what}: token for token", flush=True)
        return
    z = x.double() @ w.double().T
    for t in range(got.shape[0]):
        a, b = z[t, got[t]].item(), z[t, want[t]].item()
        assert abs(a - b) <= tol * max(abs(a), abs(b)), (what, t, int(got[t]), int(want[t]), a, b)
        assert not pairs or int(got[t]) % 2 == 0, (what, t, int(got[t]))
    print(f"ok   {what}: equal up to near ties", flush=True)


def test_records(device):
    w = head(1)
    rows, k = 3, 8
    x, tx = x_rows(device, rows, 2)
    dh = lmhead.DeviceHead(device, w, fmt="bfp4", chunks=CHUNKS, k=k, rescore=False)
    vals, ids = dh.candidates(tx, rows)
    y = torch.cat([ttnn.to_torch(linear.matmul(tx, tw, None)).float().reshape(-1, dh.step)[:rows] for tw, _ in dh.blocks], 1)
    for t in range(rows):
        ok = ids[t] >= 0
        same(f"records row {t}: values at their ids", y[t][ids[t][ok]], vals[t][ok])
        top = torch.sort(vals[t][ok], descending=True).values[:k]
        same(f"records row {t}: the best {k} of all logits", top, torch.topk(y[t], k).values)
    dh.deallocate()


def test_host_rescore(device):
    w = head(3)
    dh = lmhead.DeviceHead(device, w, fmt="bfp4", chunks=CHUNKS)
    for rows in (1, 5):
        x, tx = x_rows(device, rows, 4 + rows)
        agree(f"host rescore rows {rows}: tokens against the bf16 host head", dh(tx, rows), host_tokens(x, w), x, w)
    dh.deallocate()


@pytest.mark.parametrize("kind,seed,pairs", [("random", 5, False), ("ties", 6, True)])
@pytest.mark.parametrize("logits", ["bf16", "float32"])
def test_device_pick(device, kind, seed, pairs, logits):
    w = head(seed, pairs)
    host = lmhead.DeviceHead(device, w, fmt="bfp4", chunks=CHUNKS, logits=logits)
    dev = lmhead.DeviceHead(device, w, fmt="bfp4", chunks=CHUNKS, logits=logits, device_pick=True)
    for rows in (1, 4):
        x, tx = x_rows(device, rows, 7 + rows)
        want, got = host(tx, rows), dev(tx, rows)
        agree(f"device pick ({kind}, {logits} logits) rows {rows}: tokens against the host rescore", got, want, x, w,
              1e-6 if logits == "float32" else 2.0 ** -7, pairs)
        if kind == "random" and logits == "bf16":
            agree(f"device pick rows {rows}: tokens against the bf16 host head", got, host_tokens(x, w), x, w)
    dev.deallocate()
    host.deallocate()


def test_small_records(device):
    w = head(14)
    for rows in (1, 3):
        x, tx = x_rows(device, rows, 15 + rows)
        host = lmhead.DeviceHead(device, w, fmt="bfp4", chunks=CHUNKS, k=4)
        dev = lmhead.DeviceHead(device, w, fmt="bfp4", chunks=CHUNKS, k=4, device_pick=True)
        agree(f"device pick, k 4, rows {rows}: tokens against the host rescore", dev(tx, rows), host(tx, rows), x, w)
        plain = lmhead.DeviceHead(device, w, fmt="bfp4", chunks=CHUNKS, k=4, rescore=False)
        vals, ids = plain.candidates(tx, rows)
        picked = lmhead.DeviceHead(device, w, fmt="bfp4", chunks=CHUNKS, k=4, rescore=False, device_pick=True)
        best = ids[torch.arange(rows), vals.argmax(dim=1)]
        same(f"records pick, k 4, rows {rows}: rows against the host's argmax over the records", picked(tx, rows), best)
        for h in (host, dev, plain, picked):
            h.deallocate()


def test_padded_head(device):
    w = head(9)
    valid = VOCAB - 3 * 32 - 5  # the last rows are padding: never candidates
    rows, k = 2, 8
    x, tx = x_rows(device, rows, 10)
    dh = lmhead.DeviceHead(device, w, fmt="bfp4", chunks=CHUNKS, k=k, rescore=False)
    r = dh.logits_topk(tx, rows)
    rows_t = head_pick.head_rows(device, w)
    tok, _, _ = head_pick.tokens(head_pick.pick(r, tx, rows_t, rows, k, valid=valid), rows)
    vals, ids = linear.topk_records(r, rows, k)
    vals = torch.where(ids >= valid, torch.full_like(vals, float("-inf")), vals)
    cand = ids.gather(1, vals.topk(16, dim=1).indices)
    z = torch.einsum("rd,rcd->rc", x.float(), w[cand.clamp(min=0).reshape(-1)].float().reshape(rows, 16, DIM))
    z = z.to(torch.bfloat16).float()
    z = torch.where((cand >= 0) & (cand < valid), z, torch.full_like(z, float("-inf")))
    want = lmhead.pick_token(z, cand, VOCAB)
    same(f"padded head (valid {valid}): tokens against the host rescore of the valid candidates", tok, want)
    assert int(tok.max()) < valid
    short = head_pick.head_rows(device, w[:valid])  # a table of the valid rows only serves the padded head
    dv = lmhead.DeviceHead(device, w, fmt="bfp4", chunks=CHUNKS, k=k, device_pick=True, valid=valid, rows=short)
    same(f"padded head (valid {valid}), a table of the valid rows only: tokens", dv(tx, rows), want)
    dv.deallocate()
    ttnn.deallocate(short)
    ttnn.deallocate(rows_t)
    dh.deallocate()


def test_records_pick(device):
    w = head(11)
    rows, k = 3, 8
    g = torch.Generator().manual_seed(12)
    tmap = torch.randperm(1 << 20, generator=g)[:VOCAB]  # row i of the sub-head is token tmap[i]
    x, tx = x_rows(device, rows, 13)
    plain = lmhead.DeviceHead(device, w, fmt="bfp4", chunks=CHUNKS, k=k, rescore=False)
    vals, ids = plain.candidates(tx, rows)
    best = ids[torch.arange(rows), vals.argmax(dim=1)]  # the host's argmax over the same records
    picked = lmhead.DeviceHead(device, w, fmt="bfp4", chunks=CHUNKS, k=k, rescore=False, device_pick=True)
    same("records pick: rows against the host's argmax over the records", picked(tx, rows), best)
    mapped = lmhead.DeviceHead(device, w, fmt="bfp4", chunks=CHUNKS, k=k, rescore=False, device_pick=True,
                               token_map=tmap.tolist())
    same("records pick with a token map: tokens", mapped(tx, rows), tmap[best])
    ids_out = ttnn.from_torch(torch.zeros(1, 1, dtype=torch.int32), dtype=ttnn.uint32, layout=ttnn.ROW_MAJOR_LAYOUT,
                              device=device)
    mapped.logits_topk(tx, rows, ids_out=ids_out)
    assert int(ttnn.to_torch(ids_out).reshape(-1)[0]) == int(tmap[best][0])
    for h in (plain, picked, mapped):
        h.deallocate()
