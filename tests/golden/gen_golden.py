"""gen_golden.py: makes tests/golden/*.npz from the reference's own host functions.

Run where the reference checkout is, with its path as the argument:

    python tests/golden/gen_golden.py /path/to/tensix-kernels

The reference's modules import ttnn at the top; a MagicMock stands in for it, which is enough for the pure-host
functions used here: moe.moe8.bfp4_tiles / bfp4_values (the only in-tree statement of the block-float quantiser, pinned
bit for bit to ttnn's BFP4_b conversion by moe/tests/test_moe.py:84-89), dense_reader.linear.records_host /
interleave_glu / bf16_ceil / reference, common.device.split_arg. Nothing of the reference is copied: only the
outputs of running it on seeded inputs are stored.
"""

import hashlib
import sys
from pathlib import Path
from unittest.mock import MagicMock

import numpy as np
import torch

if len(sys.argv) < 2:
    sys.exit("usage: python tests/golden/gen_golden.py /path/to/tensix-kernels")
ref = Path(sys.argv[1])
sys.modules["ttnn"] = MagicMock()
sys.path.insert(0, str(ref))
from common import device as cdev  # noqa: E402
from dense_reader import linear as rlin  # noqa: E402
from moe import moe8  # noqa: E402
from int4 import w4a16  # noqa: E402
from ternary_matmul import t2 as tern  # noqa: E402

out = Path(__file__).resolve().parent
sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()  # noqa: E731


def retile(v):
    """bfp4_values' [KT, NT, 32, 32] -> [K, N]."""
    kt, nt = v.shape[:2]
    return np.ascontiguousarray(v.transpose(0, 2, 1, 3).reshape(kt * 32, nt * 32))


# 1. the quantiser: the input of moe/tests/test_moe.py:84-88, and test_formats' weight as [K, N]
g = torch.Generator().manual_seed(0)
w1 = torch.randn(256, 512, generator=g) * 0.02
w1[3, 5], w1[7, 9] = 0.0, -1e-30
t1 = moe8.bfp4_tiles(w1)
v1 = retile(moe8.bfp4_values(t1))
g = torch.Generator().manual_seed(2)
w2 = (torch.randn(2048, 1024, generator=g) * 0.02).T.contiguous()
t2 = moe8.bfp4_tiles(w2)
# 2. rounding cases in one face row (ties to even, the clamp without an exponent bump, signs, flush of small values)
w3 = torch.zeros(32, 32)
w3[0, :16] = torch.tensor([1.0, 0.5, 0.25, 0.125, 0.0625, 0.1875, 0.3125, 0.4375, 0.5625, 0.6875, 0.9375, 0.96875,
                           -0.96875, -0.0624, 1.9999, -1.0])
v3 = retile(moe8.bfp4_values(moe8.bfp4_tiles(w3)))
# 3. wide exponent spread inside face rows, denormals, zeros, huge values
g = torch.Generator().manual_seed(5)
w4 = torch.randn(64, 64, generator=g) * torch.exp2(torch.randint(-40, 40, (64, 64), generator=g).float())
w4[0, :16] = 0.0
w4[1, 0] = 1e-40
w4[2, 3] = 3e38
t4 = moe8.bfp4_tiles(w4)
np.savez_compressed(
    out / "quantiser_bfp4.npz",
    w1_sha=sha(w1.numpy()), t1=t1, v1_sha=sha(v1), v1_row0=v1[0, :64],
    t2_sha=sha(t2), t2_head=t2[:2, :2],
    w3=w3.numpy(), v3=v3,
    w4=w4.numpy(), t4=t4, v4=retile(moe8.bfp4_values(t4)),
)

# 4. host helpers of dense_reader/linear.py
gate = torch.arange(128.0).reshape(64, 2)
il = rlin.interleave_glu(gate, -gate)
s = torch.tensor([0.0201, 1.0, 3.14159, 1e-8, 0.7, 123.456, 65504.0])
bits = torch.tensor([0x3FC0, 0xC000, 0x0000, 0x8000, 0x7F80, 0xFF80, 0x0001, 0x8001, 0x4049], dtype=torch.int32)
keys = torch.where(bits >= 0x8000, (~bits) & 0xFFFF, bits | 0x8000)
rec = torch.zeros(3, 2 * 2 * 4, dtype=torch.int32)  # 3 records of rows 2, k 4
rec[0, :8] = keys[:8]
rec[0, 8:] = torch.arange(100, 108)
rec[1, :4] = keys[5:9]
rec[1, 8:12] = torch.tensor([7, 0xFFFFFFFF - (1 << 32), 9, 10], dtype=torch.int64).to(torch.int32)
vals, idx = rlin.records_host(rec, 2, 4)
x = torch.randn(3, 64, generator=torch.Generator().manual_seed(9))
wk = torch.randn(64, 32, generator=torch.Generator().manual_seed(10)) * 0.02
sc = torch.rand(32, generator=torch.Generator().manual_seed(11)) + 0.5
np.savez_compressed(
    out / "host_helpers.npz",
    il=il.numpy(), ceil_in=s.numpy(), ceil_out=rlin.bf16_ceil(s).numpy(),
    split=np.array([cdev.split_arg(True, v) for v in (0.5, 0.6, 2 / 3, 0.75)] + [cdev.split_arg(False)], np.int64),
    bf16_bits=bits.numpy(), keys=keys.numpy(), rec=rec.numpy(), rec_vals=vals.numpy(), rec_idx=idx.numpy(),
    x=x.numpy(), wk=wk.numpy(), sc=sc.numpy(), ref=rlin.reference(x, wk).numpy(), ref_sc=rlin.reference(x, wk, sc).numpy(),
)
print("t1", sha(t1), "v1", sha(v1), "t2", sha(t2))


# 6. the int4 weight with group scales (int4/w4a16.py): nibbles, dequantized and reference on the test file's own
# case generator (int4/tests/test_int4.py:27-31, seeds of test_matmul's first case and a small one)
def int4_case(n, k, seed):
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(-7, 8, (n, k), generator=g).to(torch.int8)
    scales = (torch.rand(n, k // 32, generator=g) * 0.01 + 0.001).to(torch.bfloat16)
    return codes, scales


c1, s1 = int4_case(64, 96, 5)
g = torch.Generator().manual_seed(6)
x1 = torch.randn(1, 96, generator=g)
c2, s2 = int4_case(1152, 1024, 1024 + 1152)
g = torch.Generator().manual_seed(1152)
x2 = torch.randn(1, 1024, generator=g)
x2[:, torch.randperm(1024, generator=g)[:8]] *= 20
np.savez_compressed(
    out / "int4.npz",
    codes1=c1.numpy(), scales1_bits=s1.view(torch.int16).numpy(), x1=x1.numpy(),
    nib1=w4a16.nibbles(c1.T.contiguous()).numpy(), deq1=w4a16.dequantized(c1, s1).numpy(),
    ref1=w4a16.reference(x1, c1, s1).numpy(),
    codes2_sha=sha(c2.numpy()), nib2_sha=sha(w4a16.nibbles(c2.T.contiguous()).numpy()),
    deq2_sha=sha(w4a16.dequantized(c2, s2).numpy()), ref2=w4a16.reference(x2, c2, s2).numpy(),
)
print("wrote", out / "int4.npz")


# 7. the ternary weight (ternary_matmul/t2.py): tiles in its three forms, rotate, dequantize, reference on the test file's
# own generators (ternary_matmul/tests/test_ternary.py:35-62)
def t2_weight(n, k, g_, seed, zeros=0.3):
    gen = torch.Generator().manual_seed(seed)
    u = torch.randint(0, 2000, (n, k), generator=gen, dtype=torch.int16)
    trits = torch.where(u < 2000 * zeros, 0, torch.where(u % 2 == 0, 1, -1)).to(torch.int8)
    scales = (0.01 + 0.02 * torch.rand(n, k // g_, generator=gen)).to(torch.float16)
    return trits, scales


tr, sc = t2_weight(64, 2048, 128, 5)
gen = torch.Generator().manual_seed(6)
sg = torch.where(torch.rand(2048, generator=gen) < 0.5, -1.0, 1.0)
gen = torch.Generator().manual_seed(7)
xt = torch.randn(2, 2048, generator=gen).to(torch.bfloat16)
np.savez_compressed(
    out / "ternary.npz",
    trits=tr.numpy(), scales_bits=sc.view(torch.int16).numpy(), signs=sg.numpy(), x_bits=xt.view(torch.int16).numpy(),
    tiles_bfp2=tern.tiles(tr.T.contiguous(), "bfp2").numpy(), tiles_bfp2c=tern.tiles(tr.T.contiguous(), "bfp2c").numpy(),
    tiles_bfp4=tern.tiles(tr.T.contiguous(), "bfp4").numpy(),
    rotated=tern.rotate(xt.double(), sg).numpy(), deq=tern.dequantize(tr, sc.to(torch.bfloat16), 128).numpy(),
    ref=tern.reference(xt, tr, sc, 128).numpy(), sylvester8=tern.sylvester(8).numpy(),
)
print("wrote", out / "ternary.npz")


# 8. the mixture-of-experts layer (moe/moe8.py): the K-block form of the quantiser, reference / reference_rows / union on
# a small layer of experts on the bfloat4_b grid (the generators of moe/tests/test_moe.py:35-56 at a smaller shape)
ME, MH, MI, MK = 6, 64, 32, 3


def moe_grid(w):
    k, n = w.shape
    v = moe8.bfp4_values(moe8.bfp4_tiles(w))
    return torch.from_numpy(v.transpose(0, 2, 1, 3).reshape(k, n).copy())


gen = torch.Generator().manual_seed(21)
mgu = torch.stack([moe_grid(torch.randn(MH, 2 * MI, generator=gen) * 0.1) for _ in range(ME)])
mdn = torch.stack([moe_grid(torch.randn(MI, MH, generator=gen) * 0.05) for _ in range(ME)])
mgb = torch.randn(ME, 2 * MI, generator=gen) * 0.5
mx = torch.randn(4, MH, generator=gen).to(torch.bfloat16)
mids = torch.stack([torch.randperm(ME, generator=gen)[:MK] for _ in range(4)])
mw = torch.softmax(torch.randn(4, MK, generator=gen), -1).to(torch.bfloat16)
moe_out = {}
for act in ("silu", "gelu_tanh", "swiglu_oai"):
    y, h = moe8.reference(mx[:1].float(), mgu, mdn, mids[0].tolist(), mw[0].float(), act)
    yb, hb = moe8.reference(mx[:1].float(), mgu, mdn, mids[0].tolist(), mw[0].float(), act, mgb)
    moe_out.update({f"y_{act}": y.numpy(), f"h_{act}": h.numpy(), f"yb_{act}": yb.numpy(), f"hb_{act}": hb.numpy()})
moe_out["rows_silu"] = moe8.reference_rows(mx.float(), mgu, mdn, mids.tolist(), mw.float(), "silu").numpy()
moe_out["rows_oai_bias"] = moe8.reference_rows(mx.float(), mgu, mdn, mids.tolist(), mw.float(), "swiglu_oai", mgb).numpy()
# the router: random rows with ties (every other row rounded to bf16), rows of equal logits, of large and of tiny ones
gen = torch.Generator().manual_seed(31)
rl = torch.randn(12, 64, generator=gen) * 3
rl[::2] = rl[::2].to(torch.bfloat16).float()
rl[8] = 1.5
rl[9] = torch.randn(64, generator=gen) * 40
rl[10] = torch.randn(64, generator=gen) * 1e-6
rl[11, :10] = 2.5
rb = torch.randn(64, generator=gen) * 0.1
route_cases = {
    "softmax": dict(kind="softmax"), "sigmoid": dict(kind="sigmoid"), "sigmoid_raw": dict(kind="sigmoid", norm=False),
    "sigmoid_bias": dict(kind="sigmoid", bias=rb),
    "groups": dict(kind="sigmoid", bias=rb, groups=(8, 3), scale=2.5, slot=64),
}
for name, kw in route_cases.items():
    ri, rw = moe8.route_reference(rl, 6, **kw)
    moe_out[f"route_ids_{name}"], moe_out[f"route_w_{name}"] = ri.numpy(), rw.numpy()
np.savez_compressed(
    out / "moe.npz",
    route_logits=rl.numpy(), route_bias=rb.numpy(), sigmoid_table=np.array(moe8.sigmoid_table(), np.int64),
    gu=mgu.numpy(), dn=mdn.numpy(), gb=mgb.numpy(), x_bits=mx.view(torch.int16).numpy(), ids=mids.numpy(),
    w_bits=mw.view(torch.int16).numpy(), union=np.array(moe8.union(mids, ME), np.int64),
    union_clip=np.array(moe8.union(torch.tensor([[5, 9, 2], [2, 7, 0]]), 6), np.int64),
    t1_kblock_sha=sha(moe8.bfp4_tiles(w1, kblock=True)), t4_kblock=moe8.bfp4_tiles(w4, kblock=True),
    v4_kblock=retile(moe8.bfp4_values(moe8.bfp4_tiles(w4, kblock=True), kblock=True)),
    **moe_out,
)
print("wrote", out / "moe.npz")
