"""device.py: the device-side helpers dense_reader/linear.py imports, for a B200.

Mirror of the names in the reference's common/device.py (file:line below are that file's). A Tensix device spreads a
weight over DRAM banks and places cores next to them; a B200 has one flat HBM space, so "banks" here are only a number
a weight's memory config records (the HBM stacks by default), kept so that max_banks / check_banks behave as callers
expect. Placement, read virtual channels and the loader split are Tensix mechanisms: the functions exist, validate and
return what callers can carry around, and steer nothing.
"""

from fractions import Fraction

from common import ttnn_like as ttnn

TILE = 32

# Tensix multiplier passes (common/device.py:21-26). Products here are exact in fp32 whatever the name says.
FIDELITY = {"lofi": "lofi", "hifi2": "hifi2", "hifi3": "hifi3", "hifi4": "hifi4"}

# Caps the banks a weight's memory config reports (None: every bank of the device). (:29)
MAX_BANKS = None
# Core placement policy of the reference (:34); accepted, unused.
PLACE = "optimal"


def dram_banks(device, max_banks=None):
    """The banks weights are sharded over: the device's, at most max_banks (default MAX_BANKS). (:37-42)"""
    g = device.dram_grid_size()
    n = g.x * g.y
    cap = max_banks if max_banks is not None else MAX_BANKS
    return min(n, cap) if cap else n


def bank_grid(banks):
    """The shard grid's name for banks 0 .. banks - 1. (:45-48)"""
    assert banks >= 1, banks
    return f"banks[0..{banks - 1}]"


def is_dram_sharded(t):
    """(:51-53)"""
    mc = t.memory_config()
    return mc.buffer_type == ttnn.BufferType.DRAM and mc.memory_layout == ttnn.TensorMemoryLayout.WIDTH_SHARDED


def check_banks(t, max_banks=None):
    """ValueError for a width-sharded weight over more banks than max_banks (default MAX_BANKS; None: no limit).
    (:56-62)"""
    cap = max_banks if max_banks is not None else MAX_BANKS
    if t is None or not cap or not is_dram_sharded(t):
        return
    have = t.memory_config().shard_spec.num_cores()
    if have > cap:
        raise ValueError(f"a weight sharded over {have} DRAM banks (at most {cap}: max_banks)")


def sharded_memcfg(device, k, n, banks=None, max_banks=None):
    """Width-sharded over `banks` banks, N padded to a multiple of banks * 32. (:65-71)"""
    banks = banks or dram_banks(device, max_banks)
    padded = ttnn.padded_cols(n, banks)
    spec = ttnn.ShardSpec(banks, (k, padded // banks))
    return ttnn.MemoryConfig(ttnn.TensorMemoryLayout.WIDTH_SHARDED, ttnn.BufferType.DRAM, spec)


def place(device, banks, sharded):
    """A "core" per work item (:77-100). Work items here are CTAs; CTA i runs wherever the hardware puts it."""
    return list(range(len(banks)))


def read_vcs(work):
    """DRAM read virtual channels (:103-114): none on a GPU."""
    return [0] * len(work)


def split_arg(split, share=0.5):
    """The reference's SPLIT compile argument for a reader's share of the weight chunks (:117-132): 0 without split, 1
    for an even alternation, else period << 24 | mask of the writer's positions in the period (spread out, never
    position 0, never adjacent). Kept so that callers' settings validate the same way; the B200 kernel has one
    producer."""
    if not split:
        return 0
    share = float(share)
    assert 0.5 <= share <= 0.75, f"a split share of {share} (the reader's; 0.5 to 0.75)"
    if share == 0.5:
        return 1
    writer = Fraction(1 - share).limit_denominator(24)
    period, count = writer.denominator, writer.numerator
    mask = 0
    for i in range(count):
        mask |= 1 << ((2 * i + 1) * period // (2 * count))
    assert 3 <= period <= 24 and not mask & 1 and not mask & (mask >> 1), (share, period, mask)
    return (period << 24) | mask


def l1_free(device):
    """Bytes of on-chip memory a CTA's buffers may take (:135-141): the 227 KB of shared memory a CTA can have."""
    return 227 * 1024
