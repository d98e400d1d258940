"""testing.py: the checks the path's tests use, with the reference's bars (its common/testing.py:16-41): relative
Frobenius error and PCC against a float64 reference, bit-for-bit equality, and an expected exception."""

import sys
import traceback

import torch


def check(name, y, r, rel=0.01, pcc=0.9999):
    """y against r: relative Frobenius error below rel, PCC above pcc, every value finite."""
    y, r = y.float().cpu(), r.float().cpu()
    err = ((y - r).norm() / r.norm()).item()
    p = torch.corrcoef(torch.stack([y.flatten(), r.flatten()]))[0, 1].item()
    ok = bool(torch.isfinite(y).all()) and err < rel and p > pcc
    print(f"{'ok  ' if ok else 'FAIL'} {name}: rel {100 * err:.4f} % pcc {p:.6f}", flush=True)
    assert ok, (name, err, p)


def same(name, a, b):
    """a and b bit for bit."""
    ok = a.shape == b.shape and a.dtype == b.dtype and torch.equal(a, b)
    print(f"{'ok  ' if ok else 'FAIL'} {name}: bit for bit {'equal' if ok else 'DIFFERENT'}", flush=True)
    assert ok, name


def raises(name, exc, fn):
    """fn() raises exc."""
    try:
        fn()
    except exc as e:
        print(f"ok   {name}: {type(e).__name__}", flush=True)
        return
    print(f"FAIL {name}: no {exc.__name__}", flush=True)
    raise AssertionError(name)


def main(globs):
    """Run a module's test_* functions (all, or those named on the command line) on device 0."""
    from common import ttnn_like as ttnn

    tests = [(n, f) for n, f in globs.items() if n.startswith("test_") and callable(f)]
    only = sys.argv[1:]
    device = ttnn.open_device(device_id=0)
    failed = []
    for n, f in tests:
        if only and n not in only:
            continue
        try:
            f(device)
            print(f"PASS {n}", flush=True)
        except Exception:
            traceback.print_exc()
            failed.append(n)
            print(f"FAIL {n}", flush=True)
    ttnn.close_device(device)
    return 1 if failed else 0
