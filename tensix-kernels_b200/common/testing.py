"""testing.py: the checks the path's tests use, with the reference's bars and line format (its common/testing.py:16-41):
relative Frobenius error and PCC against a float64 reference, bit-for-bit equality, and an expected exception. Every
check prints one line, "ok   <name>: ..." or "FAIL <name>: ...", and raises AssertionError on a failure."""

import sys
import traceback

import torch


def _line(passed, name, detail):
    print(("ok   " if passed else "FAIL ") + f"{name}: {detail}", flush=True)
    return passed


def check(name, y, r, rel=0.01, pcc=0.9999):
    """y against r: relative Frobenius error below rel, PCC above pcc, every value finite."""
    got, want = y.detach().float().cpu().reshape(-1), r.detach().float().cpu().reshape(-1)
    err = float((got - want).norm() / want.norm())
    corr = float(torch.corrcoef(torch.stack((got, want)))[0, 1])
    finite = bool(torch.isfinite(got).all())
    passed = _line(finite and err < rel and corr > pcc, name, f"rel {100 * err:.4f} % pcc {corr:.6f}")
    assert passed, (name, err, corr)


def same(name, a, b):
    """a and b bit for bit (shape and dtype included)."""
    equal = tuple(a.shape) == tuple(b.shape) and a.dtype == b.dtype and bool(torch.equal(a, b))
    assert _line(equal, name, "bit for bit " + ("equal" if equal else "DIFFERENT")), name


def raises(name, exc, fn):
    """fn() raises exc."""
    caught = None
    try:
        fn()
    except exc as e:
        caught = e
    if caught is None:
        _line(False, name, f"no {exc.__name__}")
        raise AssertionError(name)
    _line(True, name, type(caught).__name__)


def main(globs):
    """Run a module's test_* functions (all, or those named on the command line) on device 0; the exit code."""
    from common import ttnn_like as ttnn

    wanted = set(sys.argv[1:])
    device = ttnn.open_device(device_id=0)
    bad = 0
    for name in [n for n, f in globs.items() if n.startswith("test_") and callable(f) and (not wanted or n in wanted)]:
        try:
            globs[name](device)
        except Exception:
            traceback.print_exc()
            bad += 1
            print(f"FAIL {name}", flush=True)
        else:
            print(f"PASS {name}", flush=True)
    ttnn.close_device(device)
    return int(bad > 0)
