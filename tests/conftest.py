import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (test infrastructure). Built by `make -C oracle`."""
    from oracle import oracle as O
    O.lib()
    return O


@pytest.fixture(scope="session")
def cgb():
    import cantors_gift_b200 as pkg
    pkg.lib()
    return pkg


@pytest.fixture(scope="session")
def ops(cgb):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cantors_gift_b200 import ops as _ops
    return _ops


def report_metrics(what, **values):
    """Appends one JSON line per checked case to the file $CG_B200_PARITY_REPORT names (when set): how far
    each case lands from the reference on every metric, not only the asserted ones."""
    path = os.environ.get("CG_B200_PARITY_REPORT")
    if not path:
        return
    import json
    with open(path, "a") as f:
        f.write(json.dumps({"case": what, **{k: float(v) for k, v in values.items()}}) + "\n")


def error_metrics(y, ref):
    """(max|y-ref| / max|ref|, 99.9th percentile of |y-ref| / max(|ref|, 1e-3 max|ref|))."""
    y = np.asarray(y, dtype=np.float64).ravel()
    ref = np.asarray(ref, dtype=np.float64).ravel()
    scale = max(np.abs(ref).max(), 1e-30)
    diff = np.abs(y - ref)
    norm = diff.max() / scale
    rel = diff / np.maximum(np.abs(ref), 1e-3 * scale)
    return norm, float(np.percentile(rel, 99.9))


def assert_close(y, ref, tol, what=""):
    """Both metrics must be within `tol` (1e-4 for fp32 paths, 1e-2 for bf16/f16 paths)."""
    norm, p999 = error_metrics(y, ref)
    report_metrics(what, max_normalised=norm, p999_relative=p999, tol=tol)
    assert norm <= tol and p999 <= tol, f"{what}: max-normalised {norm:.3e}, p99.9 relative {p999:.3e}, tol {tol}"


def assert_close_rms(y, ref, tol, what="", p999_tol=None):
    """max|y-ref| / max|ref| <= tol and rms(y-ref) / rms(ref) <= tol. For results that are sums of
    many rounded terms of mixed sign (attention outputs, whole blocks): elements near zero carry the
    absolute rounding noise of the terms, so a per-element relative error is dominated by them.
    The per-element 99.9th-percentile metric of error_metrics is computed and reported as well, and
    asserted against `p999_tol` where one is given."""
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    err = np.abs(y - ref)
    norm = err.max() / max(np.abs(ref).max(), 1e-30)
    rms = np.sqrt((err ** 2).mean()) / max(np.sqrt((ref ** 2).mean()), 1e-30)
    _, p999 = error_metrics(y, ref)
    report_metrics(what, max_normalised=norm, rms_ratio=rms, p999_relative=p999, tol=tol)
    assert norm <= tol and rms <= tol, f"{what}: max-normalised {norm:.3e}, rms ratio {rms:.3e}, tol {tol}"
    if p999_tol is not None:
        assert p999 <= p999_tol, f"{what}: p99.9 relative {p999:.3e}, bound {p999_tol}"
