import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cacti_b200 import capi
    capi.lib()      # raises if the shared object is missing: there is no fallback
    return torch.device("cuda:0")


def pytest_terminal_summary(terminalreporter):
    """Every comparison that used a wider floor, a floor of its own or another rtol than the plain bound
    (rtol * max(|ref|, 0.1 rms)): how many of its elements the plain bound would have rejected."""
    from tests import tolerances
    rows = tolerances.OVERRIDES
    if not rows:
        return
    agg = {}
    for what, kind, n, outside, worst in rows:
        key = (what.split(" B=")[0][:60], kind)
        a = agg.setdefault(key, [0, 0, 0, 0.0])
        a[0] += 1; a[1] += n; a[2] += outside; a[3] = max(a[3], worst)
    tr = terminalreporter
    tr.write_sep("-", "comparisons with a tolerance override: elements outside the plain bound")
    clean = sum(1 for a in agg.values() if a[2] == 0)
    for (what, kind), (calls, n, outside, worst) in sorted(agg.items(), key=lambda kv: -kv[1][2]):
        if outside:
            tr.write_line(f"{outside:>10} of {n:>12} ({100.0 * outside / n:6.3f} %)  worst {worst:7.2f} x plain bound  [{kind}] {what} ({calls} calls)")
    tr.write_line(f"{clean} further overridden comparisons had no element outside the plain bound")
