"""GPU parity of the fused AdamW32 update against the three-program f32 chain of the oracle (bit-exact)."""
import numpy as np
import pytest
import torch

from cacti_b200 import capi, ops
from oracle import ref_chain as R
from tests.gpu_util import bits, dev, host, offset_view

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("gdtype", [np.float16, np.float32])
@pytest.mark.parametrize("n", [1, 7, 8, 1000, 3200 * 33 + 5])
def test_adamw32_matches_chain(cuda, gdtype, n):
    w = R.normal(1, (n,), np.float32, 0.02)
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    dw, dm, dv = dev(w), dev(m), dev(v)
    p16 = torch.empty(n, dtype=torch.float16, device="cuda")
    for it in (1, 2, 3):                       # a few steps, state carried on both sides
        g = R.normal(10 + it, (n,), gdtype, 0.5)
        ops.adamw32_step(dw, dm, dv, dev(g), it, lr=1e-3, wd=0.01, grad_unscale=0.5, param_out=p16)
        w, m, v, p = R.ref_adamw32_step(w, m, v, g, it, lr=1e-3, wd=0.01, grad_unscale=0.5, param_dtype=np.float16)
        assert np.array_equal(bits(host(dm)), bits(m)), f"m step {it}"
        assert np.array_equal(bits(host(dv)), bits(v)), f"v step {it}"
        assert np.array_equal(bits(host(dw)), bits(w)), f"w step {it}"
        assert np.array_equal(bits(host(p16)), bits(p)), f"param step {it}"


def test_adamw32_unaligned_and_errors(cuda):
    n = 1001
    w, m, v = R.normal(2, (n,), np.float32), R.normal(3, (n,), np.float32, 0.1), np.abs(R.normal(4, (n,), np.float32, 0.1))
    g = R.normal(5, (n,), np.float16)
    dw, dm, dv = offset_view(w, 1), offset_view(m, 3), offset_view(v, 2)
    ops.adamw32_step(dw, dm, dv, offset_view(g, 1), 7)
    rw, rm, rv = R.ref_adamw32_step(w, m, v, g, 7)
    assert np.array_equal(bits(host(dw)), bits(rw)) and np.array_equal(bits(host(dm)), bits(rm)) and np.array_equal(bits(host(dv)), bits(rv))
    L = capi.lib()
    P = 0x1000
    assert L.cacti_b200_adamw32_step(P, P, P, 0, P, 8, capi.R_16F, capi.R_16F, 1.0, 1e-3, 0.0, 0.1, 1e-3, 1e-8, 0, None) == capi.ERR_INVALID_VALUE
    assert L.cacti_b200_adamw32_step(P, P, P, 0, P, 8, 7, capi.R_16F, 1.0, 1e-3, 0.0, 0.1, 1e-3, 1e-8, 1, None) == capi.ERR_DTYPE
    assert L.cacti_b200_adamw32_step(P, P, P, 0, P, 0, capi.R_16F, capi.R_16F, 1.0, 1e-3, 0.0, 0.1, 1e-3, 1e-8, 1, None) == capi.OK
