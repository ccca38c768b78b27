"""The workspace-free RMSNorm entry point against the regular one.

cacti_b200_rmsnorm_fwd_bwd_noalloc exists for hosts that cannot hand the library a workspace: cacti's pctx
keeps nearly all device memory in its own arena, so a thunk that runs while the arena is full (or at a point
where the CUDA allocator must not be entered) has nowhere to get one.  The entry point keeps its dgamma
partials in an array inside the library image instead.  This test drives it through the C ABI twice in a row
(the array is shared by all calls and keeps the previous call's contents) and compares with the regular
entry point, which gets a caller-allocated workspace.  It lives in a file that sorts last so that a run that
stops at the first failure has already been through every other test.
"""
import numpy as np
import pytest
import torch

from cacti_b200 import capi
from oracle import ref_chain as R
from tests.gpu_util import dev, host
from tests.tolerances import assert_close

pytestmark = pytest.mark.gpu


def _both(x, gamma, dy, eps, dgamma_dtype=None):
    L = capi.lib()
    rows, cols = x.shape
    dt = {torch.float16: capi.R_16F, torch.float32: capi.R_32F}[x.dtype]
    gdt = dt if dgamma_dtype is None else dgamma_dtype
    gtorch = x.dtype if dgamma_dtype is None else torch.float32
    st = torch.cuda.current_stream().cuda_stream
    outs = []
    for noalloc in (False, True):
        y, dx = torch.empty_like(x), torch.empty_like(x)
        dg = torch.empty(cols, dtype=gtorch, device=x.device)
        if noalloc:
            rc = L.cacti_b200_rmsnorm_fwd_bwd_noalloc(y.data_ptr(), dx.data_ptr(), dg.data_ptr(), x.data_ptr(),
                                                      gamma.data_ptr(), dy.data_ptr(), eps, rows, cols, dt, gdt, 0, 0, st)
        else:
            ws = torch.empty(L.cacti_b200_rmsnorm_workspace_bytes(rows, cols), dtype=torch.uint8, device=x.device)
            rc = L.cacti_b200_rmsnorm_fwd_bwd(y.data_ptr(), dx.data_ptr(), dg.data_ptr(), x.data_ptr(), gamma.data_ptr(),
                                              dy.data_ptr(), eps, rows, cols, dt, gdt, 0, 0, ws.data_ptr(), ws.numel(), st)
        assert rc == capi.OK, rc
        outs.append((y, dx, dg))
    return outs


def test_noalloc_matches_workspace_entry_twice(cuda):
    # two calls in a row with different shapes and data: the second must not see the first one's partials
    cases = [((4096, 3200), np.float16, 100), ((300, 1024), np.float32, 200), ((33, 100), np.float16, 300)]
    for shape, dtype, seed in cases:
        kind = "float16" if dtype == np.float16 else "float32"
        x = dev(R.normal(seed, shape, dtype))
        gamma = dev(R.normal(seed + 1, (shape[1],), dtype, 0.02, 1.0))
        dy = dev(R.normal(seed + 2, shape, dtype))
        (y0, dx0, dg0), (y1, dx1, dg1) = _both(x, gamma, dy, 1e-6)
        assert torch.equal(y0, y1) and torch.equal(dx0, dx1)          # row-local results do not depend on the grid
        assert_close(host(dg1), host(dg0), kind, f"dgamma {shape}")   # column partials may be grouped differently
        # and against the CPU oracle, like the regular entry point is in the parity tests
        # (the oracle's single-rounding fp64 form, the one the shape sweep of the regular entry point is held to)
        ry, rdx, rdg = R.ideal64_rmsnorm(host(x), host(gamma), host(dy), 1e-6)
        assert_close(host(y1), ry, kind, f"y {shape} vs oracle")
        assert_close(host(dx1), rdx, kind, f"dx {shape} vs oracle")
        assert_close(host(dg1), rdg, kind, f"dgamma {shape} vs oracle")
    # fp32 partial output, as a collective would consume it
    x, gamma, dy = dev(R.normal(1, (512, 3200), np.float16)), dev(R.normal(2, (3200,), np.float16)), dev(R.normal(3, (512, 3200), np.float16))
    (_, _, a), (_, _, b) = _both(x, gamma, dy, 1e-6, dgamma_dtype=capi.R_32F)
    assert_close(host(b), host(a), "float32", "f32 dgamma")


def test_noalloc_rejects_shapes_beyond_its_array(cuda):
    L = capi.lib()
    P = 0x1000      # never dereferenced: the size check comes first
    assert L.cacti_b200_rmsnorm_fwd_bwd_noalloc(P, P, P, P, P, P, 1e-6, 8, 4097, capi.R_16F, capi.R_16F, 0, 0, None) == capi.ERR_SCRATCH_LIMIT
    assert L.cacti_b200_rmsnorm_fwd_bwd_noalloc(P, P, P, P, P, P, 1e-6, 2 * 148 * 4096 + 1, 7, capi.R_16F, capi.R_16F, 0, 0, None) == capi.ERR_SCRATCH_LIMIT
    assert b"scratch" in L.cacti_b200_error_string(capi.ERR_SCRATCH_LIMIT)
