"""The C++ host shim: arena, pins, soft-OOM spill policy (CPU, fake backend) and thunks under memory pressure (GPU)."""
import numpy as np
import pytest

from cacti_b200 import capi
from cacti_b200.host import binding as H
from oracle import ref_chain as R
from tests.tolerances import assert_close


def test_arena_and_spill_policy_on_fake_backend():
    KB = 1024
    ctx = H.Ctx(cuda=False, arena_bytes=64 * KB)
    L, h = ctx.L, ctx.h
    data = [np.full(16 * KB // 4, i + 1, dtype=np.float32) for i in range(6)]
    cells = [ctx.cell(d) for d in data]
    for c in cells[:4]:                      # 4 x 16 KB fill the arena
        assert L.cbh_pread(h, c) != 0
    assert L.cbh_in_use(h) == 64 * KB and ctx.stats()["spills"] == 0
    assert L.cbh_pread(h, cells[4]) != 0     # soft OOM: oldest unpinned cell is spilled, allocation retried
    s = ctx.stats()
    assert s["spills"] == 1 and s["oom_retries"] == 1 and not L.cbh_cell_resident(h, cells[0])
    for c, d in zip(cells, data):            # values survive spill and reload
        assert np.array_equal(ctx.get(c, d), d)
    # pinned cells are never evicted
    for c in cells[1:5]:
        if L.cbh_cell_resident(h, c):
            L.cbh_pin(h, c)
    assert L.cbh_pread(h, cells[5]) == 0 and ctx.stats()["hard_oom"] == 1      # everything resident is pinned
    for c in cells[1:5]:
        if L.cbh_cell_resident(h, c):
            L.cbh_unpin(h, c)
    assert L.cbh_pread(h, cells[5]) != 0
    # unlive, non-stable cells are dropped without a copy; stable ones are spilled
    before = ctx.stats()
    victim = next(c for c in cells if L.cbh_cell_resident(h, c))
    L.cbh_cell_unlive(h, victim)
    missing = next(c for c in cells if not L.cbh_cell_resident(h, c))
    assert L.cbh_pread(h, missing) != 0
    after = ctx.stats()
    assert after["drops"] == before["drops"] + 1 and after["spills"] == before["spills"]
    with pytest.raises(RuntimeError):
        ctx.get(victim, data[0])
    ctx.close()


def test_arena_free_list_reuse_and_soft_limit():
    ctx = H.Ctx(cuda=False, arena_bytes=1 << 20, soft_limit=3 * 4096)
    L, h = ctx.L, ctx.h
    cells = [ctx.cell(np.arange(1024, dtype=np.float32) + i) for i in range(5)]
    for c in cells:
        assert L.cbh_pread(h, c) != 0
    assert L.cbh_in_use(h) <= 3 * 4096                     # the soft limit, not the arena size, bounds residency
    assert ctx.stats()["spills"] == 2
    small = ctx.cell(np.zeros(10, dtype=np.float32))
    assert L.cbh_pread(h, small) != 0 and L.cbh_in_use(h) <= 3 * 4096
    assert L.cbh_pread(h, small) % 256 == 0                # ALLOC_ALIGN
    ctx.close()


@pytest.mark.gpu
def test_thunks_under_memory_pressure(cuda):
    """Run a small forward/backward slice through the shim with an arena that cannot hold every cell."""
    rows, cols = 512, 1024
    f16 = capi.R_16F
    x = R.normal(1, (rows, cols), np.float16)
    gamma = R.normal(2, (cols,), np.float16, 0.02, 1.0)
    w = R.normal(3, (cols, cols), np.float16, 0.03)
    nbytes = x.nbytes
    ctx = H.Ctx(cuda=True, arena_bytes=16 * nbytes, soft_limit=int(4.5 * nbytes))
    L, h = ctx.L, ctx.h
    cx, cg, cw = ctx.cell(x, stable=True), ctx.cell(gamma, stable=True), ctx.cell(w, stable=True)
    cy = ctx.cell(nbytes=nbytes)
    assert L.cbh_thunk_rmsnorm_fwd(h, H.APPLY, cy, cx, cg, 1e-6, rows, cols, f16) == 0
    cz = ctx.cell(nbytes=nbytes)
    assert L.cbh_thunk_matmul(h, H.APPLY, cz, cy, cw, rows, cols, cols, 0, 1, 1.0, f16) == 0       # z = y W^T
    cs = ctx.cell(nbytes=nbytes)
    assert L.cbh_thunk_add(h, H.APPLY, cs, cx, cz, rows * cols, f16) == 0                           # residual
    cp = ctx.cell(nbytes=nbytes)
    assert L.cbh_thunk_softmax_fwd(h, H.APPLY, cp, cs, rows, cols, 0, 0, f16) == 0
    dp = R.normal(4, (rows, cols), np.float16)
    cdp = ctx.cell(dp)
    old = R.normal(5, (rows, cols), np.float16)
    cds = ctx.cell(old)
    assert L.cbh_thunk_softmax_bwd(h, H.ACCUMULATE, cds, cs, cdp, rows, cols, 0, 0, f16) == 0       # ds += adjoint
    assert L.cbh_thunk_matmul(h, H.ACCUMULATE, cz, cy, cw, rows, cols, cols, 0, 1, 1.0, f16) == 0  # z += y W^T
    st = ctx.stats()
    assert st["spills"] > 0 and st["reloads"] > 0 and st["hard_oom"] == 0, st
    # oracle, op by op on the values the previous thunk actually produced (a 1-ulp f16 difference in one op's
    # output would otherwise be charged to the next op)
    y, _, _ = R.ref_rmsnorm_fwd(x, gamma, 1e-6)
    gy = ctx.get(cy, x)
    assert_close(gy, y, "float16", "y")
    gz2 = ctx.get(cz, x)                                            # z after Apply then Accumulate = 2 y W^T
    z1 = R.ref_gemm(gy, w, False, True)
    assert_close(gz2, R.ref_gemm(gy, w, False, True, beta=1.0, c=z1), "float16", "z accumulate", floor_frac=1.0)
    gs = ctx.get(cs, x)
    assert_close(gs, x + z1, "float16", "residual add", floor_frac=1.0)
    assert_close(ctx.get(cp, x), R.ref_softmax_fwd(gs)[0], "float16", "P")
    assert_close(ctx.get(cds, x), old + R.ref_softmax_bwd(gs, dp), "float16", "dS accumulate", floor_frac=1.0)
    assert np.array_equal(ctx.get(cx, x), x)                # a stable input that was spilled comes back intact
    ctx.close()


@pytest.mark.gpu
def test_reference_style_sync_per_thunk(cuda):
    x = R.normal(6, (64, 256), np.float16)
    g = R.normal(7, (256,), np.float16, 0.02, 1.0)
    ctx = H.Ctx(cuda=True, arena_bytes=1 << 20, sync_each_thunk=True)
    cx, cg, cy = ctx.cell(x), ctx.cell(g), ctx.cell(nbytes=x.nbytes)
    assert ctx.L.cbh_thunk_rmsnorm_fwd(ctx.h, H.APPLY, cy, cx, cg, 1e-6, 64, 256, capi.R_16F) == 0
    assert ctx.L.cbh_thunk_rmsnorm_fwd(ctx.h, H.ACCUMULATE, cy, cx, cg, 1e-6, 64, 256, capi.R_16F) == 0
    y, _, _ = R.ref_rmsnorm_fwd(x, g, 1e-6)
    assert_close(ctx.get(cy, x), y + y, "float16", "y accumulated twice", floor_frac=1.0)
    ctx.close()


@pytest.mark.gpu
def test_two_output_fused_thunk_matches_the_two_thunks(cuda):
    """add + rmsnorm as one two-output thunk through the shim: same bits as thunk_add followed by thunk_rmsnorm_fwd."""
    rows, cols = 96, 3200
    f16 = capi.R_16F
    a, b = R.normal(11, (rows, cols), np.float16), R.normal(12, (rows, cols), np.float16, 0.3)
    gamma = R.normal(13, (cols,), np.float16, 0.02, 1.0)
    ctx = H.Ctx(cuda=True, arena_bytes=64 * a.nbytes, soft_limit=64 * a.nbytes)
    L, h = ctx.L, ctx.h
    ca, cb, cg = ctx.cell(a), ctx.cell(b), ctx.cell(gamma)
    cs1, cy1, cs2, cy2 = (ctx.cell(nbytes=a.nbytes) for _ in range(4))
    assert L.cbh_thunk_add(h, H.APPLY, cs1, ca, cb, rows * cols, f16) == 0
    assert L.cbh_thunk_rmsnorm_fwd(h, H.APPLY, cy1, cs1, cg, 1e-6, rows, cols, f16) == 0
    assert L.cbh_thunk_add_rmsnorm_fwd(h, H.APPLY, cy2, cs2, ca, cb, cg, 1e-6, rows, cols, f16) == 0
    assert L.cbh_thunk_add_rmsnorm_fwd(h, H.ACCUMULATE, cy2, cs2, ca, cb, cg, 1e-6, rows, cols, f16) == capi.ERR_INVALID_VALUE
    assert np.array_equal(ctx.get(cs1, a).view(np.uint16), ctx.get(cs2, a).view(np.uint16))
    assert np.array_equal(ctx.get(cy1, a).view(np.uint16), ctx.get(cy2, a).view(np.uint16))
