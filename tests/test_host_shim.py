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


def test_arena_front_and_back_cursors():
    """Short-lived blocks grow from the front, long-lived ones from the back; the two cursors never cross; a freed
    block next to a cursor gives the space back to it, any other goes to the free list of its side."""
    L = H.lib()
    a = L.cbh_arena_create(16 * 256)
    try:
        f0, f1 = L.cbh_arena_alloc(a, 256, 0), L.cbh_arena_alloc(a, 512, 0)
        b0, b1 = L.cbh_arena_alloc(a, 256, 1), L.cbh_arena_alloc(a, 1024, 1)
        assert (f0, f1) == (0, 256) and (b0, b1) == (15 * 256, 11 * 256)
        assert L.cbh_arena_front(a) == 3 * 256 and L.cbh_arena_back(a) == 11 * 256 and L.cbh_arena_in_use(a) == 8 * 256
        assert L.cbh_arena_alloc(a, 9 * 256, 0) == 2 ** 64 - 1 and L.cbh_arena_alloc(a, 9 * 256, 1) == 2 ** 64 - 1   # would cross
        assert L.cbh_arena_alloc(a, 8 * 256, 0) == 3 * 256                    # exactly the gap
        assert L.cbh_arena_front(a) == L.cbh_arena_back(a)
        L.cbh_arena_free(a, 3 * 256)
        assert L.cbh_arena_front(a) == 3 * 256
        L.cbh_arena_free(a, b0)                                               # not at the back cursor: a hole of the back side
        assert L.cbh_arena_back(a) == 11 * 256
        assert L.cbh_arena_alloc(a, 256, 0) == 3 * 256                        # a front request does not take a back hole
        assert L.cbh_arena_alloc(a, 256, 1) == b0                             # a back request does
        L.cbh_arena_free(a, b0)
        L.cbh_arena_free(a, b1)                                               # at the cursor: it moves up over the hole too
        assert L.cbh_arena_back(a) == 16 * 256
        for off in (0, 256, 3 * 256):
            L.cbh_arena_free(a, off)
        assert L.cbh_arena_front(a) == 0 and L.cbh_arena_in_use(a) == 0
    finally:
        L.cbh_arena_destroy(a)


def test_vmem_soft_limit_strings():
    """CACTI_VMEM_SOFT_LIMIT as the reference reads it (src/pctx/nvgpu.rs:1438-1463): a bare number is a fraction of
    the device's memory (clamped, 32 MiB kept free), a number with a unit is bytes; 64 KiB granularity."""
    L = H.lib()
    G, M = 1 << 30, 1 << 20
    total, avail = 180 * G, 170 * G

    def parse(t):
        return L.cbh_parse_vmem_soft_limit(t.encode(), total, avail)

    assert parse("0.5") == 90 * G and parse("0.25") == 45 * G
    assert parse("1") == avail - 32 * M and parse("20000") == avail - 32 * M     # a bare integer is a (clamped) fraction too
    assert parse("64GiB") == 64 * G and parse("40 GiB") == 40 * G and parse("512MiB") == 512 * M and parse("3gib") == 3 * G
    assert parse("64GB") == 64 * 10 ** 9 // 65536 * 65536 and parse("100M") == 100 * 10 ** 6 // 65536 * 65536
    assert parse("65537B") == 65536
    for bad in ("", "abc", "12x", "-1", "1.5.2", "4 GiB extra"):
        assert parse(bad) == 0, bad


def test_freed_cells_give_back_memory_and_ids():
    ctx = H.Ctx(cuda=False, arena_bytes=8 * 4096)
    L, h = ctx.L, ctx.h
    a = ctx.cell(np.arange(1024, dtype=np.float32))
    assert L.cbh_pread(h, a) != 0 and L.cbh_in_use(h) == 4096
    L.cbh_pin(h, a)
    assert L.cbh_cell_free(h, a) != 0                       # pinned: a thunk is using it
    L.cbh_unpin(h, a)
    ctx.free(a)
    assert L.cbh_in_use(h) == 0
    b = ctx.cell(np.ones(16, dtype=np.float32))
    assert b == a                                            # the id is handed out again, as a fresh cell
    assert np.array_equal(ctx.get(b, np.ones(16, dtype=np.float32)), np.ones(16, dtype=np.float32))
    stable = ctx.cell(np.zeros(1024, dtype=np.float32), stable=True)
    p_front, p_back = L.cbh_pread(h, b), L.cbh_pread(h, stable)
    assert p_back - p_front == 8 * 4096 - 4096               # long-lived cells come from the back of the arena
    ctx.close()


def _small_llama():
    from cacti_b200 import llama_step as LS
    return LS.LlamaShape(layers=2, d_model=200, heads=2, head_dim=100, ffn=512, vocab=1000, seq=256)


@pytest.mark.gpu
@pytest.mark.parametrize("fused_bwd", [True, False])
def test_training_step_through_cells_with_and_without_spilling(cuda, fused_bwd):
    """The config-5 step (reduced size) driven through cells and thunks: with the soft limit above the step's peak
    nothing spills; with it below, activations go to page-locked host memory during the forward pass and come back
    in the backward pass.  Loss and every gradient are bit-identical between the two, and bit-identical to the same
    step over torch-owned memory (same kernels, same arguments, other addresses)."""
    import torch
    from cacti_b200 import dp, llama_step as LS
    from cacti_b200.cell_step import CellTrainStep
    cfg, batch = _small_llama(), 2
    P = LS.init_weights(cfg, cuda, seed=3)
    g = torch.Generator(device=cuda).manual_seed(4)
    tok = torch.randint(0, cfg.vocab, (batch * cfg.seq,), device=cuda, dtype=torch.int32, generator=g)
    tgt = torch.randint(0, cfg.vocab, (batch * cfg.seq,), device=cuda, dtype=torch.int32, generator=g)
    grads, _ = dp.alloc_bucketed_grads(P)
    mode = "fused-bwd" if fused_bwd else "fused"        # attention adjoint in one thunk, or P and dS as cells + block matmuls
    loss_t = float(LS.TrainStep(cfg, P, batch, attention=mode).forward_backward(tok, tgt, grads).item())
    flat_t = {k: v.cpu().numpy() for k, v in LS.flat_params(grads)}
    W = {k: v.cpu().numpy() for k, v in P.items() if k != "layers"}
    W["layers"] = [{k: v.cpu().numpy() for k, v in Lw.items()} for Lw in P["layers"]]
    results = {}
    for name, limit in (("roomy", 0), ("tight", None)):
        arena = 256 << 20
        if limit is None:                      # below the peak of the roomy run, above what one thunk pins at once
            limit = int(results["roomy"][2]["peak_in_use"] * 0.45)
        ctx = H.Ctx(cuda=True, arena_bytes=arena, soft_limit=limit)
        step = CellTrainStep(ctx, cfg, W, batch, fused_bwd=fused_bwd)
        loss = step.forward_backward(tok.cpu().numpy(), tgt.cpu().numpy())
        grads_c = {k: step.gradient(k) for k in flat_t}
        results[name] = (loss, grads_c, ctx.stats())
        ctx.close()
    roomy, tight = results["roomy"], results["tight"]
    assert roomy[2]["spills"] == 0 and roomy[2]["hard_oom"] == 0
    assert tight[2]["spills"] > 0 and tight[2]["reloads"] > 0 and tight[2]["hard_oom"] == 0, tight[2]
    assert tight[2]["spill_bytes"] > 0 and tight[2]["peak_in_use"] <= int(roomy[2]["peak_in_use"] * 0.45)
    assert roomy[0] == tight[0] == loss_t
    for k, ref in flat_t.items():
        assert np.array_equal(roomy[1][k].view(np.uint16), ref.view(np.uint16)), k
        assert np.array_equal(tight[1][k].view(np.uint16), ref.view(np.uint16)), k


@pytest.mark.gpu
def test_adamw_as_an_initialize_thunk(cuda):
    """The optimizer update staged as the reference stages it, an Initialize-mode thunk that reads and overwrites its
    outputs (src/op.rs:950-1023): three steps through cells, master weights bit-identical to the oracle's chain."""
    n = 5000
    w0 = R.normal(21, (n,), np.float32, 0.02)
    ctx = H.Ctx(cuda=True, arena_bytes=1 << 22)
    L, h = ctx.L, ctx.h
    master, m1, m2 = ctx.cell(w0, stable=True), ctx.cell(np.zeros(n, np.float32), stable=True), ctx.cell(np.zeros(n, np.float32), stable=True)
    p16 = ctx.cell(nbytes=2 * n, stable=True)
    rw, rm, rv = w0, np.zeros(n, np.float32), np.zeros(n, np.float32)
    for it in (1, 2, 3):
        g = R.normal(30 + it, (n,), np.float16)
        cg = ctx.cell(g)
        assert L.cbh_thunk_adamw32_step(h, H.APPLY, master, m1, m2, p16, cg, n, capi.R_16F, capi.R_16F, 1.0, 1e-3, 0.01, 0.1, 1e-3,
                                        1e-8, it) == capi.ERR_INVALID_VALUE          # not an Apply or Accumulate thunk
        assert L.cbh_thunk_adamw32_step(h, H.INITIALIZE, master, m1, m2, p16, cg, n, capi.R_16F, capi.R_16F, 1.0, 1e-3, 0.01, 0.1,
                                        1e-3, 1e-8, it) == 0
        ctx.free(cg)
        out = R.ref_adamw32_step(rw, rm, rv, g, it, lr=1e-3, wd=0.01, param_dtype=np.float16)
        rw, rm, rv = out[0], out[1], out[2]
    assert np.array_equal(ctx.get(master, w0).view(np.uint32), rw.view(np.uint32))
    assert np.array_equal(ctx.get(m1, w0).view(np.uint32), rm.view(np.uint32))
    assert np.array_equal(ctx.get(p16, np.zeros(n, np.float16)).view(np.uint16), rw.astype(np.float16).view(np.uint16))
    ctx.close()
