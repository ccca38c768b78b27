"""GPU parity tests: every entry point of the C ABI against the CPU oracle on the same seeded inputs.

Tolerances (tests/tolerances.py): fp32 1e-5 relative; fp16 2e-3 relative / one fp16 ulp; bf16 (no
reference chain) one bf16 ulp of the fp64 result; index gathers bit-exact.
"""
import os

import numpy as np
import pytest
import torch

from cacti_b200 import capi, ops
from oracle import ref_chain as R
from tests.golden import make_golden as G
from tests.gpu_util import bits, dev, host, offset_view
from tests.tolerances import assert_close

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden_small.npz"))
KIND = {np.dtype(np.float32): "float32", np.dtype(np.float16): "float16"}


# ------------------------------------------------------------------------------------------- K1
@pytest.mark.parametrize("case", [1, 2])
def test_rmsnorm_golden(cuda, case):
    a = G.inputs(case)
    kind = KIND[a["x"].dtype]
    x, g, dy = dev(a["x"]), dev(a["gamma"]), dev(a["dy"])
    y = ops.rmsnorm_fwd(x, g, a["eps"])
    dx, dg = ops.rmsnorm_bwd(x, g, dy, a["eps"])
    y2, dx2, dg2 = ops.rmsnorm_fwd_bwd(x, g, dy, a["eps"])
    for got, name in ((y, "y"), (y2, "y"), (dx, "dx"), (dx2, "dx"), (dg, "dgamma"), (dg2, "dgamma")):
        assert_close(host(got), GOLD[f"c{case}_{name}"], kind, f"rmsnorm {name}")
    assert torch.equal(y, y2) and torch.equal(dx, dx2) and torch.equal(dg, dg2)


def test_rmsnorm_config1_full(cuda):
    """benchmark config 1: [256 x 3200] fp32, gamma = 1 + 0.02 N(0,1), eps 1e-6, seed 0."""
    x = R.normal(0, (256, 3200))
    gamma = R.normal(1, (3200,), scale=0.02, shift=1.0)
    dy = R.normal(2, (256, 3200))
    y, dx, dg = ops.rmsnorm_fwd_bwd(dev(x), dev(gamma), dev(dy), 1e-6)
    ry, _, _ = R.ref_rmsnorm_fwd(x, gamma, 1e-6)
    rdx, rdg = R.ref_rmsnorm_bwd(x, gamma, dy, 1e-6)
    assert_close(host(y), ry, "float32", "y")
    assert_close(host(dx), rdx, "float32", "dx")
    assert_close(host(dg), rdg, "float32", "dgamma")
    i64 = R.ideal64_rmsnorm(x, gamma, dy, 1e-6)
    for got, ref, n in zip((y, dx, dg), i64, ("y", "dx", "dgamma")):
        assert_close(host(got), ref, "float32", n + " vs fp64")


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("rows,cols", [(1, 1), (2, 2), (3, 7), (33, 8), (3, 9), (2, 100), (33, 104), (5, 3200),
                                       (3, 4104), (2, 8200), (1, 20000)])
def test_rmsnorm_shapes(cuda, dtype, rows, cols):
    kind = KIND[np.dtype(dtype)]
    x = R.normal(10, (rows, cols), dtype)
    gamma = R.normal(11, (cols,), dtype, 0.02, 1.0)
    dy = R.normal(12, (rows, cols), dtype)
    y, dx, dg = ops.rmsnorm_fwd_bwd(dev(x), dev(gamma), dev(dy), 1e-6)
    ry, rdx, rdg = R.ideal64_rmsnorm(x, gamma, dy, 1e-6)
    assert_close(host(y), ry, kind, "y")
    # dx = gamma*dy/s - x*c is a difference of O(|dy|) terms (for cols = 1 it cancels to ~eps): hold it to the
    # scale of its terms
    assert_close(host(dx), rdx, kind, "dx", floor_abs=float(np.abs(dy.astype(np.float64)).max()) if cols < 16 else 0.0)
    assert_close(host(dg), rdg, kind, "dgamma")
    # separate entry points give the same bits as the fused one
    assert torch.equal(ops.rmsnorm_fwd(dev(x), dev(gamma), 1e-6), y)


def test_rmsnorm_unaligned_view_and_accumulate(cuda):
    a = G.inputs(2)
    x, dy = offset_view(a["x"], 1), offset_view(a["dy"], 3)
    g = dev(a["gamma"])
    y, dx, dg = ops.rmsnorm_fwd_bwd(x, g, dy, a["eps"])
    assert_close(host(y), GOLD["c2_y"], "float16", "y (unaligned)")
    assert_close(host(dx), GOLD["c2_dx"], "float16", "dx (unaligned)")
    assert_close(host(dg), GOLD["c2_dgamma"], "float16", "dgamma (unaligned)")
    # Accumulate mode: out = T(old + T(new)) in the output dtype, for dx and dgamma, fast and element-wise paths
    for xin, dyin in ((dev(a["x"]), dev(a["dy"])), (x, dy)):
        old_dx = R.normal(77, a["x"].shape, np.float16)
        old_dg = R.normal(78, (3200,), np.float16)
        dxa, dga = dev(old_dx), dev(old_dg)
        ops.rmsnorm_bwd(xin, g, dyin, a["eps"], dx=dxa, dgamma=dga, beta_dx=1, beta_dgamma=1)
        assert_close(host(dxa), old_dx + GOLD["c2_dx"], "float16", "dx accumulate", floor_frac=1.0)
        assert_close(host(dga), old_dg + GOLD["c2_dgamma"], "float16", "dgamma accumulate", floor_frac=1.0)


def test_rmsnorm_f32_partial_and_bf16(cuda):
    a = G.inputs(2)
    _, dg32 = ops.rmsnorm_bwd(dev(a["x"]), dev(a["gamma"]), dev(a["dy"]), a["eps"], dgamma_dtype=torch.float32)
    assert dg32.dtype == torch.float32
    _, _, ref = R.ideal64_rmsnorm(a["x"].astype(np.float32), a["gamma"].astype(np.float32), a["dy"].astype(np.float32), 1e-6)
    assert_close(host(dg32), ref, "float32", "f32 dgamma partial")
    x = R.bf16_round(R.normal(20, (9, 3200)))
    gm = R.bf16_round(R.normal(21, (3200,), scale=0.02, shift=1.0))
    dy = R.bf16_round(R.normal(22, (9, 3200)))
    y, dx, dg = ops.rmsnorm_fwd_bwd(dev(x, bf16=True), dev(gm, bf16=True), dev(dy, bf16=True), 1e-6)
    ry, rdx, rdg = R.ideal64_rmsnorm(x, gm, dy, 1e-6)
    assert_close(host(y), ry, "bfloat16", "bf16 y")
    assert_close(host(dx), rdx, "bfloat16", "bf16 dx")
    assert_close(host(dg), rdg, "bfloat16", "bf16 dgamma")


def test_rmsnorm_deterministic(cuda):
    x, g, dy = (dev(R.normal(s, sh, np.float16)) for s, sh in ((1, (4096, 3200)), (2, (3200,)), (3, (4096, 3200))))
    a = ops.rmsnorm_fwd_bwd(x, g, dy, 1e-6)
    b = ops.rmsnorm_fwd_bwd(x, g, dy, 1e-6)
    assert all(torch.equal(p, q) for p, q in zip(a, b))


# ------------------------------------------------------------------------------------------- K2
@pytest.mark.parametrize("case", [3, 4])
def test_softmax_golden(cuda, case):
    a = G.inputs(case)
    s, dp = dev(a["s"]), dev(a["dp"])
    p = ops.softmax_fwd(s, a["mask"])
    ds = ops.softmax_bwd(s, dp, a["mask"])
    p2, ds2 = ops.softmax_fwd_bwd(s, dp, a["mask"])
    assert_close(host(p), GOLD[f"c{case}_p"], "float16", "P")
    assert_close(host(ds), GOLD[f"c{case}_ds"], "float16", "dS")
    assert torch.equal(p, p2) and torch.equal(ds, ds2)
    keep = R.causal_keep_mask(*a["s"].shape, *a["mask"])
    assert (bits(host(p))[~keep] == 0).all() and (bits(host(ds))[~keep] == 0).all()   # exact +0
    # input that already carries -inf above the diagonal, no in-kernel mask: same result
    pre = np.where(keep, a["s"], np.float16(-np.inf))
    p3, ds3 = ops.softmax_fwd_bwd(dev(pre), dp, None)
    assert_close(host(p3), GOLD[f"c{case}_p"], "float16", "P (pre-masked)")
    assert_close(host(ds3)[keep], GOLD[f"c{case}_ds"][keep], "float16", "dS (pre-masked)")


@pytest.mark.parametrize("tokens", [70, 2500])
@pytest.mark.parametrize("heads,hd,pitch,bf16", [(32, 100, 128, False), (3, 64, 64, False), (2, 20, 32, False), (4, 100, 128, True),
                                                 (1, 20, 28, False)])
def test_rope_fwd_pitched_equals_rope_then_pad(cuda, heads, hd, pitch, bf16, tokens):
    """Head-pitched RoPE output = rope_fwd followed by block_pad, bit for bit; positions wrap and start at an offset.
    Token rows of a multiple of 16 bytes take the staged kernel (2500 tokens: every ring slot and output buffer of a
    group is reused many times), the last shape (40-byte rows) the per-thread one."""
    seq = 32
    x = dev(R.normal(95, (tokens, heads, hd), np.float32), bf16=True) if bf16 else dev(R.normal(95, (tokens, heads, hd), np.float16))
    cos, sin = ops.rope_tables(seq, hd, 10000.0, x.dtype, "cuda")
    want = ops.block_pad(ops.rope_fwd(x, cos, sin, pos_off=5).view(1, tokens, heads, hd), pitch).view(tokens, heads, pitch)
    got = torch.full((tokens, heads, pitch), 7.0, dtype=x.dtype, device="cuda")
    ops.rope_fwd_pitched(x, cos, sin, pitch, pos_off=5, y=got)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    L = capi.lib()
    P = x.data_ptr()
    assert L.cacti_b200_rope_fwd_pitched(P, P, P, P, 4, 2, 100, 96, 8, 0, capi.R_16F, None) == capi.ERR_INVALID_VALUE   # pitch < head_dim
    assert L.cacti_b200_rope_fwd_pitched(P, P, P, P, 4, 2, 102, 128, 8, 0, capi.R_16F, None) == capi.ERR_SHAPE
    assert L.cacti_b200_rope_fwd_pitched(P, P, P, P, 4, 2, 100, 128, 8, 0, capi.R_32F, None) == capi.ERR_DTYPE


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("rows,cols", [(1, 8), (37, 3200), (300, 104), (64, 8192), (5, 20000), (9, 7), (16, 3201)])
def test_add_rmsnorm_fwd_equals_separate_steps(cuda, dtype, rows, cols):
    """The residual add fused into the norm gives the bits of add followed by rmsnorm_fwd (and the oracle's values);
    shapes that fall back to two launches included; in-place sum."""
    kind = KIND[np.dtype(dtype)]
    a, b = R.normal(90, (rows, cols), dtype), R.normal(91, (rows, cols), dtype, 0.3)
    gm = R.normal(92, (cols,), dtype, 0.5) + dtype(1)
    total_ref = ops.add(dev(a), dev(b))
    y_ref = ops.rmsnorm_fwd(total_ref, dev(gm), 1e-6)
    y, total = ops.add_rmsnorm_fwd(dev(a), dev(b), dev(gm), 1e-6)
    assert torch.equal(total.view(torch.uint8), total_ref.view(torch.uint8))
    assert torch.equal(y.view(torch.uint8), y_ref.view(torch.uint8))
    assert_close(host(y), R.ref_rmsnorm_fwd((a + b).astype(dtype), gm, 1e-6)[0], kind, "fused add + norm")
    inplace = dev(a)
    y2, t2 = ops.add_rmsnorm_fwd(inplace, dev(b), dev(gm), 1e-6, total=inplace)
    assert t2.data_ptr() == inplace.data_ptr() and torch.equal(y2.view(torch.uint8), y_ref.view(torch.uint8))
    assert torch.equal(inplace.view(torch.uint8), total_ref.view(torch.uint8))


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("rows,cols,mask", [(1, 1, None), (3, 2, None), (33, 7, (1, 7, 0)), (5, 8, None),
                                            (6, 9, (2, 3, 0)), (4, 100, (1, 4, 50)), (33, 104, None),
                                            (64, 256, (1, 64, 0)), (16, 2048, (4, 4, 1000)), (7, 2056, None),
                                            (5, 4096, (1, 5, 3000)), (3, 33000, None), (2, 70000, (1, 2, 10))])
def test_softmax_shapes(cuda, dtype, rows, cols, mask):
    kind = KIND[np.dtype(dtype)]
    s = R.normal(30, (rows, cols), dtype, 0.5)
    dp = R.normal(31, (rows, cols), dtype)
    keep = R.causal_keep_mask(rows, cols, *mask) if mask else None
    p, ds = ops.softmax_fwd_bwd(dev(s), dev(dp), mask)
    rp, _ = R.ref_softmax_fwd(s, keep)
    rds = R.ref_softmax_bwd(s, dp, keep)
    assert_close(host(p), rp, kind, "P")
    assert_close(host(ds), rds, kind, "dS")
    if keep is not None:
        assert (bits(host(p))[~keep] == 0).all() and (bits(host(ds))[~keep] == 0).all()
    assert torch.equal(ops.softmax_fwd(dev(s), mask), p)
    assert torch.equal(ops.softmax_bwd(dev(s), dev(dp), mask), ds)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("rows,cols,mask", [(64, 256, (1, 64, 0)), (600, 1024, (1, 600, 0)), (48, 2048, (4, 12, 512)),
                                            (40, 1000, (2, 20, 77)), (9, 3001, (1, 9, 1000)), (8, 64, (1, 8, -3))])
def test_softmax_trimmed_zero_fill(cuda, dtype, rows, cols, mask):
    """CACTI_B200_MASK_CAUSAL_TRIM: the same values as the causal mode up to column B(q_pos), nothing written beyond."""
    s = dev(R.normal(34, (rows, cols), dtype, 0.5))
    dp = dev(R.normal(35, (rows, cols), dtype))
    p_full, ds_full = ops.softmax_fwd_bwd(s, dp, mask)
    p = torch.full_like(s, 7.0)
    ds = torch.full_like(s, 7.0)
    ops.softmax_fwd_bwd(s, dp, mask + (True,), p=p, ds=ds)
    q_div, q_mod, q_off = mask
    q = (torch.arange(rows, device="cuda") // q_div) % q_mod + q_off
    bound = torch.where(torch.tensor(q_off % 256 == 0, device="cuda"), q // 256 * 256 + 256, (q + 320 + 7) // 8 * 8)
    bound = torch.where(q < 0, cols, bound)                       # all-masked rows are written in full (NaN)
    written = torch.arange(cols, device="cuda")[None, :] < bound[:, None]
    for got, full in ((p, p_full), (ds, ds_full)):
        assert torch.equal(torch.where(written, got, 0).view(torch.uint8), torch.where(written, full, 0).view(torch.uint8))
        assert (got[~written] == 7.0).all()
    p1 = torch.full_like(s, 7.0)
    ops.softmax_fwd(s, mask + (True,), p=p1)
    assert torch.equal(p1.view(torch.uint8), p.view(torch.uint8))
    ds1 = torch.full_like(s, 7.0)
    ops.softmax_bwd(s, dp, mask + (True,), ds=ds1)
    assert torch.equal(ds1.view(torch.uint8), ds.view(torch.uint8))


def test_softmax_unaligned_accumulate_bf16_dead_rows(cuda):
    a = G.inputs(3)
    s, dp = offset_view(a["s"], 1), offset_view(a["dp"], 5)
    p, ds = ops.softmax_fwd_bwd(s, dp, a["mask"])
    assert_close(host(p), GOLD["c3_p"], "float16", "P (unaligned)")
    assert_close(host(ds), GOLD["c3_ds"], "float16", "dS (unaligned)")
    for sin_, dpin in ((dev(a["s"]), dev(a["dp"])), (s, dp)):
        old = R.normal(79, a["s"].shape, np.float16)
        acc = dev(old)
        ops.softmax_bwd(sin_, dpin, a["mask"], ds=acc, beta=1)
        assert_close(host(acc), old + GOLD["c3_ds"], "float16", "dS accumulate", floor_frac=1.0)
    sb = R.bf16_round(R.normal(32, (9, 512), scale=0.5))
    db = R.bf16_round(R.normal(33, (9, 512)))
    p, ds = ops.softmax_fwd_bwd(dev(sb, bf16=True), dev(db, bf16=True), (1, 9, 100))
    keep = R.causal_keep_mask(9, 512, 1, 9, 100)
    rp, rds = R.ideal64_softmax(sb, db, keep)
    assert_close(host(p), rp, "bfloat16", "bf16 P")
    assert_close(host(ds), rds, "bfloat16", "bf16 dS")
    # rows whose every column is masked (q_pos < 0): the reference chain yields NaN (exp(-inf - -inf))
    for cols in (64, 70):
        p, ds = ops.softmax_fwd_bwd(dev(R.normal(1, (4, cols), np.float16)), dev(R.normal(2, (4, cols), np.float16)), (1, 4, -2))
        hp = host(p)
        assert np.isnan(hp[:2]).all() and np.isnan(host(ds)[:2]).all() and not np.isnan(hp[2:]).any()


def test_softmax_config2_properties(cuda):
    """benchmark config 2 at full size [1,32,2048,2048] f16: size-independent properties + sampled rows."""
    rows, cols = 32 * 2048, 2048
    gen = torch.Generator(device="cuda").manual_seed(0)
    s = (torch.randn(rows, cols, device="cuda", generator=gen) * 0.1).half()
    dp = torch.randn(rows, cols, device="cuda", generator=gen).half()
    for mask in ((1, 2048, 0), (32, 2048, 0)):         # [B,H,Sq,Sk] and the reference's [B,Sq,H,Sk]
        p, ds = ops.softmax_fwd_bwd(s, dp, mask)
        q = (torch.arange(rows, device="cuda") // mask[0]) % mask[1]
        keep = torch.arange(cols, device="cuda")[None, :] <= q[:, None]
        assert (p[~keep].view(torch.int16) == 0).all() and (ds[~keep].view(torch.int16) == 0).all()
        assert (p.float().sum(-1) - 1).abs().max().item() < 2e-3          # rows sum to 1 (f16 rounding noise)
        assert ds.float().sum(-1).abs().max().item() < 2e-2               # sum_j dS_j = 0
        idx = np.array([0, 1, 31, 32, 2047, 2048, 40000, rows - 1])
        sh, dph = host(s[idx]), host(dp[idx])
        kh = host(keep[idx])
        rp, _ = R.ref_softmax_fwd(sh, kh)
        rds = R.ref_softmax_bwd(sh, dph, kh)
        assert_close(host(p[idx]), rp, "float16", "P sampled rows")
        assert_close(host(ds[idx]), rds, "float16", "dS sampled rows")


# ------------------------------------------------------------------------------------------- K3
def test_rope_golden_and_tables(cuda):
    a = G.inputs(5)
    cos, sin = ops.rope_tables(a["seq"], 100, a["theta"])
    # device powf/cosf/sinf vs the host's: one fp16 ulp
    assert_close(host(cos), GOLD["c5_cos"], "float16", "cos table", rtol=2.0 ** -10, floor_frac=1.0)
    assert_close(host(sin), GOLD["c5_sin"], "float16", "sin table", rtol=2.0 ** -10, floor_frac=1.0)
    c, s = dev(GOLD["c5_cos"]), dev(GOLD["c5_sin"])
    x, dy = dev(a["x"]), dev(a["dy"])
    y = ops.rope_fwd(x, c, s)
    dx = ops.rope_bwd(dy, c, s)
    y2, dx2 = ops.rope_fwd_bwd(x, dy, c, s)
    # same f16 op sequence as the reference chain: bit-exact
    assert np.array_equal(bits(host(y)), bits(GOLD["c5_y"]))
    assert np.array_equal(bits(host(dx)), bits(GOLD["c5_dx"]))
    assert torch.equal(y, y2) and torch.equal(dx, dx2)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("tokens,heads,hd,seq,off", [(1, 1, 2, 1, 0), (5, 3, 6, 4, 0), (7, 2, 8, 3, 2), (9, 32, 100, 4, 1),
                                                     (4, 5, 128, 8, 0), (3, 3, 10, 2, 0), (6, 4, 104, 16, 5)])
def test_rope_shapes(cuda, dtype, tokens, heads, hd, seq, off):
    kind = KIND[np.dtype(dtype)]
    x = R.normal(40, (tokens, heads, hd), dtype)
    dy = R.normal(41, (tokens, heads, hd), dtype)
    cos, sin = R.ref_rope_tables(seq, hd, 10000.0, dtype)
    pos = (np.arange(tokens) + off) % seq
    y, dx = ops.rope_fwd_bwd(dev(x), dev(dy), dev(cos), dev(sin), pos_off=off)
    ry, rdx = R.ref_rope_fwd(x, cos, sin, pos), R.ref_rope_bwd(dy, cos, sin, pos)
    if dtype == np.float16:
        assert_close(host(y), ry, kind, "y", floor_frac=1.0)
        assert_close(host(dx), rdx, kind, "dx", floor_frac=1.0)
        mism = (bits(host(y)) != bits(ry)).mean()
        assert mism < 1e-3, mism          # element-wise path double-rounds the add in rare ties
    else:
        assert np.array_equal(bits(host(y)), bits(ry)) and np.array_equal(bits(host(dx)), bits(rdx))
    assert torch.equal(ops.rope_fwd(dev(x), dev(cos), dev(sin), pos_off=off), y)
    old = R.normal(42, x.shape, dtype)
    acc = dev(old)
    ops.rope_bwd(dev(dy), dev(cos), dev(sin), pos_off=off, dx=acc, beta=1)
    assert_close(host(acc), old + rdx, kind, "dx accumulate", floor_frac=1.0)


def test_rope_unaligned_and_bf16(cuda):
    a = G.inputs(5)
    c, s = dev(GOLD["c5_cos"]), dev(GOLD["c5_sin"])
    y, dx = ops.rope_fwd_bwd(offset_view(a["x"], 1), offset_view(a["dy"], 2), c, s)
    assert_close(host(y), GOLD["c5_y"], "float16", "y (unaligned)", floor_frac=1.0)
    assert_close(host(dx), GOLD["c5_dx"], "float16", "dx (unaligned)", floor_frac=1.0)
    x = R.bf16_round(R.normal(43, (12, 4, 100)))
    dy = R.bf16_round(R.normal(44, (12, 4, 100)))
    cos32, sin32 = R.ref_rope_tables(8, 100, 10000.0, np.float32)
    cb, sb = R.bf16_round(cos32), R.bf16_round(sin32)
    pos = np.arange(12) % 8
    y, dx = ops.rope_fwd_bwd(dev(x, bf16=True), dev(dy, bf16=True), dev(cb, bf16=True), dev(sb, bf16=True))
    ry, rdx = R.ideal64_rope(x, dy, cb, sb, pos)
    assert_close(host(y), ry, "bfloat16", "bf16 y", floor_frac=1.0)
    assert_close(host(dx), rdx, "bfloat16", "bf16 dx", floor_frac=1.0)


# ------------------------------------------------------------------------------------------- K4
def test_swiglu_golden(cuda):
    a = G.inputs(6)
    g, u, dh = dev(a["gate"]), dev(a["up"]), dev(a["dh"])
    h = ops.swiglu_fwd(g, u)
    dg, du = ops.swiglu_bwd(g, u, dh)
    h2, dg2, du2 = ops.swiglu_fwd_bwd(g, u, dh)
    assert torch.equal(h, h2) and torch.equal(dg, dg2) and torch.equal(du, du2)
    for got, name in ((h, "h"), (dg, "dgate"), (du, "dup")):
        assert_close(host(got), GOLD[f"c6_{name}"], "float16", name)
        mism = (bits(host(got)) != bits(GOLD[f"c6_{name}"])).mean()
        assert mism < 5e-3, (name, mism)       # approximate exp / reciprocal flip a rounding in rare cases


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("n", [1, 7, 8, 9, 100, 1000, 4099, 8640 * 3 + 5])
def test_swiglu_shapes(cuda, dtype, n):
    kind = KIND[np.dtype(dtype)]
    g, u, dh = R.normal(50, (n,), dtype), R.normal(51, (n,), dtype), R.normal(52, (n,), dtype)
    h, dg, du = ops.swiglu_fwd_bwd(dev(g), dev(u), dev(dh))
    rh, _ = R.ref_swiglu_fwd(g, u)
    rdg, rdu = R.ref_swiglu_bwd(g, u, dh)
    assert_close(host(h), rh, kind, "h")
    assert_close(host(dg), rdg, kind, "dg")
    assert_close(host(du), rdu, kind, "du")
    # unaligned views and accumulate
    h2, dg2, du2 = ops.swiglu_fwd_bwd(offset_view(g, 1), offset_view(u, 3), offset_view(dh, 5))
    assert_close(host(h2), rh, kind, "h (unaligned)")
    assert_close(host(dg2), rdg, kind, "dg (unaligned)")
    old_g, old_u = R.normal(53, (n,), dtype), R.normal(54, (n,), dtype)
    ag, au = dev(old_g), dev(old_u)
    ops.swiglu_bwd(dev(g), dev(u), dev(dh), dgate=ag, dup=au, beta_dgate=1, beta_dup=1)
    assert_close(host(ag), old_g + rdg, kind, "dg accumulate", floor_frac=1.0)
    assert_close(host(au), old_u + rdu, kind, "du accumulate", floor_frac=1.0)


def test_swiglu_bf16_and_extremes(cuda):
    g, u, dh = (R.bf16_round(R.normal(s, (5000,), scale=2.0)) for s in (55, 56, 57))
    h, dg, du = ops.swiglu_fwd_bwd(dev(g, bf16=True), dev(u, bf16=True), dev(dh, bf16=True))
    rh, rdg, rdu = R.ideal64_swiglu(g, u, dh)
    assert_close(host(h), rh, "bfloat16", "bf16 h")
    assert_close(host(dg), rdg, "bfloat16", "bf16 dg")
    assert_close(host(du), rdu, "bfloat16", "bf16 du")
    # f16 saturation: exp(-g) overflows f16 for g < -11.09; the chain yields y = -0, t = 0
    g = np.array([-60000, -100, -12, -11, 0, 11, 12, 100, 60000], dtype=np.float16).repeat(8)
    u = np.ones_like(g)
    dh = np.ones_like(g)
    with np.errstate(over="ignore"):
        rh, _ = R.ref_swiglu_fwd(g, u)
        rdg, rdu = R.ref_swiglu_bwd(g, u, dh)
    h, dg, du = ops.swiglu_fwd_bwd(dev(g), dev(u), dev(dh))
    assert_close(host(h), rh, "float16", "h extremes")
    assert_close(host(dg), rdg, "float16", "dg extremes")
    assert_close(host(du), rdu, "float16", "du extremes")


# ------------------------------------------------------------------------------------------- K5
def test_nll_golden(cuda):
    a = G.inputs(7)
    lg = dev(a["logits"])
    for tg in (dev(a["targets"]), dev(a["targets"].astype(np.uint16))):
        ls, lr, d, st = ops.softmax_nll_fwd_bwd(lg, tg, w_scalar=float(a["w"]))
        assert host(st)[0] == 0
        assert_close(host(lr), GOLD["c7_loss_rows"], "float32", "loss rows")
        assert_close(host(ls), GOLD["c7_loss_sum"].reshape(1), "float32", "loss sum")
        assert_close(host(d), GOLD["c7_dlogits"], "float16", "dlogits")
    # gathered logit: the value the loss was formed from is the stored bit pattern
    picked = host(lg)[np.arange(3), a["targets"]]
    assert np.array_equal(bits(picked), bits(GOLD["c7_picked"]))
    # forward only, per-row weights, loss_sum without loss_rows (workspace path)
    w = dev(np.array([0.5, 0.25, 2.0], dtype=np.float32))
    ls, lr, d, _ = ops.softmax_nll_fwd_bwd(lg, dev(a["targets"]), w=w, want_grad=False, want_rows=False)
    assert d is None and lr is None
    assert_close(host(ls), (GOLD["c7_loss_rows"] * host(w)).sum(dtype=np.float32).reshape(1), "float32", "weighted sum")


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("rows,vocab", [(1, 1), (3, 2), (5, 7), (33, 8), (4, 100), (3, 1000), (9, 4096), (2, 32000),
                                        (2, 32001), (1, 65536), (2, 70001)])
def test_nll_shapes(cuda, dtype, rows, vocab):
    kind = KIND[np.dtype(dtype)]
    lg = R.normal(60, (rows, vocab), dtype, 2.0)
    tg = R.uniform_int(61, rows, vocab)
    w = np.float32(1.0 / rows)
    ls, lr, d, st = ops.softmax_nll_fwd_bwd(dev(lg), dev(tg), w_scalar=float(w))
    rl, rd, _ = R.ref_softmax_nll(lg, tg, w)
    assert host(st)[0] == 0
    assert_close(host(lr), rl, "float32", "loss rows", floor_frac=1.0)
    assert_close(host(ls), np.array([(rl * w).sum(dtype=np.float32)]), "float32", "loss sum")
    assert_close(host(d), rd, kind, "dlogits")
    old = R.normal(62, (rows, vocab), dtype)
    acc = dev(old)
    ops.softmax_nll_fwd_bwd(dev(lg), dev(tg), w_scalar=float(w), dlogits=acc, beta=1)
    assert_close(host(acc), old + rd, kind, "dlogits accumulate", floor_frac=1.0)


def test_nll_out_of_range_target_sets_status(cuda):
    lg = R.normal(63, (4, 64), np.float16)
    for bad in (64, -1):
        tg = np.array([1, bad, 3, 5], dtype=np.int32)
        ls, lr, d, st = ops.softmax_nll_fwd_bwd(dev(lg), dev(tg))
        assert host(st)[0] == capi.ERR_INDEX_RANGE
        hl = host(lr)
        assert np.isnan(hl[1]) and not np.isnan(hl[[0, 2, 3]]).any()
        torch.cuda.synchronize()          # the context is intact: nothing trapped
    good = np.array([1, 2, 3, 5], dtype=np.int32)
    _, lr, _, st = ops.softmax_nll_fwd_bwd(dev(lg), dev(good))
    assert host(st)[0] == 0 and not np.isnan(host(lr)).any()


def test_nll_config3_properties(cuda):
    """benchmark config 3 at full size: [8192 x 32000] f16 logits ~ N(0, 2^2), int32 targets, mean loss."""
    rows, vocab = 8192, 32000
    gen = torch.Generator(device="cuda").manual_seed(0)
    lg = (torch.randn(rows, vocab, device="cuda", generator=gen) * 2).half()
    tg = torch.randint(0, vocab, (rows,), device="cuda", generator=gen, dtype=torch.int32)
    # property run with w = 1 (with w = 1/8192 most f16 gradient entries are below the f16 subnormal range):
    # sum_j dlogits_ij = sum y - 1 = 0, and the target entry is the only negative one
    _, _, d1, st = ops.softmax_nll_fwd_bwd(lg, tg, w_scalar=1.0)
    assert host(st)[0] == 0
    assert d1.float().sum(-1).abs().max().item() < 2e-3
    assert ((d1 < 0).sum(-1) == 1).all() and (d1[torch.arange(rows), tg.long()] < 0).all()
    del d1
    ls, lr, d, st = ops.softmax_nll_fwd_bwd(lg, tg, w_scalar=1.0 / rows)
    assert host(st)[0] == 0
    idx = np.array([0, 1, 4095, 8191])
    rl, rd, _ = R.ref_softmax_nll(host(lg[idx]), host(tg)[idx], np.float32(1.0 / rows))
    assert_close(host(lr[idx]), rl, "float32", "loss sampled rows")
    assert_close(host(d[idx]), rd, "float16", "dlogits sampled rows")
    assert_close(host(ls), np.array([host(lr).astype(np.float64).sum() / rows], dtype=np.float32), "float32", "mean loss")


# ------------------------------------------------------------------------------------------- K6 / K7
@pytest.mark.parametrize("tok_dtype", [np.int32, np.uint16])
def test_gather_scatter_golden(cuda, tok_dtype):
    a = G.inputs(8)
    tk = dev(a["tokens"].astype(tok_dtype))
    out, st = ops.gather_rows(dev(a["table"]), tk)
    assert host(st)[0] == 0 and np.array_equal(bits(host(out)), bits(GOLD["c8_out"]))
    dt, st = ops.scatter_add_rows(dev(a["dy"]), tk, 50)
    assert host(st)[0] == 0
    assert_close(host(dt), GOLD["c8_dtable"], "float16", "dtable")
    old = R.normal(80, (50, 64), np.float16)
    acc = dev(old)
    ops.scatter_add_rows(dev(a["dy"]), tk, 50, dtable=acc, beta=1)
    assert_close(host(acc), old + GOLD["c8_dtable"], "float16", "dtable accumulate", floor_frac=1.0)
    dt2, _ = ops.scatter_add_rows(dev(a["dy"]), tk, 50)
    assert torch.equal(dt, dt2)          # run-to-run identical


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("n,vocab,cols", [(1, 1, 1), (5, 3, 7), (100, 10, 8), (3000, 17, 100), (2048, 32000, 3200)])
def test_gather_scatter_shapes(cuda, dtype, n, vocab, cols):
    kind = KIND[np.dtype(dtype)]
    table = R.normal(81, (vocab, cols), dtype)
    tok = R.uniform_int(82, n, vocab)
    dy = R.normal(83, (n, cols), dtype)
    out, st = ops.gather_rows(dev(table), dev(tok))
    assert np.array_equal(bits(host(out)), bits(table[tok]))
    out2, _ = ops.gather_rows(offset_view(table, 1), dev(tok))
    assert np.array_equal(bits(host(out2)), bits(table[tok]))
    dt, st = ops.scatter_add_rows(dev(dy), dev(tok), vocab)
    ref = np.zeros((vocab, cols), dtype=np.float64)
    np.add.at(ref, tok, dy.astype(np.float64))
    assert_close(host(dt), ref.astype(dtype), kind, "dtable")


def test_gather_out_of_range_token(cuda):
    table = R.normal(84, (10, 16), np.float16)
    tok = np.array([1, 10, 3], dtype=np.int32)
    out = dev(np.zeros((3, 16), np.float16))
    _, st = ops.gather_rows(dev(table), dev(tok), out=out)
    assert host(st)[0] == capi.ERR_INDEX_RANGE
    h = host(out)
    assert np.array_equal(h[0], table[1]) and (h[1] == 0).all() and np.array_equal(h[2], table[3])
    dt, st = ops.scatter_add_rows(dev(R.normal(85, (3, 16), np.float16)), dev(tok), 10)
    assert host(st)[0] == capi.ERR_INDEX_RANGE
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("n", [1, 7, 8, 1000, 3200 * 33 + 3])
def test_add_accumulate(cuda, dtype, n):
    a, b = R.normal(90, (n,), dtype), R.normal(91, (n,), dtype)
    assert np.array_equal(bits(host(ops.add(dev(a), dev(b)))), bits(a + b))
    assert np.array_equal(bits(host(ops.add(offset_view(a, 1), offset_view(b, 2)))), bits(a + b))
    d = dev(a)
    ops.accumulate(d, dev(b))
    assert np.array_equal(bits(host(d)), bits(a + b))
    ab, bb = R.bf16_round(a.astype(np.float32)), R.bf16_round(b.astype(np.float32))
    got = host(ops.add(dev(ab, bf16=True), dev(bb, bf16=True)))
    assert np.array_equal(got, R.bf16_round(ab + bb))


# ------------------------------------------------------------------------------------------- config 4 at full size
def test_config4_properties(cuda):
    """benchmark config 4: RoPE on [16384 x 32 x 100] f16 and SwiGLU on [16384 x 8640] f16."""
    gen = torch.Generator(device="cuda").manual_seed(0)
    tokens, heads, hd, seq = 16384, 32, 100, 2048
    cos, sin = ops.rope_tables(seq, hd)
    x = torch.randn(tokens, heads, hd, device="cuda", generator=gen).half()
    dy = torch.randn(tokens, heads, hd, device="cuda", generator=gen).half()
    y, dx = ops.rope_fwd_bwd(x, dy, cos, sin)
    # a rotation preserves the norm of every (j, j+hd/2) pair, and backward is its inverse: bwd(fwd(x)) = x
    n_in = x.float().pow(2).sum(-1)
    n_out = y.float().pow(2).sum(-1)
    assert ((n_out - n_in).abs() / n_in).max().item() < 5e-3
    back = ops.rope_bwd(y, cos, sin)
    assert (back.float() - x.float()).abs().max().item() < 8e-3
    idx = np.array([0, 1, 2047, 2048, 9999, tokens - 1])
    ch, sh = host(cos), host(sin)
    assert np.array_equal(bits(host(y[idx])), bits(R.ref_rope_fwd(host(x[idx]), ch, sh, idx % seq)))
    assert np.array_equal(bits(host(dx[idx])), bits(R.ref_rope_bwd(host(dy[idx]), ch, sh, idx % seq)))
    del x, dy, y, dx, back
    n = 16384 * 8640
    g = torch.randn(n, device="cuda", generator=gen).half()
    u = torch.randn(n, device="cuda", generator=gen).half()
    dh = torch.randn(n, device="cuda", generator=gen).half()
    h, dg, du = ops.swiglu_fwd_bwd(g, u, dh)
    for lo in (0, 8640 * 5000 + 3, n - 4096):
        sl = slice(lo, lo + 4096)
        rh, _ = R.ref_swiglu_fwd(host(g[sl]), host(u[sl]))
        rdg, rdu = R.ref_swiglu_bwd(host(g[sl]), host(u[sl]), host(dh[sl]))
        assert_close(host(h[sl]), rh, "float16", "h slice")
        assert_close(host(dg[sl]), rdg, "float16", "dg slice")
        assert_close(host(du[sl]), rdu, "float16", "du slice")
    # linearity in the upstream gradient: dg(2 dh) = 2 dg(dh) exactly in f16 (power-of-two scaling)
    # (away from the f16 subnormal range, where doubling before or after a rounding differs)
    dg2, du2 = ops.swiglu_bwd(g, u, dh * 2)
    assert ((dg2 != dg * 2) & (dg.abs() > 1e-2)).float().mean().item() < 1e-5
    assert ((du2 != du * 2) & (du.abs() > 1e-2)).float().mean().item() < 1e-5
