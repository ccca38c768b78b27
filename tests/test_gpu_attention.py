"""GPU parity tests of the fused causal attention forward and of block_pad.

Oracle: the reference chain in f64 with its rounding points (scores rounded to the storage type, softmax in f32 on
the rounded scores; src/librarium/llama.rs:501-507).  Tolerance: the block matmul's, 2e-3 relative to max(|ref|, rms),
measured against max(|ref|, sum_j p_j |v_j|): the context is a sum of 16-bit-rounded probabilities times V, each
term carrying a relative rounding error of 2^-12 (in the reference's own chain as well), so the error scales with the
sum of magnitudes, not with the possibly cancelled result."""
import ctypes as C

import numpy as np
import pytest
import torch

from cacti_b200 import capi, ops
from oracle import ref_chain as R
from tests.gpu_util import dev, host
from tests.tolerances import assert_close

pytestmark = pytest.mark.gpu


ref_attention = R.ref_causal_attention


@pytest.mark.parametrize("ncol,rows", [(3, 37), (32, 700)])
@pytest.mark.parametrize("cols,cols_pad", [(100, 128), (64, 128), (7, 16), (128, 128), (30, 33)])
def test_block_pad(cuda, cols, cols_pad, ncol, rows):
    """Rows of whole blocks that are multiples of 16 bytes take the staged kernel (32 blocks of 100: 6400-byte rows, 1400
    of them: every ring slot is reused), the others the per-thread kernels."""
    x = dev(R.normal(70, (2, rows, ncol, cols), np.float16))
    y = ops.block_pad(x, cols_pad)
    assert torch.equal(y[..., :cols], x) and (y[..., cols:] == 0).all()
    L = capi.lib()
    assert L.cacti_b200_block_pad(y.data_ptr(), x.data_ptr(), 2, rows, ncol, cols, cols - 1, capi.R_16F, None) == capi.ERR_INVALID_VALUE
    assert L.cacti_b200_block_pad(y.data_ptr(), x.data_ptr(), 2, rows, ncol, cols, cols_pad, capi.R_32F, None) == capi.ERR_DTYPE


@pytest.mark.parametrize("bsz,s,h,hd", [(1, 128, 1, 128), (2, 256, 3, 100), (1, 640, 2, 64), (2, 1024, 2, 100)])
def test_attention_fwd(cuda, bsz, s, h, hd):
    q = R.normal(71, (bsz, s, h, hd), np.float16)
    k = R.normal(72, (bsz, s, h, hd), np.float16)
    v = R.normal(73, (bsz, s, h, hd), np.float16)
    alpha = float(1.0 / np.sqrt(hd))
    qp, kp, vp = (ops.block_pad(dev(t), 128) for t in (q, k, v))
    ctx, stats = ops.attention_fwd(qp, kp, vp, hd, alpha)
    torch.cuda.synchronize()
    err = C.c_uint(7)
    assert capi.lib().cacti_b200_device_error(C.byref(err)) == capi.OK and err.value == 0
    rctx, rm, rl, mag = ref_attention(q, k, v, alpha)
    assert_close(host(ctx), rctx, "float16", f"fused attention ctx B={bsz} S={s} H={h} hd={hd}", floor_frac=1.0, floor_abs=mag)
    st = host(stats)
    # the row maximum is a maximum of 16-bit values: exact unless the fp32 accumulation order moved a score by one ulp
    assert np.abs(st[..., 0] - rm).max() <= 2.0 ** -9 * np.abs(rm).max()
    assert np.abs(st[..., 1] / (rl * np.exp(rm - st[..., 0])) - 1).max() < 2e-3
    # and against the unfused entry points on the same inputs
    sc = ops.block_gemm(dev(q), dev(k), False, True, alpha=alpha)
    pr = ops.softmax_fwd(sc.view(-1, s), (h, s, 0)).view(bsz, s, h, s)
    unfused = ops.block_gemm(pr, dev(v), False, False)
    # both sides carry their own 16-bit roundings: twice the tolerance of one
    assert_close(host(ctx), host(unfused).astype(np.float64), "float16", "fused vs unfused chain", rtol=4e-3, floor_frac=1.0,
                 floor_abs=mag)


@pytest.fixture
def two_pass_forward():
    """Run attention_fwd on the two-pass kernel (scores formed twice, exact maximum first) for the duration of a test."""
    L = capi.lib()
    assert L.cacti_b200_tune(b"attn_fwd_single", 0) == capi.OK
    yield
    assert L.cacti_b200_tune(b"attn_fwd_single", 1) == capi.OK


@pytest.mark.parametrize("bsz,s,h,hd", [(2, 256, 3, 100), (1, 640, 2, 64)])
def test_attention_fwd_two_pass_kernel(cuda, two_pass_forward, bsz, s, h, hd):
    test_attention_fwd(cuda, bsz, s, h, hd)


@pytest.fixture
def one_item_per_cta():
    """Run the single-pass forward as one CTA per (batch, query tile, head) instead of the persistent walk."""
    L = capi.lib()
    assert L.cacti_b200_tune(b"attn_fwd_persistent", 0) == capi.OK and L.cacti_b200_tune(b"attn_fwd_pair", 0) == capi.OK
    yield
    assert L.cacti_b200_tune(b"attn_fwd_persistent", 1) == capi.OK and L.cacti_b200_tune(b"attn_fwd_pair", 1) == capi.OK


@pytest.mark.parametrize("bsz,s,h,hd", [(2, 256, 3, 100), (1, 640, 2, 64)])
def test_attention_fwd_one_item_per_cta(cuda, one_item_per_cta, bsz, s, h, hd):
    test_attention_fwd(cuda, bsz, s, h, hd)


@pytest.fixture
def pair_forward():
    """Two query tiles per CTA, one per softmax group (the default wherever the number of query tiles is even)."""
    L = capi.lib()
    assert L.cacti_b200_tune(b"attn_fwd_persistent", 0) == capi.OK and L.cacti_b200_tune(b"attn_fwd_pair", 1) == capi.OK
    yield
    assert L.cacti_b200_tune(b"attn_fwd_persistent", 1) == capi.OK


@pytest.mark.parametrize("bsz,s,h,hd", [(1, 256, 1, 128), (2, 256, 3, 100), (1, 512, 2, 64), (2, 1024, 2, 100), (1, 2048, 3, 100)])
def test_attention_fwd_pair_kernel(cuda, pair_forward, bsz, s, h, hd):
    test_attention_fwd(cuda, bsz, s, h, hd)


@pytest.fixture
def no_pair_forward():
    L = capi.lib()
    assert L.cacti_b200_tune(b"attn_fwd_pair", 0) == capi.OK
    yield
    assert L.cacti_b200_tune(b"attn_fwd_pair", 1) == capi.OK


@pytest.mark.parametrize("bsz,s,h,hd", [(2, 1024, 2, 100)])
def test_attention_fwd_one_tile_per_cta_long(cuda, no_pair_forward, bsz, s, h, hd):
    test_attention_fwd(cuda, bsz, s, h, hd)


@pytest.fixture
def always_persistent():
    L = capi.lib()
    assert L.cacti_b200_tune(b"attn_fwd_persistent", 2) == capi.OK
    yield
    assert L.cacti_b200_tune(b"attn_fwd_persistent", 1) == capi.OK


@pytest.mark.parametrize("bsz,s,h,hd", [(1, 640, 2, 64), (2, 1024, 2, 100)])
def test_attention_fwd_persistent_long_sequences(cuda, always_persistent, bsz, s, h, hd):
    test_attention_fwd(cuda, bsz, s, h, hd)


def test_attention_fwd_persistent_walk_many_items(cuda):
    """More items than SMs can hold at once, of every length from 1 to 8 key tiles, so that every CTA of the persistent
    kernel walks several items (odd and even tile counts: the tile parity that selects ring slot, softmax group and
    accumulator carries over from item to item), against the oracle and the one-item-per-CTA form (which of the two
    groups takes a tile may differ between the two forms, hence the rounding: same row maxima, the rest to tolerance)."""
    bsz, s, h, hd = 3, 1024, 25, 100             # 600 items on at most 148 CTAs
    q, k, v = (dev(R.normal(60 + i, (bsz, s, h, hd), np.float16)) for i in range(3))
    alpha = float(1.0 / np.sqrt(hd))
    qp, kp, vp = (ops.block_pad(t, 128) for t in (q, k, v))
    L = capi.lib()
    assert L.cacti_b200_tune(b"attn_fwd_persistent", 2) == capi.OK          # always (the default takes it for seq <= 512 only)
    try:
        ctx_p, st_p = ops.attention_fwd(qp, kp, vp, hd, alpha)
        assert L.cacti_b200_tune(b"attn_fwd_persistent", 0) == capi.OK
        ctx_1, st_1 = ops.attention_fwd(qp, kp, vp, hd, alpha)
    finally:
        L.cacti_b200_tune(b"attn_fwd_persistent", 1)
    torch.cuda.synchronize()
    err = C.c_uint(7)
    assert L.cacti_b200_device_error(C.byref(err)) == capi.OK and err.value == 0
    rctx, rm, rl, mag = ref_attention(host(q), host(k), host(v), alpha)
    for name, ctx_, st_ in (("persistent", ctx_p, st_p), ("one item per CTA", ctx_1, st_1)):
        assert_close(host(ctx_), rctx, "float16", f"many items, {name}", floor_frac=1.0, floor_abs=mag)
        st = host(st_)
        assert np.abs(st[..., 0] - rm).max() <= 2.0 ** -9 * np.abs(rm).max()
        assert np.abs(st[..., 1] / (rl * np.exp(rm - st[..., 0])) - 1).max() < 2e-3
    assert torch.equal(st_p[..., 0], st_1[..., 0])
    assert_close(host(ctx_p), host(ctx_1).astype(np.float64), "float16", "persistent vs one item per CTA", rtol=4e-3,
                 floor_frac=1.0, floor_abs=mag)


@pytest.mark.parametrize("sign", [1.0, -1.0])
@pytest.mark.parametrize("s,hd", [(640, 64), (1024, 100)])
def test_attention_fwd_moving_maximum(cuda, s, hd, sign):
    """Scores that grow by about ten per key tile (alternating tiles by twice that), so that in the single-pass kernel
    each group's exponent reference has to move again and again and its accumulated rows are rescaled in tensor memory;
    also with a negative alpha (the sign-folded maximum).  Against the oracle, and against the two-pass kernel."""
    bsz, h = 1, 2
    alpha = sign / 8.0
    rng = np.random.default_rng(77)
    # q in eighths, k in 64ths, alpha a power of two: every product and every partial sum of a score is exact in f32 in
    # any order, so the kernel and the oracle round the same scores to 16 bits (at scores of 30 to 100 one unit of that
    # rounding is 2 to 6 % of a probability: an accumulation-order difference would otherwise decide the comparison)
    q = ((8 + rng.integers(-1, 2, (bsz, s, h, hd))) / 8.0).astype(np.float16)
    ramp = (np.arange(s) * (10.0 / 128) * 8.0 / hd).reshape(1, s, 1, 1)           # alpha q.k grows 10 per 128 keys
    ramp = ramp * np.where((np.arange(s) // 128) % 2 == 1, 1.5, 1.0).reshape(1, s, 1, 1)
    k = (sign * np.round(ramp * (1.0 + 0.05 * rng.standard_normal((bsz, s, h, hd))) * 64) / 64).astype(np.float16)
    v = R.normal(78, (bsz, s, h, hd), np.float16)
    qp, kp, vp = (ops.block_pad(dev(t), 128) for t in (q, k, v))
    rctx, rm, rl, mag = ref_attention(q, k, v, alpha)
    assert (np.diff(rm[0, 0, ::128]) > 5.6).all()              # the maximum does move by more than 2^8 between tiles
    L = capi.lib()
    out = {}
    for single in (1, 2, 0, 3):                     # persistent single-pass, one item per CTA, two-pass, two tiles per CTA
        assert L.cacti_b200_tune(b"attn_fwd_single", 1 if single else 0) == capi.OK
        assert L.cacti_b200_tune(b"attn_fwd_persistent", 2 if single == 1 else 0) == capi.OK
        assert L.cacti_b200_tune(b"attn_fwd_pair", 1 if single == 3 else 0) == capi.OK
        try:
            ctx, stats = ops.attention_fwd(qp, kp, vp, hd, alpha)
            torch.cuda.synchronize()
        finally:
            L.cacti_b200_tune(b"attn_fwd_single", 1)
            L.cacti_b200_tune(b"attn_fwd_persistent", 1)
            L.cacti_b200_tune(b"attn_fwd_pair", 1)
        err = C.c_uint(7)
        assert L.cacti_b200_device_error(C.byref(err)) == capi.OK and err.value == 0
        assert_close(host(ctx), rctx, "float16", f"moving maximum, single={single}", floor_frac=1.0, floor_abs=mag)
        st = host(stats)
        assert np.abs(st[..., 0] - rm).max() <= 2.0 ** -9 * np.abs(rm).max()
        assert np.abs(st[..., 1] / (rl * np.exp(rm - st[..., 0])) - 1).max() < 2e-3
        out[single] = (host(ctx), st)
    assert np.array_equal(out[0][1][..., 0], out[1][1][..., 0])          # the same row maxima from both kernels
    assert np.array_equal(out[1][1][..., 0], out[2][1][..., 0])          # persistent or not: the same row maxima
    if s % 256 == 0:                                 # (an odd number of query tiles falls back to one tile per CTA)
        assert np.array_equal(out[3][1][..., 0], out[2][1][..., 0])
        assert_close(out[3][0], out[0][0].astype(np.float64), "float16", "two tiles per CTA vs two-pass", rtol=4e-3, floor_frac=1.0,
                     floor_abs=mag)
    assert_close(out[1][0], out[0][0].astype(np.float64), "float16", "single-pass vs two-pass", rtol=4e-3, floor_frac=1.0,
                 floor_abs=mag)


def test_attention_fwd_bf16_and_errors(cuda):
    bsz, s, h, hd = 1, 256, 2, 100
    q, k, v = (R.bf16_round(R.normal(80 + i, (bsz, s, h, hd))) for i in range(3))
    alpha = 0.1
    qp, kp, vp = (ops.block_pad(dev(t, bf16=True), 128) for t in (q, k, v))
    ctx, _ = ops.attention_fwd(qp, kp, vp, hd, alpha)
    ref, _, _, mag = R.ref_causal_attention(q, k, v, alpha, round_scores=R.bf16_round)
    assert_close(host(ctx), ref, "bfloat16", "bf16 fused attention", floor_frac=1.0, floor_abs=mag)
    L = capi.lib()
    P = qp.data_ptr()
    assert L.cacti_b200_attention_fwd(P, P, P, P, P, 1, 200, 2, 100, 0.1, capi.R_16F, None) == capi.ERR_SHAPE      # seq % 128
    assert L.cacti_b200_attention_fwd(P, P, P, P, P, 1, 256, 2, 130, 0.1, capi.R_16F, None) == capi.ERR_SHAPE      # head_dim
    assert L.cacti_b200_attention_fwd(P, P, P, P, P, 1, 256, 2, 100, 0.1, capi.R_32F, None) == capi.ERR_DTYPE
    assert L.cacti_b200_attention_fwd(P, P, P, P, P, 0, 256, 2, 100, 0.1, capi.R_16F, None) == capi.OK
    assert L.cacti_b200_attention_fwd(0, P, P, P, P, 1, 256, 2, 100, 0.1, capi.R_16F, None) == capi.ERR_INVALID_VALUE


@pytest.mark.parametrize("bsz,s,h,hd", [(1, 128, 1, 128), (2, 256, 3, 100), (1, 640, 2, 64), (2, 1024, 2, 100)])
def test_attention_bwd_prep(cuda, bsz, s, h, hd):
    """P and dS against the unfused entry points (scores and dP through HBM, softmax_fwd_bwd), inside the bound up to
    which they are specified; nothing is written beyond it; the three hinted block matmuls of the adjoint accept them."""
    q, k, v, do = (dev(R.normal(90 + i, (bsz, s, h, hd), np.float16)) for i in range(4))
    alpha = float(1.0 / np.sqrt(hd))
    qp, kp, vp, dop = (ops.block_pad(t, 128) for t in (q, k, v, do))
    ctx, stats = ops.attention_fwd(qp, kp, vp, hd, alpha)
    p = torch.full((bsz, s, h, s), float("nan"), dtype=torch.float16, device="cuda")
    ds = torch.full_like(p, float("nan"))
    ops.attention_bwd_prep(qp, kp, vp, dop, ctx, stats, alpha, p=p, ds=ds)
    torch.cuda.synchronize()
    err = C.c_uint(7)
    assert capi.lib().cacti_b200_device_error(C.byref(err)) == capi.OK and err.value == 0
    sc = ops.block_gemm(q, k, False, True, alpha=alpha)
    dp = ops.block_gemm(do, v, False, True)
    p_ref, ds_ref = ops.softmax_fwd_bwd(sc.view(-1, s), dp.view(-1, s), (h, s, 0))
    p_ref, ds_ref = p_ref.view(bsz, s, h, s), ds_ref.view(bsz, s, h, s)
    r = torch.arange(s, device="cuda")
    bound = r // 256 * 256 + 256
    written = (r[None, :] < bound[:, None])[None, :, None, :]
    assert torch.isnan(p[~written.expand_as(p)]).all() and torch.isnan(ds[~written.expand_as(p)]).all()
    pw, dsw = torch.where(written, p, 0), torch.where(written, ds, 0)
    assert not torch.isnan(pw).any() and not torch.isnan(dsw).any()
    keep = (r[None, :] <= r[:, None])[None, :, None, :]
    assert (pw[~keep.expand_as(p)] == 0).all() and (dsw[~keep.expand_as(p)] == 0).all()
    # P: the same formula on the same rounded scores; the row sum is accumulated in another order
    assert_close(host(pw), host(p_ref).astype(np.float64), "float16", "P", rtol=2e-3)
    # dS = y (dP - c).  c is dO . O here and sum_j y_j T(dP_j) in the unfused chain: each carries the half-ulp rounding
    # of its 16-bit inputs (O there, dP here), so the two differ by up to an ulp of the row's largest |dP|, times y
    pr, dpr = host(p_ref).astype(np.float64), host(dp).astype(np.float64)
    c = (pr * dpr).sum(-1, keepdims=True)
    mag = pr * (np.abs(dpr) + np.abs(c) + np.abs(np.where(host(keep.expand_as(p)), dpr, 0)).max(-1, keepdims=True))
    assert_close(host(dsw), host(ds_ref).astype(np.float64), "float16", "dS", rtol=4e-3, floor_abs=mag)
    # the adjoint's block matmuls on the trimmed tensors (NaN beyond the bound would poison them if read)
    dv = ops.block_gemm(p, do, True, False, tri=capi.TRI_A_UPPER)
    dq = ops.block_gemm(ds, k, False, False, alpha=alpha, tri=capi.TRI_A_LOWER)
    dk = ops.block_gemm(ds, q, True, False, alpha=alpha, tri=capi.TRI_A_UPPER)
    assert_close(host(dv), host(ops.block_gemm(p_ref, do, True, False)).astype(np.float64), "float16", "dV", rtol=4e-3, floor_frac=1.0)
    # dQ and dK: c = dO . O and the unfused chain's sum_j y_j T(dP_j) are two roundings of the same number, so the two
    # chains differ by rounding noise that no element-wise bound captures on rows with one or two keys (the unfused
    # dS of row 0 is exactly 0).  Both are measured against the exact adjoint (f64, no intermediate rounding): the
    # fused chain must be as close to it as the unfused one.
    qf, kf, vf, dof = (np.transpose(host(t).astype(np.float64), (0, 2, 1, 3)) for t in (q, k, v, do))
    sce = alpha * np.einsum("bhqd,bhkd->bhqk", qf, kf)
    sce = np.where(np.tril(np.ones((s, s), bool)), sce, -np.inf)
    pe = np.exp(sce - sce.max(-1, keepdims=True))
    pe /= pe.sum(-1, keepdims=True)
    dpe = np.einsum("bhqd,bhkd->bhqk", dof, vf)
    dse = pe * (dpe - (pe * dpe).sum(-1, keepdims=True))
    exact = {"dq": alpha * np.einsum("bhqk,bhkd->bhqd", dse, kf), "dk": alpha * np.einsum("bhqk,bhqd->bhkd", dse, qf),
             "dv": np.einsum("bhqk,bhqd->bhkd", pe, dof)}
    unfused = {"dq": ops.block_gemm(ds_ref, k, False, False, alpha=alpha), "dk": ops.block_gemm(ds_ref, q, True, False, alpha=alpha),
               "dv": ops.block_gemm(p_ref, do, True, False)}
    for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
        ex = np.transpose(exact[name], (0, 2, 1, 3))
        e_f = host(got).astype(np.float64) - ex
        e_u = host(unfused[name]).astype(np.float64) - ex
        rms_f, rms_u = np.sqrt((e_f ** 2).mean()), np.sqrt((e_u ** 2).mean())
        scale = np.sqrt((ex ** 2).mean())
        assert rms_f <= 1.5 * rms_u + 1e-4 * scale, (name, rms_f, rms_u)
        assert np.abs(e_f).max() <= 3 * np.abs(e_u).max() + 2e-3 * scale, (name, np.abs(e_f).max(), np.abs(e_u).max())


@pytest.mark.parametrize("bsz,s,h,hd", [(1, 128, 1, 128), (2, 256, 3, 100), (1, 640, 2, 64), (2, 1024, 2, 100), (1, 2048, 2, 100)])
def test_attention_bwd_fused(cuda, bsz, s, h, hd):
    """dQ, dK, dV from the two fused kernels against (a) the chain they replace, attention_bwd_prep plus the three hinted
    block matmuls (same arithmetic and rounding points: the difference is the summation order inside the tensor
    cores, bounded at twice the block matmul's tolerance against the magnitude of the summed terms), and (b) the exact
    adjoint in float64 from the definition (tests/torch_defs.py), at the tolerance the chain itself is held to."""
    from tests import torch_defs as TD
    q, k, v, do = (dev(R.normal(110 + i, (bsz, s, h, hd), np.float16)) for i in range(4))
    alpha = float(1.0 / np.sqrt(hd))
    qp, kp, vp, dop = (ops.block_pad(t, 128) for t in (q, k, v, do))
    ctx, stats = ops.attention_fwd(qp, kp, vp, hd, alpha)
    dq, dk, dv = ops.attention_bwd(qp, kp, vp, dop, ctx, stats, alpha)
    dq2, dk2, dv2 = ops.attention_bwd(qp, kp, vp, dop, ctx, stats, alpha)
    torch.cuda.synchronize()
    err = C.c_uint(7)
    assert capi.lib().cacti_b200_device_error(C.byref(err)) == capi.OK and err.value == 0
    assert torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)          # fixed summation order
    p, ds = ops.attention_bwd_prep(qp, kp, vp, dop, ctx, stats, alpha)
    chain = {"dv": ops.block_gemm(p, dop, True, False, tri=capi.TRI_A_UPPER, b_valid=hd),
             "dq": ops.block_gemm(ds, kp, False, False, alpha=alpha, tri=capi.TRI_A_LOWER, b_valid=hd),
             "dk": ops.block_gemm(ds, qp, True, False, alpha=alpha, tri=capi.TRI_A_UPPER, b_valid=hd)}
    # magnitudes of the summed terms: dS = y (dP - c) is a difference, good to a few 2^-11 of y (|dP| + |c|) (c is dO . O
    # in both chains, dP and the scores are rounded to 16 bits), so dQ and dK are bounded against sums of that, not of |dS|
    qh, kh, vh, doh = (t.double().transpose(1, 2) for t in (q, k, v, do))                 # [B, H, S, hd]
    sc = alpha * qh @ kh.transpose(-1, -2)
    smax = float(sc.abs().max())
    causal = torch.ones(s, s, dtype=torch.bool, device="cuda").tril()
    pr = torch.softmax(sc.masked_fill(~causal, float("-inf")), -1)
    dpr = doh @ vh.transpose(-1, -2)
    terms = pr * (dpr.abs() + (pr * dpr).sum(-1, keepdim=True).abs())
    mag = {"dv": (pr.transpose(-1, -2) @ doh.abs()).transpose(1, 2), "dq": alpha * (terms @ kh.abs()).transpose(1, 2),
           "dk": alpha * (terms.transpose(-1, -2) @ qh.abs()).transpose(1, 2)}
    _, edq, edk, edv = TD.causal_attention(q, k, v, do, alpha)
    exact = {"dq": edq, "dk": edk, "dv": edv}
    for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert_close(host(got), host(chain[name]).astype(np.float64), "float16", f"fused {name} vs chain", rtol=4e-3,
                     floor_abs=host(mag[name]))
        assert_close(host(got), host(exact[name]), "float16", f"fused {name} vs float64 adjoint", rtol=2e-3 * max(1.0, smax),
                     floor_abs=2 * host(mag[name]))


def test_attention_bwd_fused_bf16_and_errors(cuda):
    from tests import torch_defs as TD
    bsz, s, h, hd = 1, 256, 2, 100
    q, k, v, do = (dev(R.bf16_round(R.normal(120 + i, (bsz, s, h, hd))), bf16=True) for i in range(4))
    alpha = 0.1
    qp, kp, vp, dop = (ops.block_pad(t, 128) for t in (q, k, v, do))
    ctx, stats = ops.attention_fwd(qp, kp, vp, hd, alpha)
    dq, dk, dv = ops.attention_bwd(qp, kp, vp, dop, ctx, stats, alpha)
    _, edq, edk, edv = TD.causal_attention(q, k, v, do, alpha)
    # scores, dP, P and dS each rounded to bfloat16 (2^-8): bounded against the tensor's rms at a few of those
    for name, got, ex in (("dq", dq, edq), ("dk", dk, edk), ("dv", dv, edv)):
        assert_close(host(got), host(ex), "bfloat16", f"bf16 fused {name}", rtol=2.0 ** -4, floor_frac=1.0)
    L = capi.lib()
    P = qp.data_ptr()
    args = (P, P, P, P, P, P, P, P, P)
    assert L.cacti_b200_attention_bwd(*args, 1, 200, 2, 100, 0.1, capi.R_16F, None) == capi.ERR_SHAPE
    assert L.cacti_b200_attention_bwd(*args, 1, 256, 2, 130, 0.1, capi.R_16F, None) == capi.ERR_SHAPE
    assert L.cacti_b200_attention_bwd(*args, 1, 256, 2, 100, 0.1, capi.R_32F, None) == capi.ERR_DTYPE
    assert L.cacti_b200_attention_bwd(*args, 0, 256, 2, 100, 0.1, capi.R_16F, None) == capi.OK
    assert L.cacti_b200_attention_bwd(0, P, P, P, P, P, P, P, P, 1, 256, 2, 100, 0.1, capi.R_16F, None) == capi.ERR_INVALID_VALUE
