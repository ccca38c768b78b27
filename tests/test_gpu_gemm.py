"""GPU parity tests of the tcgen05 GEMM (dense and block form) against the fp64 oracle.

Tolerance: 2e-3 relative (fp16) measured against max(|ref|, rms): the fp32 accumulation error of a
dot product scales with sum |a||b|, not with the (possibly cancelled) result.
"""
import numpy as np
import pytest
import torch

from cacti_b200 import capi, ops
from oracle import ref_chain as R
from tests.gpu_util import dev, host
from tests.tolerances import assert_close

pytestmark = pytest.mark.gpu


def _stored(seed, rows, cols, trans, scale=1.0):
    """Matrix op(X) = rows x cols, stored transposed when trans."""
    return R.normal(seed, (cols, rows) if trans else (rows, cols), np.float16, scale)


@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 128, 128), (256, 512, 320), (100, 72, 40), (1, 8, 8),
                                   (300, 260, 200), (129, 257, 65), (640, 3200, 3200)])
def test_gemm_dense(cuda, ta, tb, m, n, k):
    a = _stored(1, m, k, ta)
    b = _stored(2, k, n, tb, 0.1)
    c = ops.gemm(dev(a), dev(b), ta, tb, alpha=0.5)
    ref = R.ref_gemm(a, b, ta, tb, alpha=0.5)
    assert_close(host(c), ref, "float16", f"gemm {m}x{n}x{k} ta={ta} tb={tb}", floor_frac=1.0)
    # Accumulate mode (beta = 1), as the reference's Accumulate thunk does (src/thunk/op.rs:5053-5067)
    old = R.normal(3, (m, n), np.float16)
    cacc = dev(old)
    ops.gemm(dev(a), dev(b), ta, tb, alpha=0.5, beta=1.0, c=cacc)
    assert_close(host(cacc), R.ref_gemm(a, b, ta, tb, alpha=0.5, beta=1.0, c=old), "float16", "gemm beta=1", floor_frac=1.0)


def test_gemm_views_and_bf16(cuda):
    # leading dimensions larger than the row, unaligned base: goes through the repack path
    big_a = R.normal(4, (200, 331), np.float16)
    big_b = R.normal(5, (150, 331), np.float16, 0.1)
    ta_, tb_ = dev(big_a), dev(big_b)
    a_v, b_v = ta_[:, 3:203], tb_[:, 1:201]            # 200 x 200 and 150 x 200 views, odd offsets
    c = torch.zeros(200, 160, dtype=torch.float16, device="cuda")[:, 5:155]
    ops.gemm(a_v, b_v, False, True, c=c)
    ref = R.ref_gemm(big_a[:, 3:203], big_b[:, 1:201], False, True)
    assert_close(host(c.contiguous()), ref, "float16", "gemm on views", floor_frac=1.0)
    a = R.bf16_round(R.normal(6, (256, 192)))
    b = R.bf16_round(R.normal(7, (320, 192), scale=0.1))
    c = ops.gemm(dev(a, bf16=True), dev(b, bf16=True), False, True)
    ref = a.astype(np.float64) @ b.astype(np.float64).T
    assert_close(host(c), ref, "bfloat16", "bf16 gemm", floor_frac=1.0)


@pytest.mark.parametrize("m,n,k", [(300, 264, 200), (1000, 3200, 512)])
def test_gemm_accumulate_epilogues_agree(cuda, m, n, k):
    """beta = 1 through the two epilogues: old C brought in by TMA (aligned C) and read per thread (C a view whose row
    pitch is not a multiple of 16 bytes) must give the same bits; both against the oracle."""
    a, b = _stored(31, m, k, False), _stored(32, k, n, True, 0.1)
    old = R.normal(33, (m, n), np.float16)
    c_tma = dev(old)
    ops.gemm(dev(a), dev(b), False, True, alpha=0.5, beta=1.0, c=c_tma)
    wide = torch.zeros(m, n + 3, dtype=torch.float16, device="cuda")
    c_view = wide[:, 1:n + 1]
    c_view.copy_(dev(old))
    ops.gemm(dev(a), dev(b), False, True, alpha=0.5, beta=1.0, c=c_view)
    assert torch.equal(c_tma, c_view.contiguous())
    assert_close(host(c_tma), R.ref_gemm(a, b, False, True, alpha=0.5, beta=1.0, c=old), "float16", "gemm beta=1 (TMA epilogue)",
                 floor_frac=1.0)
    assert float(wide[:, 0].abs().max()) == 0.0 and float(wide[:, n + 1:].abs().max()) == 0.0      # nothing outside the view


@pytest.fixture
def pair_tiles():
    """Force 256-wide tiles, which run as two-SM (cta_group::2) 256 x 256 tiles, for the duration of a test."""
    L = capi.lib()
    assert L.cacti_b200_tune(b"gemm_pair", 1) == capi.OK
    assert L.cacti_b200_tune(b"gemm_bn", 256) == capi.OK
    yield
    L.cacti_b200_tune(b"gemm_bn", 0)


@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (256, 512, 320), (300, 260, 200), (129, 257, 65), (1000, 700, 1031 // 8 * 8),
                                   (640, 3200, 3200), (4096 + 128, 1024, 512)])
def test_gemm_pair_tiles(cuda, pair_tiles, ta, tb, m, n, k):
    """Same cases as the dense test on the two-SM kernel: ragged M (a tile whose second CTA is partly or wholly
    past M), ragged N and K, several tiles per CTA pair (both accumulators and every ring stage reused), TMA-store and
    direct-store (beta = 1) epilogues."""
    a = _stored(21, m, k, ta)
    b = _stored(22, k, n, tb, 0.1)
    c = ops.gemm(dev(a), dev(b), ta, tb, alpha=0.5)
    ref = R.ref_gemm(a, b, ta, tb, alpha=0.5)
    assert_close(host(c), ref, "float16", f"pair gemm {m}x{n}x{k} ta={ta} tb={tb}", floor_frac=1.0)
    old = R.normal(23, (m, n), np.float16)
    cacc = dev(old)
    ops.gemm(dev(a), dev(b), ta, tb, alpha=0.5, beta=1.0, c=cacc)
    assert_close(host(cacc), R.ref_gemm(a, b, ta, tb, alpha=0.5, beta=1.0, c=old), "float16", "pair gemm beta=1",
                 floor_frac=1.0)
    import ctypes as C
    torch.cuda.synchronize()
    err = C.c_uint(7)
    assert capi.lib().cacti_b200_device_error(C.byref(err)) == capi.OK and err.value == 0      # no bounded wait ran out


@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(256, 512, 320), (300, 260, 200), (640, 3200, 3200)])
def test_gemm_single_sm_tiles(cuda, ta, tb, m, n, k):
    """The one-SM kernel on shapes the automatic choice now gives to the two-SM one."""
    L = capi.lib()
    a = _stored(41, m, k, ta)
    b = _stored(42, k, n, tb, 0.1)
    L.cacti_b200_tune(b"gemm_pair", 0)
    try:
        c = ops.gemm(dev(a), dev(b), ta, tb, alpha=0.5)
    finally:
        L.cacti_b200_tune(b"gemm_pair", 1)
    assert_close(host(c), R.ref_gemm(a, b, ta, tb, alpha=0.5), "float16", f"1-SM gemm {m}x{n}x{k}", floor_frac=1.0)


def test_gemm_pair_tiles_match_single_sm(cuda):
    """The two kernels accumulate every output element over k in the same order (one UMMA per 16 k), so their results
    are bit-identical; block form with batch strides included."""
    L = capi.lib()
    a = dev(R.normal(31, (2, 384, 3, 128), np.float16))
    b = dev(R.normal(32, (2, 384, 3, 128), np.float16))
    x = dev(R.normal(33, (1536, 1024), np.float16))
    w = dev(R.normal(34, (2048, 1024), np.float16, 0.05))
    L.cacti_b200_tune(b"gemm_bn", 256)
    try:
        L.cacti_b200_tune(b"gemm_pair", 0)
        one = (ops.block_gemm(a, b, False, True), ops.gemm(x, w, False, True))
        L.cacti_b200_tune(b"gemm_pair", 1)
        two = (ops.block_gemm(a, b, False, True), ops.gemm(x, w, False, True))
    finally:
        L.cacti_b200_tune(b"gemm_pair", 1)
        L.cacti_b200_tune(b"gemm_bn", 0)
    for o, t in zip(one, two):
        assert torch.equal(o, t)


def test_dynamic_schedule_gives_the_same_bits(cuda):
    """Tiles drawn from the global counter (the default) or walked with a fixed stride: every tile is computed whole by
    one CTA (pair) in the same k order either way, so the results are bit-identical.  Dense on the two-SM and the
    one-SM kernel, several tiles per CTA, a grid smaller than the machine, block form with and without the causal
    hints; and the counters are left clean (the same calls repeat with the same result)."""
    L = capi.lib()
    x, w = dev(R.normal(71, (2304, 1024), np.float16)), dev(R.normal(72, (3200, 1024), np.float16, 0.05))
    q, k = dev(R.normal(73, (2, 512, 3, 128), np.float16)), dev(R.normal(74, (2, 512, 3, 128), np.float16))
    pl = torch.tril(torch.ones(512, 512, device="cuda", dtype=torch.float16))[None, :, None, :].expand(2, 512, 3, 512).contiguous()

    def run_all():
        out = [ops.gemm(x, w, False, True), ops.gemm(x, w[:, :1024].contiguous(), False, True, beta=0.0),
               ops.block_gemm(q, k, False, True, alpha=0.1), ops.block_gemm(q, k, False, True, alpha=0.1, tri=capi.TRI_C_LOWER),
               ops.block_gemm(pl, k, False, False, tri=capi.TRI_A_LOWER), ops.block_gemm(pl, k, True, False, tri=capi.TRI_A_UPPER)]
        for knob, val in ((b"gemm_pair", 0), (b"gemm_sms", 100), (b"gemm_bn", 128)):
            L.cacti_b200_tune(knob, val)
            try:
                out.append(ops.gemm(x, w, False, True))
                out.append(ops.block_gemm(q, k, False, True, alpha=0.1))
            finally:
                L.cacti_b200_tune(knob, 1 if knob == b"gemm_pair" else 0)
        return out

    dyn1 = run_all()
    dyn2 = run_all()
    assert L.cacti_b200_tune(b"gemm_dynamic", 0) == capi.OK
    try:
        fixed = run_all()
    finally:
        L.cacti_b200_tune(b"gemm_dynamic", 1)
    tri_c = 3                                       # C_LOWER leaves tiles above the diagonal unwritten: compare what is specified
    low = torch.tril(torch.ones(512, 512, device="cuda", dtype=torch.bool))[None, :, None, :]
    for i, (a, b, c) in enumerate(zip(dyn1, dyn2, fixed)):
        if i == tri_c:
            a, b, c = (torch.where(low, t, 0) for t in (a, b, c))
        assert torch.equal(a, c), i
        assert torch.equal(a, b), i
    assert_close(host(dyn1[0]), R.ref_gemm(host(x), host(w), False, True), "float16", "dynamic schedule vs oracle", floor_frac=1.0)
    import ctypes as C
    torch.cuda.synchronize()
    err = C.c_uint(7)
    assert L.cacti_b200_device_error(C.byref(err)) == capi.OK and err.value == 0


@pytest.fixture
def k_split():
    """Turn the k-split schedule of the two-SM kernel on for one test (it is off by default)."""
    L = capi.lib()
    assert L.cacti_b200_tune(b"gemm_split", 1) == capi.OK
    yield
    L.cacti_b200_tune(b"gemm_split", 0)


# tiles = ceil(m / 256) * ceil(n / 256) against 74 SM pairs: 60 (every tile split between workers), 104 (one to two
# tiles per worker: the projection shape at one sequence per GPU), 160 (two waves and a remainder: k-split region plus
# whole tiles), 52 with a ragged last row and column tile, and a short contraction (8 k-blocks)
@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(1536, 2560, 512), (2048, 3200, 3200), (4096, 2560, 640), (3200, 860, 2048), (2048, 3200, 8640)])
def test_gemm_k_split_schedule(cuda, ta, tb, m, n, k):
    """With a workspace, and the schedule switched on, the two-SM kernel shares the tiles of a partly filled last wave
    out in k-blocks: pieces of a tile computed by different CTA pairs are summed in f32 in k order by the pair that
    owns the tile.  Held to the fp64 oracle like every other matmul; equal from run to run; and within f32 summation
    noise of the whole-tile schedule (both round the same f32 sum up to its association)."""
    L = capi.lib()
    a, b = dev(_stored(51, m, k, ta)), dev(_stored(52, k, n, tb, 0.1))
    ws = ops.gemm_workspace(m, n, k, a.device)
    plain = ops.gemm(a, b, ta, tb, alpha=0.5, workspace=ws)         # off by default: every tile computed whole,
    if m % 8 == 0 and n % 8 == 0 and k % 8 == 0:                    # workspace or not
        assert torch.equal(plain, ops.gemm(a, b, ta, tb, alpha=0.5))
    old = dev(R.normal(53, (m, n), np.float16))
    cacc = old.clone()
    wide = torch.zeros(m, n + 3, dtype=torch.float16, device=a.device)
    assert L.cacti_b200_tune(b"gemm_split", 1) == capi.OK
    try:
        c1 = ops.gemm(a, b, ta, tb, alpha=0.5, workspace=ws)
        c2 = ops.gemm(a, b, ta, tb, alpha=0.5, workspace=ws)
        # Accumulate mode (direct-store epilogue) and an output view TMA cannot store to
        ops.gemm(a, b, ta, tb, alpha=0.5, beta=1.0, c=cacc, workspace=ws)
        ops.gemm(a, b, ta, tb, alpha=0.5, c=wide[:, 1:n + 1], workspace=ws)
    finally:
        L.cacti_b200_tune(b"gemm_split", 0)
    assert torch.equal(c1, c2)
    ref = R.ref_gemm(host(a), host(b), ta, tb, alpha=0.5)
    assert_close(host(c1), ref, "float16", f"k-split gemm {m}x{n}x{k} ta={ta} tb={tb}", floor_frac=1.0)
    diff = (c1.float() - plain.float()).abs()
    assert float(diff.max()) <= 2.0 ** -10 * float(plain.float().abs().max())
    assert 0 < float((diff > 0).float().mean()) < 0.2       # another summation order, yet mostly the same 16-bit values
    assert_close(host(cacc), R.ref_gemm(host(a), host(b), ta, tb, alpha=0.5, beta=1.0, c=host(old)), "float16", "k-split beta=1",
                 floor_frac=1.0)
    assert torch.equal(wide[:, 1:n + 1], c1) and not wide[:, 0].any() and not wide[:, n + 1:].any()
    import ctypes as C
    torch.cuda.synchronize()
    err = C.c_uint(7)
    assert L.cacti_b200_device_error(C.byref(err)) == capi.OK and err.value == 0


def test_gemm_k_split_fewer_sm_pairs(cuda, k_split):
    """The schedule follows the worker count: with SMs left free for a concurrent kernel (gemm_sms) the ranges are cut
    for that many pairs."""
    L = capi.lib()
    a, b = dev(_stored(61, 2048, 3200, False)), dev(_stored(62, 3200, 3200, True, 0.1))
    ws = ops.gemm_workspace(2048, 3200, 3200, a.device)
    ref = R.ref_gemm(host(a), host(b), False, True)
    for sms in (132, 100, 0):
        L.cacti_b200_tune(b"gemm_sms", sms)
        try:
            c = ops.gemm(a, b, False, True, workspace=ws)
        finally:
            L.cacti_b200_tune(b"gemm_sms", 0)
        assert_close(host(c), ref, "float16", f"k-split on {sms} SMs", floor_frac=1.0)


@pytest.mark.parametrize("hd", [100, 128, 64])
def test_block_gemm_attention_shapes(cuda, hd):
    """The four block matmuls of one attention layer and their adjoints, layout [B, S, H, hd] / [B, Sq, H, Sk]."""
    bsz, s, h = 2, 256, 3
    q = R.normal(10, (bsz, s, h, hd), np.float16)
    k = R.normal(11, (bsz, s, h, hd), np.float16)
    v = R.normal(12, (bsz, s, h, hd), np.float16)
    alpha = float(1.0 / np.sqrt(hd))
    sc = ops.block_gemm(dev(q), dev(k), False, True, alpha=alpha)                 # scores = alpha Q K^T
    ref_sc = R.ref_block_gemm(q, k, False, True, alpha=alpha)
    assert sc.shape == (bsz, s, h, s)
    assert_close(host(sc), ref_sc, "float16", "QK^T", floor_frac=1.0)
    p = R.normal(13, (bsz, s, h, s), np.float16, 0.05)
    ctx = ops.block_gemm(dev(p), dev(v), False, False)                            # ctx = P V
    assert_close(host(ctx), R.ref_block_gemm(p, v, False, False), "float16", "PV", floor_frac=1.0)
    do = R.normal(14, (bsz, s, h, hd), np.float16)
    dv = ops.block_gemm(dev(p), dev(do), True, False)                             # dV = P^T dO
    assert_close(host(dv), R.ref_block_gemm(p, do, True, False), "float16", "P^T dO", floor_frac=1.0)
    dp = ops.block_gemm(dev(do), dev(v), False, True)                             # dP = dO V^T
    assert_close(host(dp), R.ref_block_gemm(do, v, False, True), "float16", "dO V^T", floor_frac=1.0)
    ds = R.normal(15, (bsz, s, h, s), np.float16, 0.05)
    dq = ops.block_gemm(dev(ds), dev(k), False, False, alpha=alpha)               # dQ = alpha dS K
    assert_close(host(dq), R.ref_block_gemm(ds, k, False, False, alpha=alpha), "float16", "dS K", floor_frac=1.0)
    dk = ops.block_gemm(dev(ds), dev(q), True, False, alpha=alpha)                # dK = alpha dS^T Q
    assert_close(host(dk), R.ref_block_gemm(ds, q, True, False, alpha=alpha), "float16", "dS^T Q", floor_frac=1.0)


@pytest.mark.parametrize("hd,s,diag", [(100, 512, 0), (128, 640, 0), (64, 384, 70), (100, 300, -33)])
def test_block_gemm_triangular_hints(cuda, hd, s, diag):
    """The hinted block matmuls around a causal softmax equal the unhinted ones bit for bit wherever the result is
    specified: C_LOWER on the wanted triangle, A_LOWER / A_UPPER everywhere (the skipped products are exact zeros)."""
    bsz, h = 2, 3
    q = dev(R.normal(50, (bsz, s, h, hd), np.float16))
    k = dev(R.normal(51, (bsz, s, h, hd), np.float16))
    v = dev(R.normal(52, (bsz, s, h, hd), np.float16))
    do = dev(R.normal(53, (bsz, s, h, hd), np.float16))
    r = torch.arange(s, device="cuda")
    wanted = (r[None, :] <= r[:, None] + diag)[None, :, None, :]            # [1, Sq, 1, Sk]: c <= r + diag
    # scores = Q K^T and dP = dO V^T: only the wanted triangle is specified
    for a, b in ((q, k), (do, v)):
        full = ops.block_gemm(a, b, False, True, alpha=0.1)
        c = torch.full_like(full, 7.0)
        ops.block_gemm(a, b, False, True, alpha=0.1, c=c, tri=capi.TRI_C_LOWER, diag=diag)
        assert torch.equal(torch.where(wanted, c, 0), torch.where(wanted, full, 0))
    # a tile wholly beyond the diagonal is left untouched (not a promise of the interface, but it is where the
    # saving comes from: fails if the hint were ignored)
    if s >= 512 and diag == 0:
        assert torch.all(c[:, :128, :, 256:] == 7.0)
    p_low = torch.where(wanted, dev(R.normal(54, (bsz, s, h, s), np.float16, 0.05)), 0)    # zero for c > r + diag
    for b_op in (v, k):                                                                      # P V and dS K
        assert torch.equal(ops.block_gemm(p_low, b_op, False, False, tri=capi.TRI_A_LOWER, diag=diag),
                           ops.block_gemm(p_low, b_op, False, False))
    # P^T dO and dS^T Q: op(A)[r = key, kk = query] is zero for kk < r - diag
    for b_op in (do, q):
        assert torch.equal(ops.block_gemm(p_low, b_op, True, False, tri=capi.TRI_A_UPPER, diag=diag),
                           ops.block_gemm(p_low, b_op, True, False))
    import ctypes as C
    torch.cuda.synchronize()
    err = C.c_uint(7)
    assert capi.lib().cacti_b200_device_error(C.byref(err)) == capi.OK and err.value == 0


@pytest.mark.parametrize("hd,s,q_off", [(100, 512, 0), (128, 768, 256), (64, 600, 77)])
def test_trimmed_softmax_feeds_hinted_block_gemms(cuda, hd, s, q_off):
    """P and dS from the trimmed-fill softmax (garbage left beyond the fill bound) through the hinted block matmuls
    equal the fully zero-filled, unhinted chain bit for bit."""
    bsz, h = 2, 3
    sc = dev(R.normal(60, (bsz, s, h, s), np.float16, 0.5))
    dp = dev(R.normal(61, (bsz, s, h, s), np.float16))
    v = dev(R.normal(62, (bsz, s, h, hd), np.float16))
    do = dev(R.normal(63, (bsz, s, h, hd), np.float16))
    mask = (h, s, q_off)
    p_ref, ds_ref = ops.softmax_fwd_bwd(sc.view(-1, s), dp.view(-1, s), mask)
    p = torch.full_like(p_ref, float("nan"))
    ds = torch.full_like(p_ref, float("nan"))
    ops.softmax_fwd_bwd(sc.view(-1, s), dp.view(-1, s), mask + (True,), p=p, ds=ds)
    p4, ds4, pr4, dsr4 = (t.view(bsz, s, h, s) for t in (p, ds, p_ref, ds_ref))
    assert torch.equal(ops.block_gemm(p4, v, False, False, tri=capi.TRI_A_LOWER, diag=q_off), ops.block_gemm(pr4, v, False, False))
    assert torch.equal(ops.block_gemm(ds4, v, False, False, alpha=0.1, tri=capi.TRI_A_LOWER, diag=q_off),
                       ops.block_gemm(dsr4, v, False, False, alpha=0.1))
    assert torch.equal(ops.block_gemm(p4, do, True, False, tri=capi.TRI_A_UPPER, diag=q_off), ops.block_gemm(pr4, do, True, False))
    assert torch.equal(ops.block_gemm(ds4, do, True, False, alpha=0.1, tri=capi.TRI_A_UPPER, diag=q_off),
                       ops.block_gemm(dsr4, do, True, False, alpha=0.1))


def test_block_gemm_broadcast_and_accumulate(cuda):
    a = R.normal(20, (3, 64, 2, 40), np.float16)
    b1 = R.normal(21, (1, 40, 2, 24), np.float16)      # broadcast over block rows
    b2 = R.normal(22, (3, 40, 1, 24), np.float16)      # broadcast over block columns
    for b in (b1, b2):
        c = ops.block_gemm(dev(a), dev(b))
        assert_close(host(c), R.ref_block_gemm(a, b), "float16", "broadcast block gemm", floor_frac=1.0)
    old = R.normal(23, (3, 64, 2, 24), np.float16)
    cacc = dev(old)
    ops.block_gemm(dev(a), dev(b1), beta=1.0, c=cacc)
    assert_close(host(cacc), R.ref_block_gemm(a, b1, beta=1.0, c=old), "float16", "block gemm beta=1", floor_frac=1.0)


def test_gemm_argument_errors(cuda):
    L = capi.lib()
    import ctypes as C
    one, zero = C.byref(C.c_float(1.0)), C.byref(C.c_float(0.0))
    P = 0x1000
    assert L.cacti_b200_gemm(P, P, P, 8, 8, 8, 8, 8, 8, 0, 1, one, zero, capi.R_32F, 0, 0, None) == capi.ERR_DTYPE
    assert L.cacti_b200_gemm(P, P, P, 8, 8, 8, 4, 8, 8, 0, 1, one, zero, capi.R_16F, 0, 0, None) == capi.ERR_INVALID_VALUE
    assert L.cacti_b200_gemm(P, P, P, 0, 8, 8, 8, 8, 8, 0, 1, one, zero, capi.R_16F, 0, 0, None) == capi.OK
    # misaligned operand without a workspace
    assert L.cacti_b200_gemm(P, P + 2, P, 8, 8, 8, 8, 8, 8, 0, 1, one, zero, capi.R_16F, 0, 0, None) == capi.ERR_WORKSPACE
    err = C.c_uint(0)
    assert L.cacti_b200_device_error(C.byref(err)) == capi.OK and err.value == 0


def test_gemm_deterministic(cuda):
    a, b = dev(R.normal(30, (512, 640), np.float16)), dev(R.normal(31, (384, 640), np.float16))
    c1, c2 = ops.gemm(a, b, False, True), ops.gemm(a, b, False, True)
    assert torch.equal(c1, c2)
