"""The oracle (oracle/ref_chain.py) against an independent statement of the same ops: PyTorch float64 formulas written
from the mathematical definitions, gradients by autograd (tests/torch_defs.py).  Runs on the CPU.

The oracle restates the reference's thunk chains with their rounding points; nothing reference-held pins it (the
reference has no tests and cannot be built here), so this is the cross-check against a shared misreading of a
formula.  Tolerances are the path's own: 1e-5 relative in fp32, 2e-3 relative / one fp16 ulp in fp16 for a single
rounding, scaled by the number of 16-bit roundings where the reference's chain rounds after every primitive
(stated per case).  Where an output is a difference of terms (softmax and RoPE adjoints, the target column of the
cross-entropy gradient) the bound is taken against the magnitude of the terms, passed as `floor_abs`, instead of
widening the floor to the tensor's RMS.
"""
import numpy as np
import torch

from oracle import ref_chain as R
from tests import torch_defs as TD
from tests.tolerances import assert_close


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a).astype(np.float64))


def n(x):
    return x.detach().cpu().numpy()


def test_rmsnorm_fp32_and_fp16():
    for dtype, kind in ((np.float32, "float32"), (np.float16, "float16")):
        x = R.normal(0, (64, 3200), dtype)
        gamma = R.normal(1, (3200,), dtype, 0.02, 1.0)
        dy = R.normal(2, (64, 3200), dtype)
        y, dx, dgamma = TD.rmsnorm(t(x), t(gamma), t(dy), 1e-6)
        ry, rt, _ = R.ref_rmsnorm_fwd(x, gamma, 1e-6)
        rdx, rdg = R.ref_rmsnorm_bwd(x, gamma, dy, 1e-6)
        assert_close(ry, n(y), kind, f"rmsnorm y {kind}")
        # dx = (gamma dy) / s - x c / (D s^3): bounded against the sum of the two terms' magnitudes; in fp16 the chain
        # rounds each of them to 16 bits before the add (two roundings and the sum's)
        s = np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-6)
        c = (gamma.astype(np.float64) * dy.astype(np.float64) * x.astype(np.float64)).sum(-1, keepdims=True)
        terms = np.abs(gamma.astype(np.float64) * dy) / s + np.abs(x * c) / (3200 * s ** 3)
        assert_close(rdx, n(dx), kind, f"rmsnorm dx {kind}", floor_abs=terms, rtol=None if kind == "float32" else 3e-3)
        # dgamma_j = sum_i dy_ij t_ij: an f32 sum of 64 terms, bounded against sum_i |dy_ij t_ij|
        assert_close(rdg, n(dgamma), kind, f"rmsnorm dgamma {kind}", floor_abs=np.abs(dy.astype(np.float64) * rt).sum(0))


def test_causal_softmax_and_adjoint():
    heads, seq = 3, 160
    s = R.normal(3, (heads * seq, seq), np.float16, 0.1)
    dp = R.normal(4, (heads * seq, seq), np.float16)
    for q_div, layout in ((1, "[B,H,Sq,Sk]"), (heads, "[B,Sq,H,Sk]")):
        q_pos = (torch.arange(heads * seq) // q_div) % seq
        p, ds = TD.causal_softmax(t(s), t(dp), q_pos)
        keep = R.causal_keep_mask(heads * seq, seq, q_div, seq, 0)
        assert np.array_equal(keep, n(torch.arange(seq)[None, :] <= q_pos[:, None]))
        rp, _ = R.ref_softmax_fwd(s, keep)
        rds = R.ref_softmax_bwd(s, dp, keep)
        assert_close(rp, n(p), "float16", f"softmax P {layout}")
        assert (rp[~keep] == 0).all() and (rds[~keep] == 0).all()
        # dS_j = y_j (dP_j - sum_k y_k dP_k): against y_j (|dP_j| + |c|)
        c = (n(p) * dp.astype(np.float64)).sum(-1, keepdims=True)
        assert_close(rds, n(ds), "float16", f"softmax dS {layout}", floor_abs=n(p) * (np.abs(dp.astype(np.float64)) + np.abs(c)))
    # no mask
    p, ds = TD.causal_softmax(t(s), t(dp), None)
    assert_close(R.ref_softmax_fwd(s, None)[0], n(p), "float16", "softmax P unmasked")


def test_cross_entropy_loss_and_gradient():
    rows, vocab = 24, 32000
    logits = R.normal(5, (rows, vocab), np.float16, 2.0)
    targets = R.uniform_int(6, rows, vocab)
    w = 1.0 / rows
    loss, d = TD.cross_entropy(t(logits), torch.from_numpy(targets), w)
    rloss, rd, picked = R.ref_softmax_nll(logits, targets, np.float32(w))
    assert_close(rloss, n(loss), "float32", "nll loss rows")
    assert np.array_equal(picked, logits[np.arange(rows), targets])            # the gather is exact
    # w (y - onehot): against w (y + onehot)
    y = np.exp(logits.astype(np.float64) - logits.astype(np.float64).max(-1, keepdims=True))
    y /= y.sum(-1, keepdims=True)
    mag = y.copy()
    mag[np.arange(rows), targets] += 1.0
    assert_close(rd, n(d), "float16", "nll dlogits", floor_abs=w * mag)
    assert abs(float((w * rloss.astype(np.float64)).sum()) - float((w * n(loss)).sum())) < 1e-5 * float((w * n(loss)).sum())


def test_swiglu_chain():
    gate, up, dh = (R.normal(7 + i, (96, 864), np.float16) for i in range(3))
    h, dg, du = TD.swiglu(t(gate), t(up), t(dh))
    rh, _ = R.ref_swiglu_fwd(gate, up)
    rdg, rdu = R.ref_swiglu_bwd(gate, up, dh)
    # the reference's chain rounds to fp16 after every primitive: neg, exp, add, div, mul for h (four roundings that
    # matter) and about eight for dgate; allow one fp16 half-ulp (2^-12 relative... 2.4e-4) per rounding on top of 2e-3
    assert_close(rh, n(h), "float16", "swiglu h", rtol=3e-3)
    assert_close(rdu, n(du), "float16", "swiglu dup", rtol=3e-3)
    # dgate = dh u (y (1 - t) + t): y (1 - t) and t are added after rounding; against |dh u| (|y (1 - t)| + |t|)
    g64 = gate.astype(np.float64)
    sig = 1 / (1 + np.exp(-g64))
    terms = np.abs(dh.astype(np.float64) * up) * (np.abs(g64 * sig * (1 - sig)) + sig)
    assert_close(rdg, n(dg), "float16", "swiglu dgate", rtol=4e-3, floor_abs=terms)


def test_rope_tables_and_rotation():
    seq, heads, hd = 64, 4, 100
    cos64, sin64 = TD.rope_angles(seq, hd)
    rcos, rsin = R.ref_rope_tables(seq, hd)
    # tables: f32 evaluation rounded to fp16 (|angle| < 64 here, so the f32 argument error is below 1e-5)
    assert_close(rcos, n(cos64), "float16", "cos table", floor_abs=1e-2)
    assert_close(rsin, n(sin64), "float16", "sin table", floor_abs=1e-2)
    tokens = 2 * seq
    pos = np.arange(tokens) % seq
    x, dy = R.normal(10, (tokens, heads, hd), np.float16), R.normal(11, (tokens, heads, hd), np.float16)
    # the rotation itself, on the reference's own (rounded) tables: three fp16 roundings (two products, one sum),
    # bounded against |x cos| + |rot(x) sin|
    y, dx = TD.rope(t(x), t(dy), t(rcos), t(rsin), torch.from_numpy(pos))
    c, s = rcos.astype(np.float64)[pos][:, None, :], rsin.astype(np.float64)[pos][:, None, :]
    half = hd // 2

    def swap(a):
        return np.concatenate([a[..., half:], a[..., :half]], -1)

    x64, dy64 = x.astype(np.float64), dy.astype(np.float64)
    assert_close(R.ref_rope_fwd(x, rcos, rsin, pos), n(y), "float16", "rope y", floor_abs=np.abs(x64 * c) + np.abs(swap(x64) * s))
    assert_close(R.ref_rope_bwd(dy, rcos, rsin, pos), n(dx), "float16", "rope dx",
                 floor_abs=np.abs(dy64 * c) + swap(np.abs(dy64 * s)))


def test_causal_attention():
    bsz, seq, heads, hd = 1, 96, 2, 100
    q, k, v, do = (R.normal(12 + i, (bsz, seq, heads, hd), np.float16) for i in range(4))
    alpha = hd ** -0.5
    ctx, _, _, _ = TD.causal_attention(t(q), t(k), t(v), t(do), alpha)
    rctx, _, _, mag = R.ref_causal_attention(q, k, v, alpha)
    # the oracle rounds the scores to fp16 as block_matmul_scale stores them: d ctx = sum_j p_j ds_j (v_j - ctx), |ds| <=
    # 2^-11 |s|, so the context moves by at most that much relative to sum_j p_j |v_j| times the largest |s|
    smax = float(np.abs(alpha * np.einsum("bqhd,bkhd->bhqk", q.astype(np.float64), k.astype(np.float64))).max())
    assert_close(rctx, n(ctx), "float16", "attention ctx", rtol=2e-3 * max(1.0, smax), floor_abs=2 * mag)
