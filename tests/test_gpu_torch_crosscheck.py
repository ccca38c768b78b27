"""The CUDA kernels against PyTorch float64 formulas written from the mathematical definitions (tests/torch_defs.py),
gradients by autograd, at the benchmark configurations' full shapes (configs 1 to 4, and the attention block of
config 5 for one sequence).  The comparison runs on the device.

This is the second, independent witness beside the oracle: the oracle restates the reference's chains and could share
a misreading with the kernels; these formulas come from the definitions alone.  Tolerances as in
tests/test_oracle_vs_torch.py: 1e-5 relative in fp32; 2e-3 relative / one fp16 ulp per rounding in fp16, against the
magnitude of the terms where an output is a difference of terms.
"""
import math

import numpy as np
import pytest
import torch

from cacti_b200 import capi, ops
from tests import torch_defs as TD
from tests.tolerances import ABS_MIN, FLOOR_FRAC, RTOL

pytestmark = pytest.mark.gpu


def close(got, ref, kind, what, rtol=None, floor_abs=None):
    """tests.tolerances.assert_close on device tensors (same bound, no host copies of gigabyte tensors)."""
    got, ref = got.double(), ref.double()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    nan_r = torch.isnan(ref)
    assert torch.equal(torch.isnan(got), nan_r), f"{what}: NaN pattern differs"
    got, ref = torch.where(nan_r, 0.0, got), torch.where(nan_r, 0.0, ref)
    rtol = RTOL[kind] if rtol is None else rtol
    rms = float(ref.pow(2).mean().sqrt())
    floor = torch.clamp(ref.abs(), min=FLOOR_FRAC[kind] * rms)
    if floor_abs is not None:
        floor = torch.maximum(floor, floor_abs.double())
    bound = rtol * floor + ABS_MIN[kind]
    err = (got - ref).abs()
    bad = err > bound
    if bool(bad.any()):
        i = int(torch.argmax(err / bound))
        raise AssertionError(f"{what}: {int(bad.sum())}/{bad.numel()} out of tolerance; worst at flat index {i}: got "
                             f"{float(got.flatten()[i])!r} ref {float(ref.flatten()[i])!r} err {float(err.flatten()[i]):.3e} "
                             f"bound {float(bound.flatten()[i]):.3e}")


def rnd(gen, *shape, scale=1.0, shift=0.0, dtype=torch.float16):
    return (torch.randn(*shape, device="cuda", generator=gen) * scale + shift).to(dtype)


@pytest.fixture
def gen(cuda):
    return torch.Generator(device="cuda").manual_seed(0)


@pytest.mark.parametrize("rows,dtype,kind", [(256, torch.float32, "float32"), (16384, torch.float16, "float16")])
def test_rmsnorm_config1_and_step_shape(gen, rows, dtype, kind):
    x, gamma, dy = rnd(gen, rows, 3200, dtype=dtype), rnd(gen, 3200, scale=0.02, shift=1.0, dtype=dtype), rnd(gen, rows, 3200, dtype=dtype)
    y, dx, dgamma = ops.rmsnorm_fwd_bwd(x, gamma, dy, 1e-6)
    ry, rdx, rdg = TD.rmsnorm(x, gamma, dy, 1e-6)
    close(y, ry, kind, f"rmsnorm y {kind}")
    x64, g64, dy64 = x.double(), gamma.double(), dy.double()
    s = (x64.pow(2).mean(-1, keepdim=True) + 1e-6).sqrt()
    c = (g64 * dy64 * x64).sum(-1, keepdim=True)
    close(dx, rdx, kind, f"rmsnorm dx {kind}", floor_abs=(g64 * dy64).abs() / s + (x64 * c).abs() / (3200 * s ** 3))
    close(dgamma, rdg, kind, f"rmsnorm dgamma {kind}", floor_abs=(dy64 * x64 / s).abs().sum(0))


def test_causal_softmax_config2(gen):
    heads, seq = 32, 2048
    s, dp = rnd(gen, heads * seq, seq, scale=0.1), rnd(gen, heads * seq, seq)
    p, ds = ops.softmax_fwd_bwd(s, dp, (1, seq, 0))
    q_pos = torch.arange(heads * seq, device="cuda") % seq
    rp, rds = TD.causal_softmax(s, dp, q_pos)
    close(p, rp, "float16", "softmax P")
    c = (rp * dp.double()).sum(-1, keepdim=True)
    close(ds, rds, "float16", "softmax dS", floor_abs=rp * (dp.double().abs() + c.abs()))
    masked = torch.arange(seq, device="cuda")[None, :] > q_pos[:, None]
    assert not p[masked].any() and not ds[masked].any()


def test_cross_entropy_config3(gen):
    rows, vocab = 8192, 32000
    logits = rnd(gen, rows, vocab, scale=2.0)
    targets = torch.randint(0, vocab, (rows,), device="cuda", dtype=torch.int32, generator=gen)
    w = 1.0 / rows
    loss_sum, loss_rows, d, status = ops.softmax_nll_fwd_bwd(logits, targets, w_scalar=w)
    assert int(status.item()) == 0
    rloss, rd = TD.cross_entropy(logits, targets, w)
    close(loss_rows, rloss, "float32", "nll loss rows")
    mean = float((rloss * w).sum())
    assert abs(float(loss_sum.item()) - mean) <= 1e-5 * abs(mean)
    y = torch.softmax(logits.double(), -1)
    y[torch.arange(rows, device="cuda"), targets.long()] += 1.0
    close(d, rd, "float16", "nll dlogits", floor_abs=w * y)


def test_rope_config4(gen):
    tokens, heads, hd, seq = 16384, 32, 100, 2048
    cos, sin = ops.rope_tables(seq, hd)
    c64, s64 = TD.rope_angles(seq, hd, device="cuda")
    # the tables are f32 evaluations rounded to fp16; the f32 argument p * w carries up to 2^-24 * 2047 of error
    close(cos, c64, "float16", "cos table", floor_abs=torch.full_like(c64, 0.1))
    close(sin, s64, "float16", "sin table", floor_abs=torch.full_like(c64, 0.1))
    x, dy = rnd(gen, tokens, heads, hd), rnd(gen, tokens, heads, hd)
    y, dx = ops.rope_fwd_bwd(x, dy, cos, sin)
    pos = torch.arange(tokens, device="cuda") % seq
    ry, rdx = TD.rope(x, dy, cos, sin, pos)              # on the kernel's own tables: the rotation alone
    half = hd // 2

    def swap(a):
        return torch.cat([a[..., half:], a[..., :half]], -1)

    c, s = cos.double()[pos][:, None, :], sin.double()[pos][:, None, :]
    close(y, ry, "float16", "rope y", floor_abs=(x.double() * c).abs() + (swap(x.double()) * s).abs())
    close(dx, rdx, "float16", "rope dx", floor_abs=(dy.double() * c).abs() + swap((dy.double() * s).abs()))


def test_swiglu_config4(gen):
    gate, up, dh = (rnd(gen, 16384, 8640) for _ in range(3))
    h, dg, du = ops.swiglu_fwd_bwd(gate, up, dh)
    rh, rdg, rdu = TD.swiglu(gate, up, dh)
    # the reference's fp16 chain rounds after every primitive (tests/test_oracle_vs_torch.py::test_swiglu_chain)
    close(h, rh, "float16", "swiglu h", rtol=3e-3)
    close(du, rdu, "float16", "swiglu dup", rtol=3e-3)
    g64 = gate.double()
    sig = torch.sigmoid(g64)
    close(dg, rdg, "float16", "swiglu dgate", rtol=4e-3, floor_abs=(dh.double() * up.double()).abs() * ((g64 * sig * (1 - sig)).abs() + sig))


def test_attention_block_of_config5_one_sequence(gen):
    """Fused forward and the backward chain the training step runs (bwd_prep, then the three hinted block matmuls)
    against scaled_dot_product_attention(is_causal=True) in float64 with autograd."""
    bsz, seq, heads, hd = 1, 2048, 32, 100
    alpha = 1.0 / math.sqrt(hd)
    q, k, v, do = (rnd(gen, bsz, seq, heads, hd) for _ in range(4))
    qp, kp, vp, dop = (ops.block_pad(t, 128) for t in (q, k, v, do))
    ctx, stats = ops.attention_fwd(qp, kp, vp, hd, alpha)
    p, ds = ops.attention_bwd_prep(qp, kp, vp, dop, ctx, stats, alpha)
    dv = ops.block_gemm(p, dop, True, False, tri=capi.TRI_A_UPPER, b_valid=hd)
    dq = ops.block_gemm(ds, kp, False, False, alpha=alpha, tri=capi.TRI_A_LOWER, b_valid=hd)
    dk = ops.block_gemm(ds, qp, True, False, alpha=alpha, tri=capi.TRI_A_UPPER, b_valid=hd)
    rctx, rdq, rdk, rdv = TD.causal_attention(q, k, v, do, alpha)
    # error model: scores and probabilities are rounded to fp16 (2^-11 relative each) before they are used, so every
    # output is good to a few 2^-11 of the sum of magnitudes of its terms; the sums below are those magnitudes
    qh, kh, vh, doh = (t.double().transpose(1, 2) for t in (q, k, v, do))                 # [B, H, S, hd]
    sc = alpha * qh @ kh.transpose(-1, -2)
    smax = float(sc.abs().max())
    causal = torch.ones(seq, seq, dtype=torch.bool, device="cuda").tril()
    pr = torch.softmax(sc.masked_fill(~causal, float("-inf")), -1)
    dpr = doh @ vh.transpose(-1, -2)
    cdot = (pr * dpr).sum(-1, keepdim=True)
    dsa = pr * (dpr.abs() + cdot.abs())                                                   # |terms| of dS
    tol = 2e-3 * max(1.0, smax)
    close(ctx, rctx, "float16", "attention ctx", rtol=tol, floor_abs=(pr @ vh.abs()).transpose(1, 2) * 2)
    close(dv, rdv, "float16", "attention dV", rtol=tol, floor_abs=(pr.transpose(-1, -2) @ doh.abs()).transpose(1, 2) * 2)
    close(dq, rdq, "float16", "attention dQ", rtol=tol, floor_abs=alpha * (dsa @ kh.abs()).transpose(1, 2) * 2)
    close(dk, rdk, "float16", "attention dK", rtol=tol, floor_abs=alpha * (dsa.transpose(-1, -2) @ qh.abs()).transpose(1, 2) * 2)
