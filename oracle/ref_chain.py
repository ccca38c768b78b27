"""CPU oracle: numpy restatement of cacti's thunk chains for the autodiff hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package may import this module;
it is used by tests/, by the smoke check and by the CPU-baseline leg of bench.py.

PARITY UNPINNED: the reference (peterhj/cacti) ships no tests, golden vectors or
fixtures, and cannot be built without its Rust/Futhark toolchain, so this
restatement is checked only against (a) an fp64 single-rounding evaluation of
the same formulas (the ``ideal64_*`` functions below) and (b) the independent C
restatement in ``oracle/ref_chain.c``.

Every ``ref_*`` function follows the reference's op order and *rounding points*:
each primitive thunk of the reference materialises its output in the cell's
dtype, so an f16 chain rounds to f16 after every primitive.  numpy evaluates
float16 arithmetic by computing in float32 and rounding once, which is the
per-op rounding the reference's f16 programs have.

The arithmetic itself is produced in the reference by the Futhark compiler
(fork peterhj/futhark, branch patch-0.26, driven by futhark_ffi 0.1.0-devel;
neither is in the reference tree).  The Futhark *programs* are in-tree strings
and are what is restated here; file:line citations are into the reference tree.
Reduction order inside Futhark's ``reduce`` is unspecified; ``order`` selects
numpy's pairwise sum or a strict left-to-right sum so tests can bracket it.
"""
from __future__ import annotations

import numpy as np

F16 = np.float16
F32 = np.float32
F64 = np.float64


# --------------------------------------------------------------------------- helpers
def _sum_rows(a: np.ndarray, order: str = "pairwise") -> np.ndarray:
    """Row sums over the innermost axis in a's own dtype (f32 in every chain)."""
    if order == "pairwise":
        return a.sum(axis=-1, dtype=a.dtype)
    if order == "sequential":
        return np.add.accumulate(a, axis=-1, dtype=a.dtype)[..., -1]
    raise ValueError(order)


def _sum_cols(a: np.ndarray, order: str = "pairwise") -> np.ndarray:
    if order == "pairwise":
        return a.sum(axis=0, dtype=a.dtype)
    if order == "sequential":
        return np.add.accumulate(a, axis=0, dtype=a.dtype)[-1]
    raise ValueError(order)


def bf16_round(a: np.ndarray) -> np.ndarray:
    """Round float32 to bfloat16 (round-to-nearest-even), returned as float32."""
    a = np.ascontiguousarray(a, dtype=F32)
    u = a.view(np.uint32).astype(np.uint64)
    nan = np.isnan(a)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = r.astype(np.uint32).view(F32).copy()
    out[nan] = np.nan
    return out


def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    return (bf16_round(a).view(np.uint32) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(F32)


# --------------------------------------------------------------------------- A1 RMSNorm
def ref_rmsnorm_fwd(x, gamma, eps, order="pairwise"):
    """y = T(f32(gamma) * (f32(x) / sqrt(mean(f32(x)^2) + eps))).

    Reference composition: src/librarium/llama.rs:442-451 (cast -> square ->
    inner_mean -> +eps -> sqrt -> broadcast div -> broadcast mul -> lossy_cast).
    square src/thunk/op.rs:2553, inner_mean :3211, add_scalar :1426, sqrt :2640,
    broadcast div :2430 and mul :2129 promote both sides to f32.
    Returns (y, t, s): t = x/s in f32, s = sqrt(v+eps) per row (f32)."""
    T = x.dtype
    xf = x.astype(F32)
    q = xf * xf
    v = _sum_rows(q, order) / F32(x.shape[-1])
    s = np.sqrt(v + F32(eps), dtype=F32)
    t = xf / s[..., None]
    y = (gamma.astype(F32)[None, :] * t).astype(T)
    return y, t, s


def ref_rmsnorm_bwd(x, gamma, dy, eps, order="pairwise", cross_row="f32"):
    """Adjoint of ref_rmsnorm_fwd with the reference's rounding points.

    dx is accumulated from two contributions, each rounded to T before the add
    (two separate `+=` in T): the broadcast-div branch and the square branch
    (sqrt adjoint src/thunk/op.rs:2643-2649, square adjoint :2556-2558, generic
    Futhark vjp for broadcast mul/div and inner_mean src/thunk/mod.rs:523-667;
    adjoint dtype = primal argument dtype :594-595).
    cross_row: "f32" sums the per-row dgamma terms in f32 and rounds once;
    "T" rounds every per-row term to T first and sums in T (the other shape the
    vjp of a broadcast f16 argument can take)."""
    T = x.dtype
    D = F32(x.shape[-1])
    _, t, s = ref_rmsnorm_fwd(x, gamma, eps, order)
    xf = x.astype(F32)
    gf = dy.astype(F32)
    gam = gamma.astype(F32)[None, :]
    if cross_row == "f32":
        dgamma = _sum_cols(gf * t, order).astype(T)
    else:
        dgamma = _sum_cols((gf * t).astype(T), order)
    dt = gam * gf
    dx1 = (dt / s[:, None]).astype(T)
    ds = _sum_rows(dt * (-xf / (s * s)[:, None]), order)
    dv = ds / (s + s)
    dq = dv / D
    dxf = dq[:, None] * (xf + xf)
    dx2 = dxf.astype(T)
    dx = (dx1 + dx2).astype(T)
    return dx, dgamma


def ideal64_rmsnorm(x, gamma, dy, eps):
    """fp64 evaluation with one final rounding: y, dx, dgamma."""
    T = x.dtype
    x64, g64, dy64 = x.astype(F64), gamma.astype(F64), dy.astype(F64)
    D = x.shape[-1]
    s = np.sqrt((x64 * x64).mean(axis=-1) + F64(F32(eps)))
    t = x64 / s[:, None]
    y = g64[None, :] * t
    dgamma = (dy64 * t).sum(axis=0)
    c = (g64[None, :] * dy64 * x64).sum(axis=-1)
    dx = (g64[None, :] * dy64) / s[:, None] - x64 * (c / (D * s ** 3))[:, None]
    return y.astype(T), dx.astype(T), dgamma.astype(T)


# --------------------------------------------------------------------------- A2 masked row softmax
def causal_keep_mask(rows, cols, q_div, q_mod, q_off=0):
    """keep[r, c] = not (c > q_pos(r)), q_pos(r) = (r // q_div) % q_mod + q_off.

    The reference mask (BlockTriElemAffine, src/thunk/op.rs:4238-4257) compares
    the index of dim 1 with the index of dim 3 of a [B,Sq,H,Sk] tensor; with the
    rows flattened, q_pos = (r // H) % Sq.  A [B,H,Sq,Sk] layout has
    q_pos = r % Sq (q_div = 1)."""
    r = np.arange(rows, dtype=np.int64)
    q = (r // q_div) % q_mod + q_off
    c = np.arange(cols, dtype=np.int64)
    return c[None, :] <= q[:, None]


def _softmax_f32(a, order):
    m = a.max(axis=-1)
    e = np.exp(a - m[:, None], dtype=F32)
    z = _sum_rows(e, order)
    return e / z[:, None]


def ref_softmax_fwd(scores, keep=None, order="pairwise"):
    """P = T(softmax_row(mask(f32(S)))).  scores: [rows, cols] in T.

    cast src/librarium/llama.rs:502; mask (upper: 0*u + -inf) :466-468 and
    src/thunk/op.rs:4248; inner_softmax src/thunk/op.rs:3296-3372 (max, exp of
    difference, sum, true division); lossy_cast back llama.rs:505.
    Returns (P, y) with y the f32 probabilities."""
    T = scores.dtype
    a = scores.astype(F32)
    if keep is not None:
        a = np.where(keep, a, F32(-np.inf))
    y = _softmax_f32(a, order)
    return y.astype(T), y


def ref_softmax_bwd(scores, dP, keep=None, order="pairwise"):
    """dS = T(mask'(u - (sum u) y)), u = y*f32(dP), y recomputed in f32.

    Recomputation of y: src/thunk/op.rs:3376-3382; post_adj :3443-3445; mask
    adjoint (upper -> 0*da + 0) :4265-4276; cast adjoint = lossy_cast :658-662."""
    T = scores.dtype
    _, y = ref_softmax_fwd(scores, keep, order)
    g = dP.astype(F32)
    u = y * g
    c = _sum_rows(u, order)
    da = u - c[:, None] * y
    if keep is not None:
        da = np.where(keep, da, F32(0))
    return da.astype(T)


def ideal64_softmax(scores, dP, keep=None):
    T = scores.dtype
    a = scores.astype(F64)
    if keep is not None:
        a = np.where(keep, a, -np.inf)
    e = np.exp(a - a.max(axis=-1, keepdims=True))
    y = e / e.sum(axis=-1, keepdims=True)
    u = y * dP.astype(F64)
    da = u - u.sum(axis=-1, keepdims=True) * y
    if keep is not None:
        da = np.where(keep, da, 0.0)
    return y.astype(T), da.astype(T)


# --------------------------------------------------------------------------- A3 RoPE
def ref_rope_tables(seq, head_dim, theta=10000.0, dtype=F16):
    """cos/sin tables [seq, head_dim], computed in f32 then rounded to dtype.

    src/librarium/llama.rs:389-411: exp_i = f32(i) * (-2/hd); inv_freq = theta **
    exp_i; freq = pos (outer) inv_freq; freq2 = concat(freq, freq); cos, sin."""
    half = head_dim // 2
    e = np.arange(half, dtype=F32) * F32(-2.0 / head_dim)
    inv_freq = np.power(F32(theta), e, dtype=F32)
    pos = np.arange(seq, dtype=F32)
    freq = (pos[:, None] * inv_freq[None, :]).astype(F32)
    freq2 = np.concatenate([freq, freq], axis=-1)
    return np.cos(freq2, dtype=F32).astype(dtype), np.sin(freq2, dtype=F32).astype(dtype)


def _rot(x):
    h = x.shape[-1] // 2
    return np.concatenate([-x[..., h:], x[..., :h]], axis=-1)


def _rot_adj(z):
    h = z.shape[-1] // 2
    return np.concatenate([z[..., h:], -z[..., :h]], axis=-1)


def ref_rope_fwd(x, cos, sin, pos):
    """y = (x (*) cos) (+) (rot(x) (*) sin), every op rounded in x's dtype.

    x: [tokens, heads, hd]; cos/sin: [seq, hd]; pos: [tokens] int.
    symplectic_embed src/librarium/llama.rs:463-465; rotate-half :999-1046;
    both operands share one dtype so the arithmetic type is that dtype
    (src/thunk/op.rs:2126-2133)."""
    c = cos[pos][:, None, :]
    s = sin[pos][:, None, :]
    a = x * c
    b = _rot(x) * s
    return a + b


def ref_rope_bwd(dy, cos, sin, pos):
    """dx = (g (*) cos) (+) R(g (*) sin), R(z) = [z[h:], -z[:h]] (tables are constants)."""
    c = cos[pos][:, None, :]
    s = sin[pos][:, None, :]
    return dy * c + _rot_adj(dy * s)


def ideal64_rope(x, dy, cos, sin, pos):
    T = x.dtype
    c = cos.astype(F64)[pos][:, None, :]
    s = sin.astype(F64)[pos][:, None, :]
    x64, g64 = x.astype(F64), dy.astype(F64)
    return (x64 * c + _rot(x64) * s).astype(T), (g64 * c + _rot_adj(g64 * s)).astype(T)


# --------------------------------------------------------------------------- A4 SwiGLU
def _exp_T(x):
    """exp of a T array evaluated in f32 and rounded to T.  (numpy's native float16 exp loop is a
    reduced-accuracy half-precision routine on CPUs with AVX512-FP16, so it is never used here.)"""
    return np.exp(x.astype(F32), dtype=F32).astype(x.dtype)


def ref_swiglu_fwd(gate, up):
    """h = silu(g) (*) u with silu(g) = g / (1 + exp(-g)), rounded per primitive.

    standard_silu src/thunk/op.rs:2898; mul :2047; call site
    src/librarium/llama.rs:526-527.  Returns (h, y) with y = silu(g)."""
    T = gate.dtype
    one = T.type(1)
    y = gate / (one + _exp_T(-gate))
    return y * up, y


def ref_swiglu_bwd(gate, up, dh):
    """du = y*dh; dg = (dh*u) * (y*(1-t) + t), t = logistic(g) = 1/(1+exp(-g)).

    mul adjoint src/thunk/op.rs:2050-2054; silu adjoint :2901-2908; logistic :2852."""
    T = gate.dtype
    one = T.type(1)
    _, y = ref_swiglu_fwd(gate, up)
    du = y * dh
    dy = dh * up
    t = one / (one + _exp_T(-gate))
    dg = dy * (y * (one - t) + t)
    return dg, du


def ideal64_swiglu(gate, up, dh):
    T = gate.dtype
    g, u, d = gate.astype(F64), up.astype(F64), dh.astype(F64)
    t = 1.0 / (1.0 + np.exp(-g))
    y = g * t
    return (y * u).astype(T), (d * u * (y * (1 - t) + t)).astype(T), (y * d).astype(T)


# --------------------------------------------------------------------------- A5 softmax-NLL
def ref_softmax_nll(logits, targets, w, order="pairwise"):
    """Per-row loss and dlogits.

    loss_i = -log(softmax(f32(x_i))[k_i]) (src/thunk/op.rs:3520-3546); dlogits =
    T(w_i * (softmax(x_i) - onehot(k_i))) (adjoint :3555-3567: recomputed softmax,
    dense one-hot :937-994, sub, broadcast mul by the upstream per-row scale).
    Targets outside [0, V) are a reference assertion failure (:3538); here they
    raise.  Returns (loss_rows f32, dlogits T, gathered logit T)."""
    T = logits.dtype
    rows, V = logits.shape
    k = np.asarray(targets).astype(np.int64)
    if ((k < 0) | (k >= V)).any():
        raise IndexError("target out of range")
    a = logits.astype(F32)
    y = _softmax_f32(a, order)
    idx = np.arange(rows)
    loss = -np.log(y[idx, k], dtype=F32)
    onehot = np.zeros_like(y)
    onehot[idx, k] = F32(1)
    w = np.broadcast_to(np.asarray(w, dtype=F32), (rows,))
    d = (w[:, None] * (y - onehot)).astype(T)
    return loss, d, logits[idx, k]


def ideal64_softmax_nll(logits, targets, w):
    T = logits.dtype
    rows, V = logits.shape
    k = np.asarray(targets).astype(np.int64)
    a = logits.astype(F64)
    m = a.max(axis=-1, keepdims=True)
    lse = m[:, 0] + np.log(np.exp(a - m).sum(axis=-1))
    idx = np.arange(rows)
    loss = lse - a[idx, k]
    y = np.exp(a - lse[:, None])
    y[idx, k] -= 1.0
    w = np.broadcast_to(np.asarray(w, dtype=F64), (rows,))
    return loss, (w[:, None] * y).astype(T)


# --------------------------------------------------------------------------- A8 embedding gather / scatter-add
def ref_gather_rows(table, tokens):
    """out[i] = table[tok[i]] (bit-exact copy).  outer_select src/thunk/op.rs:1288-1311."""
    k = np.asarray(tokens).astype(np.int64)
    if ((k < 0) | (k >= table.shape[0])).any():
        raise IndexError("token out of range")
    return table[k]


def ref_scatter_add_rows(dy, tokens, vocab, cross_row="f32"):
    """dE[v] = sum over i with tok[i]==v of dy[i] (adjoint of the gather, produced
    by Futhark vjp; src/thunk/op.rs:1229-1314 has no hand-written pop_adj).
    cross_row as in ref_rmsnorm_bwd."""
    T = dy.dtype
    k = np.asarray(tokens).astype(np.int64)
    acc = np.zeros((vocab, dy.shape[1]), dtype=F32 if cross_row == "f32" else T)
    for i in range(dy.shape[0]):          # token order
        acc[k[i]] = acc[k[i]] + dy[i].astype(acc.dtype)
    return acc.astype(T)


# --------------------------------------------------------------------------- A9 add / accumulate
def ref_add(a, b):
    """Elementwise add in the operands' dtype (AddFutThunkSpec src/thunk/op.rs:1480-1535;
    Accumulate mode `oy + y`, src/thunk/mod.rs:1691-1733)."""
    return a + b


# --------------------------------------------------------------------------- AdamW32 (optimizer thunks)
def ref_adamw32_step(w, m, v, g, iter_nr, lr=1e-3, wd=0.0, a1=0.1, a2=1e-3, eps=1e-8, grad_unscale=1.0, param_dtype=None):
    """AdamW32::step (src/librarium/adamw.rs:46-61): three in-place f32 programs, evaluated in order.

    m <- m + a1*(s*f32(g) - m)                      src/thunk/op.rs:3929-3934
    v <- v + a2*((s*f32(g))*(s*f32(g)) - v)         :3991-3998
    w <- w + (-lr)*(u*(m/(sqrt(v)+e)) + wd*w)       :4051-4055, scalars as in src/op.rs:985-1012
    Returns new (w, m, v[, param]) as f32 arrays (param in param_dtype)."""
    f = F32

    def powi(a, b):          # f32 repeated squaring, as Rust's f32::powi (src/op.rs:990,1000)
        r = f(1.0)
        while True:
            if b & 1:
                r = f(r * a)
            b //= 2
            if b == 0:
                return r
            a = f(a * a)

    a1f, a2f = f(a1), f(a2)
    unbias1 = a1f if iter_nr == 1 else f(f(1.0) - powi(f(1.0) - a1f, iter_nr))
    unbias2 = np.sqrt(a2f) if iter_nr == 1 else np.sqrt(f(f(1.0) - powi(f(1.0) - a2f, iter_nr)))
    u = f(unbias2 / unbias1)
    e = f(f(eps) * unbias2)
    sg = f(grad_unscale) * g.astype(F32)
    m2 = m + a1f * (sg - m)
    v2 = v + a2f * (sg * sg - v)
    w2 = w + f(-lr) * (u * (m2 / (np.sqrt(v2) + e)) + f(wd) * w)
    out = (w2.astype(F32), m2.astype(F32), v2.astype(F32))
    if param_dtype is not None:
        out = out + (w2.astype(param_dtype),)
    return out


# --------------------------------------------------------------------------- A6/A7 GEMM
def ref_gemm(a, b, ta=False, tb=False, alpha=1.0, beta=0.0, c=None):
    """C = T(alpha * op(A) op(B) + beta * C), fp64 accumulation then one rounding.

    cuBLAS GemmEx with f16 operands and COMPUTE_32F, no reduced-precision
    reductions (cacti_gpu_cu_ffi/src/lib.rs:727-791); call site
    src/thunk/op.rs:4658-4668."""
    T = a.dtype
    A = a.astype(F64).T if ta else a.astype(F64)
    B = b.astype(F64).T if tb else b.astype(F64)
    acc = F64(F32(alpha)) * (A @ B)
    if beta != 0.0 and c is not None:
        acc = acc + F64(F32(beta)) * c.astype(F64)
    return acc.astype(T)


def ref_block_gemm(a, b, ta=False, tb=False, alpha=1.0, beta=0.0, c=None):
    """4-d block matmul: a [nrow_a, ra, ncol_a, ca], b [nrow_b, rb, ncol_b, cb];
    per block (i, j): C[i,:,j,:] = alpha * op(A[i,:,j,:]) op(B[i,:,j,:]) (+ beta C),
    block-broadcast when an operand has nrow or ncol equal to 1.

    BlockMatrixMulThunkSpec::_calculate_out_ty src/thunk/op.rs:4936-5022; base
    pointer arithmetic :5174-5189."""
    T = a.dtype
    nrow = max(a.shape[0], b.shape[0])
    ncol = max(a.shape[2], b.shape[2])
    outs = None
    for i in range(nrow):
        for j in range(ncol):
            A = a[i if a.shape[0] > 1 else 0, :, j if a.shape[2] > 1 else 0, :].astype(F64)
            B = b[i if b.shape[0] > 1 else 0, :, j if b.shape[2] > 1 else 0, :].astype(F64)
            A = A.T if ta else A
            B = B.T if tb else B
            blk = F64(F32(alpha)) * (A @ B)
            if outs is None:
                outs = np.zeros((nrow, blk.shape[0], ncol, blk.shape[1]), dtype=F64)
            outs[i, :, j, :] = blk
    if beta != 0.0 and c is not None:
        outs = outs + F64(F32(beta)) * c.astype(F64)
    return outs.astype(T)


def ref_causal_attention(q, k, v, alpha, round_scores=None):
    """The attention block of one decoder layer as the reference stages it (src/librarium/llama.rs:501-507):
    block_matmul_scale (scores = alpha q.k, fp32 accumulation, stored in the operand type), cast to f32,
    block_causal_attention_mask (src/thunk/op.rs:4189-4278), inner_softmax (:3257-3383), lossy_cast, block_matmul.
    q, k, v: [B, S, H, hd].  Computed in f64 from the rounded scores, with no rounding of the probabilities, so that
    both the reference's chain (which rounds exp / sum) and a fused kernel (which may round exp) can be held to it.
    round_scores: function rounding an f32 array to the storage type (default: the dtype of q).
    Returns (ctx [B, S, H, hd] f64, row maximum [B, H, S], row sum of exp(s - max) [B, H, S],
    sum_j p_j |v_j| [B, S, H, hd], the magnitude rounding errors scale with)."""
    qf, kf, vf = (np.transpose(t.astype(F64), (0, 2, 1, 3)) for t in (q, k, v))               # [B, H, S, hd]
    acc = np.einsum("bhqd,bhkd->bhqk", qf, kf).astype(F32)
    sc32 = F32(alpha) * acc
    sc = (sc32.astype(q.dtype) if round_scores is None else round_scores(sc32)).astype(F64)
    s = sc.shape[-1]
    sc = np.where(np.tril(np.ones((s, s), bool)), sc, -np.inf)
    m = sc.max(-1, keepdims=True)
    e = np.exp(sc - m)
    l = e.sum(-1, keepdims=True)
    ctx = np.einsum("bhqk,bhkd->bhqd", e / l, vf)
    mag = np.einsum("bhqk,bhkd->bhqd", e / l, np.abs(vf))
    return np.transpose(ctx, (0, 2, 1, 3)), m[..., 0], l[..., 0], np.transpose(mag, (0, 2, 1, 3))



# --------------------------------------------------------------------------- seeded inputs
def normal(seed, shape, dtype=F32, scale=1.0, shift=0.0):
    """standard_normal in f32 from default_rng(seed), scaled and shifted, then cast."""
    a = np.random.default_rng(seed).standard_normal(shape, dtype=F32)
    return (a * F32(scale) + F32(shift)).astype(dtype)


def uniform_int(seed, n, hi, dtype=np.int32):
    return np.random.default_rng(seed).integers(0, hi, size=n).astype(dtype)
