"""Torch-tensor front end of the C ABI: argument marshalling only, no arithmetic.

Every function takes CUDA tensors (torch owns the memory and the stream), passes raw pointers to
libcacti_b200.so and raises CactiB200Error on a non-zero return code.  Function names follow the
C ABI, which follows the reference ops: rms_norm (src/librarium/llama.rs:442-451), inner_softmax
(src/op.rs trait MathUnaryOps), symplectic_embed (llama.rs:463-465), standard_silu * up
(llama.rs:526-527), inner_softmax_categorical_nll (src/op.rs:1223-1231), outer_select
(src/op.rs:1207-1220).
"""
from __future__ import annotations

import torch

from . import capi
from .capi import MASK_CAUSAL, MASK_CAUSAL_TRIM, MASK_NONE, R_16BF, R_16F, R_16U, R_32F, R_32I, check, lib

_DT = {torch.float32: R_32F, torch.float16: R_16F, torch.bfloat16: R_16BF}
_IDX = {torch.int32: R_32I, torch.uint16: R_16U, torch.int16: R_16U}


def _dt(t: torch.Tensor) -> int:
    return _DT[t.dtype]


def _ptr(t) -> int:
    if t is None:
        return 0
    if not t.is_cuda:
        raise ValueError("cacti_b200 takes device tensors only (there is no CPU path)")
    return t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _ws(nbytes: int, device) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


# ---- K1 ---------------------------------------------------------------------------------------
def rmsnorm_workspace(rows: int, cols: int, device) -> torch.Tensor:
    return _ws(lib().cacti_b200_rmsnorm_workspace_bytes(rows, cols), device)


def rmsnorm_fwd(x, gamma, eps, y=None):
    rows, cols = x.shape
    y = torch.empty_like(x) if y is None else y
    check(lib().cacti_b200_rmsnorm_fwd(_ptr(y), _ptr(x), _ptr(gamma), eps, rows, cols, _dt(x), _stream()), "rmsnorm_fwd")
    return y


def add_rmsnorm_fwd(a, b, gamma, eps, y=None, total=None):
    """(y, total) with total = a + b (rounded to the storage type) and y = rmsnorm(total); one pass over HBM."""
    rows, cols = a.shape
    y = torch.empty_like(a) if y is None else y
    total = torch.empty_like(a) if total is None else total
    check(lib().cacti_b200_add_rmsnorm_fwd(_ptr(y), _ptr(total), _ptr(a), _ptr(b), _ptr(gamma), eps, rows, cols, _dt(a),
                                           _stream()), "add_rmsnorm_fwd")
    return y, total


def rmsnorm_bwd(x, gamma, dy, eps, dx=None, dgamma=None, beta_dx=0, beta_dgamma=0, dgamma_dtype=None, workspace=None):
    rows, cols = x.shape
    dx = torch.empty_like(x) if dx is None else dx
    if dgamma is None:
        dgamma = torch.empty(cols, dtype=dgamma_dtype or x.dtype, device=x.device)
    ws = rmsnorm_workspace(rows, cols, x.device) if workspace is None else workspace
    check(lib().cacti_b200_rmsnorm_bwd(_ptr(dx), _ptr(dgamma), _ptr(dy), _ptr(x), _ptr(gamma), eps, rows, cols, _dt(x),
                                       _dt(dgamma), beta_dx, beta_dgamma, _ptr(ws), ws.numel(), _stream()), "rmsnorm_bwd")
    return dx, dgamma


def rmsnorm_fwd_bwd(x, gamma, dy, eps, y=None, dx=None, dgamma=None, beta_dx=0, beta_dgamma=0, dgamma_dtype=None,
                    workspace=None):
    rows, cols = x.shape
    y = torch.empty_like(x) if y is None else y
    dx = torch.empty_like(x) if dx is None else dx
    if dgamma is None:
        dgamma = torch.empty(cols, dtype=dgamma_dtype or x.dtype, device=x.device)
    ws = rmsnorm_workspace(rows, cols, x.device) if workspace is None else workspace
    check(lib().cacti_b200_rmsnorm_fwd_bwd(_ptr(y), _ptr(dx), _ptr(dgamma), _ptr(x), _ptr(gamma), _ptr(dy), eps, rows,
                                           cols, _dt(x), _dt(dgamma), beta_dx, beta_dgamma, _ptr(ws), ws.numel(),
                                           _stream()), "rmsnorm_fwd_bwd")
    return y, dx, dgamma


# ---- K2 ---------------------------------------------------------------------------------------
def _mask_args(mask):
    """mask: None, (q_div, q_mod, q_off) or (q_div, q_mod, q_off, trim); trim selects CACTI_B200_MASK_CAUSAL_TRIM."""
    if mask is None:
        return MASK_NONE, 1, 1, 0
    q_div, q_mod, q_off = mask[:3]
    return (MASK_CAUSAL_TRIM if len(mask) > 3 and mask[3] else MASK_CAUSAL), q_div, q_mod, q_off


def softmax_fwd(s, mask=None, p=None):
    rows, cols = s.shape
    p = torch.empty_like(s) if p is None else p
    m = _mask_args(mask)
    check(lib().cacti_b200_softmax_fwd(_ptr(p), _ptr(s), rows, cols, *m, _dt(s), _stream()), "softmax_fwd")
    return p


def softmax_bwd(s, dp, mask=None, ds=None, beta=0):
    rows, cols = s.shape
    ds = torch.empty_like(s) if ds is None else ds
    m = _mask_args(mask)
    check(lib().cacti_b200_softmax_bwd(_ptr(ds), _ptr(s), _ptr(dp), rows, cols, *m, _dt(s), beta, _stream()), "softmax_bwd")
    return ds


def softmax_fwd_bwd(s, dp, mask=None, p=None, ds=None, beta=0):
    rows, cols = s.shape
    p = torch.empty_like(s) if p is None else p
    ds = torch.empty_like(s) if ds is None else ds
    m = _mask_args(mask)
    check(lib().cacti_b200_softmax_fwd_bwd(_ptr(p), _ptr(ds), _ptr(s), _ptr(dp), rows, cols, *m, _dt(s), beta, _stream()),
          "softmax_fwd_bwd")
    return p, ds


# ---- K3 ---------------------------------------------------------------------------------------
def rope_tables(seq, head_dim, theta=10000.0, dtype=torch.float16, device="cuda"):
    cos = torch.empty(seq, head_dim, dtype=dtype, device=device)
    sin = torch.empty_like(cos)
    check(lib().cacti_b200_rope_tables(_ptr(cos), _ptr(sin), seq, head_dim, theta, _DT[dtype], _stream()), "rope_tables")
    return cos, sin


def rope_fwd(x, cos, sin, pos_off=0, y=None):
    tokens, heads, hd = x.shape
    y = torch.empty_like(x) if y is None else y
    check(lib().cacti_b200_rope_fwd(_ptr(y), _ptr(x), _ptr(cos), _ptr(sin), tokens, heads, hd, cos.shape[0], pos_off,
                                    _dt(x), _stream()), "rope_fwd")
    return y


def rope_fwd_pitched(x, cos, sin, head_pitch=128, pos_off=0, y=None):
    """RoPE whose output heads are head_pitch wide, zeros after head_dim (= rope_fwd then block_pad, in one pass)."""
    tokens, heads, hd = x.shape
    y = torch.empty(tokens, heads, head_pitch, dtype=x.dtype, device=x.device) if y is None else y
    check(lib().cacti_b200_rope_fwd_pitched(_ptr(y), _ptr(x), _ptr(cos), _ptr(sin), tokens, heads, hd, head_pitch,
                                            cos.shape[0], pos_off, _dt(x), _stream()), "rope_fwd_pitched")
    return y


def rope_bwd(dy, cos, sin, pos_off=0, dx=None, beta=0):
    tokens, heads, hd = dy.shape
    dx = torch.empty_like(dy) if dx is None else dx
    check(lib().cacti_b200_rope_bwd(_ptr(dx), _ptr(dy), _ptr(cos), _ptr(sin), tokens, heads, hd, cos.shape[0], pos_off,
                                    _dt(dy), beta, _stream()), "rope_bwd")
    return dx


def rope_fwd_bwd(x, dy, cos, sin, pos_off=0, y=None, dx=None, beta=0):
    tokens, heads, hd = x.shape
    y = torch.empty_like(x) if y is None else y
    dx = torch.empty_like(x) if dx is None else dx
    check(lib().cacti_b200_rope_fwd_bwd(_ptr(y), _ptr(dx), _ptr(x), _ptr(dy), _ptr(cos), _ptr(sin), tokens, heads, hd,
                                        cos.shape[0], pos_off, _dt(x), beta, _stream()), "rope_fwd_bwd")
    return y, dx


# ---- K4 ---------------------------------------------------------------------------------------
def swiglu_fwd(gate, up, h=None):
    h = torch.empty_like(gate) if h is None else h
    check(lib().cacti_b200_swiglu_fwd(_ptr(h), _ptr(gate), _ptr(up), gate.numel(), _dt(gate), _stream()), "swiglu_fwd")
    return h


def swiglu_bwd(gate, up, dh, dgate=None, dup=None, beta_dgate=0, beta_dup=0):
    dgate = torch.empty_like(gate) if dgate is None else dgate
    dup = torch.empty_like(gate) if dup is None else dup
    check(lib().cacti_b200_swiglu_bwd(_ptr(dgate), _ptr(dup), _ptr(gate), _ptr(up), _ptr(dh), gate.numel(), _dt(gate),
                                      beta_dgate, beta_dup, _stream()), "swiglu_bwd")
    return dgate, dup


def swiglu_fwd_bwd(gate, up, dh, h=None, dgate=None, dup=None, beta_dgate=0, beta_dup=0):
    h = torch.empty_like(gate) if h is None else h
    dgate = torch.empty_like(gate) if dgate is None else dgate
    dup = torch.empty_like(gate) if dup is None else dup
    check(lib().cacti_b200_swiglu_fwd_bwd(_ptr(h), _ptr(dgate), _ptr(dup), _ptr(gate), _ptr(up), _ptr(dh), gate.numel(),
                                          _dt(gate), beta_dgate, beta_dup, _stream()), "swiglu_fwd_bwd")
    return h, dgate, dup


# ---- K5 ---------------------------------------------------------------------------------------
def softmax_nll_fwd_bwd(logits, targets, w=None, w_scalar=1.0, want_grad=True, want_sum=True, want_rows=True,
                        dlogits=None, beta=0, status=None):
    """Returns (loss_sum f32[1] | None, loss_rows f32[rows] | None, dlogits | None, status u32[1])."""
    rows, vocab = logits.shape
    dev = logits.device
    loss_sum = torch.empty(1, dtype=torch.float32, device=dev) if want_sum else None
    loss_rows = torch.empty(rows, dtype=torch.float32, device=dev) if want_rows else None
    if want_grad and dlogits is None:
        dlogits = torch.empty_like(logits)
    status = torch.zeros(1, dtype=torch.int32, device=dev) if status is None else status
    ws = _ws(lib().cacti_b200_softmax_nll_workspace_bytes(rows), dev)
    check(lib().cacti_b200_softmax_nll_fwd_bwd(_ptr(loss_sum), _ptr(loss_rows), _ptr(dlogits) if want_grad else 0,
                                               _ptr(logits), _ptr(targets), _IDX[targets.dtype], _ptr(w), w_scalar, rows,
                                               vocab, _dt(logits), beta, _ptr(status), _ptr(ws), ws.numel(), _stream()),
          "softmax_nll_fwd_bwd")
    return loss_sum, loss_rows, (dlogits if want_grad else None), status


# ---- K6 ---------------------------------------------------------------------------------------
def gather_rows(table, tokens, out=None, status=None):
    vocab, cols = table.shape
    n = tokens.numel()
    out = torch.empty(n, cols, dtype=table.dtype, device=table.device) if out is None else out
    status = torch.zeros(1, dtype=torch.int32, device=table.device) if status is None else status
    check(lib().cacti_b200_gather_rows(_ptr(out), _ptr(table), _ptr(tokens), _IDX[tokens.dtype], n, vocab, cols,
                                       _dt(table), _ptr(status), _stream()), "gather_rows")
    return out, status


def scatter_add_rows(dy, tokens, vocab, dtable=None, beta=0, status=None):
    n, cols = dy.shape
    dev = dy.device
    dtable = torch.empty(vocab, cols, dtype=dy.dtype, device=dev) if dtable is None else dtable
    status = torch.zeros(1, dtype=torch.int32, device=dev) if status is None else status
    ws = _ws(lib().cacti_b200_scatter_add_rows_workspace_bytes(n, vocab), dev)
    check(lib().cacti_b200_scatter_add_rows(_ptr(dtable), _ptr(dy), _ptr(tokens), _IDX[tokens.dtype], n, vocab, cols,
                                            _dt(dy), beta, _ptr(ws), ws.numel(), _ptr(status), _stream()),
          "scatter_add_rows")
    return dtable, status


# ---- K7 ---------------------------------------------------------------------------------------
def accumulate(dst, src):
    check(lib().cacti_b200_accumulate(_ptr(dst), _ptr(src), dst.numel(), _dt(dst), _stream()), "accumulate")
    return dst


def add(a, b, out=None):
    out = torch.empty_like(a) if out is None else out
    check(lib().cacti_b200_add(_ptr(out), _ptr(a), _ptr(b), a.numel(), _dt(a), _stream()), "add")
    return out


# ---- K8 ---------------------------------------------------------------------------------------
def adamw32_step(master, grad1_avg, grad2_avg, grad, iter_nr, lr=1e-3, wd=0.0, a1=0.1, a2=1e-3, eps=1e-8, grad_unscale=1.0,
                 param_out=None):
    check(lib().cacti_b200_adamw32_step(_ptr(master), _ptr(grad1_avg), _ptr(grad2_avg), _ptr(param_out), _ptr(grad),
                                        master.numel(), _dt(grad), _dt(param_out) if param_out is not None else R_16F,
                                        grad_unscale, lr, wd, a1, a2, eps, iter_nr, _stream()), "adamw32_step")


# ---- G1 / G2 ------------------------------------------------------------------------------------
import ctypes as _C


def _scalars(alpha, beta):
    return _C.byref(_C.c_float(alpha)), _C.byref(_C.c_float(beta))


def gemm_workspace(m, n, k, device) -> torch.Tensor:
    """Workspace of a dense matmul: room to repack operands TMA cannot address, and for the partial sums of the
    k-split schedule (a matmul given no workspace computes every tile whole)."""
    return _ws(lib().cacti_b200_gemm_workspace_bytes(m, n, k, 1, 1), device)


def gemm(a, b, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, c=None, workspace=None):
    """C = alpha * op(A) op(B) + beta * C on 2-d row-major tensors (any row stride, unit column stride)."""
    m = a.shape[1] if trans_a else a.shape[0]
    k = a.shape[0] if trans_a else a.shape[1]
    n = b.shape[0] if trans_b else b.shape[1]
    c = torch.empty(m, n, dtype=a.dtype, device=a.device) if c is None else c
    # a repack workspace is only needed when TMA cannot address an operand (16-byte base and row pitch)
    aligned = all(t.data_ptr() % 16 == 0 and (t.stride(0) * t.element_size()) % 16 == 0 for t in (a, b))
    ws = workspace
    if ws is None and not aligned:
        ws = gemm_workspace(m, n, k, a.device)
    al, be = _scalars(alpha, beta)
    check(lib().cacti_b200_gemm(_ptr(c), _ptr(a), _ptr(b), m, n, k, a.stride(0), b.stride(0), c.stride(0), int(trans_a),
                                int(trans_b), al, be, _dt(a), _ptr(ws), ws.numel() if ws is not None else 0, _stream()),
          "gemm")
    return c


def block_gemm(a, b, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, c=None, workspace=None, tri=0, diag=0,
               a_valid=None, b_valid=None):
    """Block matmul on the reference's 4-d layout [nrow, blk_rows, ncol, blk_cols] (packed); an operand with
    nrow or ncol equal to 1 is broadcast over that block dimension.  `tri` is a CACTI_B200_TRI_* hint
    (capi.TRI_C_LOWER / TRI_A_LOWER / TRI_A_UPPER) for the matmuls around a causal softmax.  a_valid / b_valid: the
    operand's rows are zero-padded (block_pad) and only that many leading columns are data."""
    nrow, ncol = max(a.shape[0], b.shape[0]), max(a.shape[2], b.shape[2])
    a_cols = a.shape[3] if a_valid is None else a_valid
    b_cols = b.shape[3] if b_valid is None else b_valid
    m = a_cols if trans_a else a.shape[1]
    k = a.shape[1] if trans_a else a_cols
    n = b.shape[1] if trans_b else b_cols
    flags = (1 if a_cols < a.shape[3] else 0) | (2 if b_cols < b.shape[3] else 0)
    c = torch.empty(nrow, m, ncol, n, dtype=a.dtype, device=a.device) if c is None else c

    def strides(t):
        so = t.shape[1] * t.shape[2] * t.shape[3] if t.shape[0] > 1 else 0
        si = t.shape[3] if t.shape[2] > 1 else 0
        return t.shape[2] * t.shape[3], so, si

    lda, sao, sai = strides(a)
    ldb, sbo, sbi = strides(b)
    ldc, sco, sci = strides(c)
    if workspace is None:
        workspace = _ws(lib().cacti_b200_gemm_workspace_bytes(m, n, k, nrow, ncol), a.device)
    al, be = _scalars(alpha, beta)
    if tri or flags:
        check(lib().cacti_b200_gemm_strided_batched_tri(_ptr(c), _ptr(a), _ptr(b), m, n, k, lda, ldb, ldc, int(trans_a),
                                                        int(trans_b), al, be, nrow, ncol, sao, sai, sbo, sbi, sco, sci,
                                                        int(tri), int(diag), flags, _dt(a), _ptr(workspace),
                                                        workspace.numel(), _stream()), "block_gemm_tri")
        return c
    check(lib().cacti_b200_gemm_strided_batched(_ptr(c), _ptr(a), _ptr(b), m, n, k, lda, ldb, ldc, int(trans_a),
                                                int(trans_b), al, be, nrow, ncol, sao, sai, sbo, sbi, sco, sci, _dt(a),
                                                _ptr(workspace), workspace.numel(), _stream()), "block_gemm")
    return c


# ---- A1 ---------------------------------------------------------------------------------------
def block_pad(x, cols_pad=128, out=None):
    """[nrow, rows, ncol, cols] -> [nrow, rows, ncol, cols_pad], zeros in the added columns."""
    nrow, rows, ncol, cols = x.shape
    out = torch.empty(nrow, rows, ncol, cols_pad, dtype=x.dtype, device=x.device) if out is None else out
    check(lib().cacti_b200_block_pad(_ptr(out), _ptr(x), nrow, rows, ncol, cols, cols_pad, _dt(x), _stream()), "block_pad")
    return out


def attention_fwd(q_pad, k_pad, v_pad, head_dim, alpha, ctx=None, stats=None):
    """Fused causal attention on head-dim-padded [B, S, H, 128] operands -> (ctx [B, S, H, head_dim], stats [B, H, S, 4])."""
    b, s, h, _ = q_pad.shape
    ctx = torch.empty(b, s, h, head_dim, dtype=q_pad.dtype, device=q_pad.device) if ctx is None else ctx
    stats = torch.empty(b, h, s, 4, dtype=torch.float32, device=q_pad.device) if stats is None else stats
    check(lib().cacti_b200_attention_fwd(_ptr(ctx), _ptr(stats), _ptr(q_pad), _ptr(k_pad), _ptr(v_pad), b, s, h, head_dim,
                                         alpha, _dt(q_pad), _stream()), "attention_fwd")
    return ctx, stats


def attention_bwd_prep(q_pad, k_pad, v_pad, dctx_pad, ctx, stats, alpha, p=None, ds=None):
    """(P, dS) [B, S, H, S] for the three hinted block matmuls of the attention adjoint; nothing beyond the trimmed-fill
    bound of each row is written."""
    b, s, h, _ = q_pad.shape
    p = torch.empty(b, s, h, s, dtype=q_pad.dtype, device=q_pad.device) if p is None else p
    ds = torch.empty(b, s, h, s, dtype=q_pad.dtype, device=q_pad.device) if ds is None else ds
    check(lib().cacti_b200_attention_bwd_prep(_ptr(p), _ptr(ds), _ptr(q_pad), _ptr(k_pad), _ptr(v_pad), _ptr(dctx_pad),
                                              _ptr(ctx), _ptr(stats), b, s, h, ctx.shape[-1], alpha, _dt(q_pad), _stream()),
          "attention_bwd_prep")
    return p, ds


def attention_bwd(q_pad, k_pad, v_pad, dctx_pad, ctx, stats, alpha, dq=None, dk=None, dv=None):
    """(dq, dk, dv) [B, S, H, head_dim]: the whole adjoint of attention_fwd, P and dS never leaving the SMs."""
    b, s, h, _ = q_pad.shape
    hd = ctx.shape[-1]
    dq, dk, dv = (torch.empty(b, s, h, hd, dtype=q_pad.dtype, device=q_pad.device) if t is None else t for t in (dq, dk, dv))
    check(lib().cacti_b200_attention_bwd(_ptr(dq), _ptr(dk), _ptr(dv), _ptr(q_pad), _ptr(k_pad), _ptr(v_pad), _ptr(dctx_pad), _ptr(ctx),
                                         _ptr(stats), b, s, h, hd, alpha, _dt(q_pad), _stream()), "attention_bwd")
    return dq, dk, dv
