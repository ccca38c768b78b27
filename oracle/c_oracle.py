"""ctypes front end of oracle/libref_chain.so (the C/OpenMP restatement).  Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None
_SUF = {np.dtype(np.float32): "f32", np.dtype(np.float16): "f16"}


def lib():
    global _lib
    if _lib is None:
        path = _build.LIB
        if not os.path.exists(path):
            path = _build.build()
        _lib = C.CDLL(path)
        _lib.rc_num_threads.restype = C.c_int
    return _lib


def num_threads() -> int:
    return lib().rc_num_threads()


def set_num_threads(n: int) -> None:
    lib().rc_set_num_threads(int(n))


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _fn(name, dtype):
    f = getattr(lib(), f"{name}_{_SUF[np.dtype(dtype)]}")
    f.restype = C.c_int
    return f


def rmsnorm_fwd_bwd(x, gamma, dy, eps, do_bwd=True):
    rows, cols = x.shape
    y, dx, dg = np.empty_like(x), np.empty_like(x), np.empty_like(gamma)
    rc = _fn("rc_rmsnorm_fwd_bwd", x.dtype)(_p(x), _p(gamma), _p(dy), C.c_float(eps), C.c_int64(rows), C.c_int64(cols),
                                            _p(y), _p(dx), _p(dg), C.c_int(int(do_bwd)))
    assert rc == 0
    return y, dx, dg


def softmax_fwd_bwd(s, dp, mask=None, do_bwd=True):
    rows, cols = s.shape
    p, ds = np.empty_like(s), np.empty_like(s)
    q_div, q_mod, q_off = mask if mask is not None else (1, 1, 0)
    rc = _fn("rc_softmax_fwd_bwd", s.dtype)(_p(s), _p(dp), C.c_int64(rows), C.c_int64(cols), C.c_int(mask is not None),
                                            C.c_int64(q_div), C.c_int64(q_mod), C.c_int64(q_off), _p(p), _p(ds),
                                            C.c_int(int(do_bwd)))
    assert rc == 0
    return p, ds


def rope_fwd_bwd(x, dy, cos, sin, pos_off=0, do_bwd=True):
    tokens, heads, hd = x.shape
    y, dx = np.empty_like(x), np.empty_like(x)
    rc = _fn("rc_rope_fwd_bwd", x.dtype)(_p(x), _p(dy), _p(cos), _p(sin), C.c_int64(tokens), C.c_int64(heads),
                                         C.c_int64(hd), C.c_int64(cos.shape[0]), C.c_int64(pos_off), _p(y), _p(dx),
                                         C.c_int(int(do_bwd)))
    assert rc == 0
    return y, dx


def swiglu_fwd_bwd(gate, up, dh, do_bwd=True):
    h, dg, du = np.empty_like(gate), np.empty_like(gate), np.empty_like(gate)
    rc = _fn("rc_swiglu_fwd_bwd", gate.dtype)(_p(gate), _p(up), _p(dh), C.c_int64(gate.size), _p(h), _p(dg), _p(du),
                                              C.c_int(int(do_bwd)))
    assert rc == 0
    return h, dg, du


def softmax_nll_fwd_bwd(logits, targets, w_scalar, w_rows=None, do_bwd=True):
    rows, cols = logits.shape
    tg = np.ascontiguousarray(targets, dtype=np.int32)
    loss = np.empty(rows, dtype=np.float32)
    dl = np.empty_like(logits)
    rc = _fn("rc_softmax_nll_fwd_bwd", logits.dtype)(_p(logits), _p(tg), _p(w_rows), C.c_float(w_scalar),
                                                     C.c_int64(rows), C.c_int64(cols), _p(loss), _p(dl),
                                                     C.c_int(int(do_bwd)))
    if rc == 2:
        raise IndexError("target out of range")
    assert rc == 0
    return loss, dl
