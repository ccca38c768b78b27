"""ctypes binding of libcacti_b200.so (the C ABI declared in include/cacti_b200.h).

The library is loaded from cacti_b200/lib/ (built in-tree by cacti_b200/build.py).  There is no
fallback of any kind: if the shared object is missing or a symbol cannot be resolved, loading
raises.
"""
from __future__ import annotations

import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("CACTI_B200_LIB", os.path.join(HERE, "lib", "libcacti_b200.so"))
HEADER = os.path.join(HERE, "..", "include", "cacti_b200.h")

OK, ERR_INVALID_VALUE, ERR_DTYPE, ERR_WORKSPACE, ERR_LAUNCH, ERR_SHAPE, ERR_INDEX_RANGE, ERR_NO_DEVICE = range(8)
ERR_SCRATCH_LIMIT = 8
R_32F, R_16F, R_16BF, R_32I, R_16U = 0, 2, 14, 10, 22
MASK_NONE, MASK_CAUSAL, MASK_CAUSAL_TRIM = 0, 1, 2

_p, _i64, _int, _f32, _sz, _st = C.c_uint64, C.c_int64, C.c_int, C.c_float, C.c_size_t, C.c_void_p

# name -> (restype, argtypes); must list every function the header declares
SIGNATURES = {
    "cacti_b200_version": (_int, []),
    "cacti_b200_error_string": (C.c_char_p, [_int]),
    "cacti_b200_last_cuda_error": (_int, []),
    "cacti_b200_tune": (_int, [C.c_char_p, _int]),
    "cacti_b200_device_error": (_int, [C.POINTER(C.c_uint)]),
    "cacti_b200_selftest_bounded_wait": (_int, [_p, _int, _st]),
    "cacti_b200_rmsnorm_workspace_bytes": (_sz, [_i64, _i64]),
    "cacti_b200_rmsnorm_fwd": (_int, [_p, _p, _p, _f32, _i64, _i64, _int, _st]),
    "cacti_b200_add_rmsnorm_fwd": (_int, [_p, _p, _p, _p, _p, _f32, _i64, _i64, _int, _st]),
    "cacti_b200_rmsnorm_bwd": (_int, [_p, _p, _p, _p, _p, _f32, _i64, _i64, _int, _int, _int, _int, _p, _sz, _st]),
    "cacti_b200_rmsnorm_fwd_bwd": (_int, [_p, _p, _p, _p, _p, _p, _f32, _i64, _i64, _int, _int, _int, _int, _p, _sz, _st]),
    "cacti_b200_rmsnorm_fwd_bwd_noalloc": (_int, [_p, _p, _p, _p, _p, _p, _f32, _i64, _i64, _int, _int, _int, _int, _st]),
    "cacti_b200_softmax_fwd": (_int, [_p, _p, _i64, _i64, _int, _i64, _i64, _i64, _int, _st]),
    "cacti_b200_softmax_bwd": (_int, [_p, _p, _p, _i64, _i64, _int, _i64, _i64, _i64, _int, _int, _st]),
    "cacti_b200_softmax_fwd_bwd": (_int, [_p, _p, _p, _p, _i64, _i64, _int, _i64, _i64, _i64, _int, _int, _st]),
    "cacti_b200_rope_tables": (_int, [_p, _p, _i64, _i64, _f32, _int, _st]),
    "cacti_b200_rope_fwd": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _int, _st]),
    "cacti_b200_rope_fwd_pitched": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _int, _st]),
    "cacti_b200_rope_bwd": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _int, _int, _st]),
    "cacti_b200_rope_fwd_bwd": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _int, _int, _st]),
    "cacti_b200_swiglu_fwd": (_int, [_p, _p, _p, _i64, _int, _st]),
    "cacti_b200_swiglu_bwd": (_int, [_p, _p, _p, _p, _p, _i64, _int, _int, _int, _st]),
    "cacti_b200_swiglu_fwd_bwd": (_int, [_p, _p, _p, _p, _p, _p, _i64, _int, _int, _int, _st]),
    "cacti_b200_softmax_nll_workspace_bytes": (_sz, [_i64]),
    "cacti_b200_softmax_nll_fwd_bwd": (_int, [_p, _p, _p, _p, _p, _int, _p, _f32, _i64, _i64, _int, _int, _p, _p, _sz, _st]),
    "cacti_b200_gather_rows": (_int, [_p, _p, _p, _int, _i64, _i64, _i64, _int, _p, _st]),
    "cacti_b200_scatter_add_rows_workspace_bytes": (_sz, [_i64, _i64]),
    "cacti_b200_scatter_add_rows": (_int, [_p, _p, _p, _int, _i64, _i64, _i64, _int, _int, _p, _sz, _p, _st]),
    "cacti_b200_accumulate": (_int, [_p, _p, _i64, _int, _st]),
    "cacti_b200_add": (_int, [_p, _p, _p, _i64, _int, _st]),
    "cacti_b200_adamw32_step": (_int, [_p, _p, _p, _p, _p, _i64, _int, _int, _f32, _f32, _f32, _f32, _f32, _f32, _int, _st]),
    "cacti_b200_gemm_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64, _i64]),
    "cacti_b200_gemm": (_int, [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _int, _int, C.POINTER(_f32),
                               C.POINTER(_f32), _int, _p, _sz, _st]),
    "cacti_b200_gemm_strided_batched": (_int, [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _int, _int,
                                               C.POINTER(_f32), C.POINTER(_f32), _i64, _i64, _i64, _i64, _i64, _i64,
                                               _i64, _i64, _int, _p, _sz, _st]),
    "cacti_b200_block_pad": (_int, [_p, _p, _i64, _i64, _i64, _i64, _i64, _int, _st]),
    "cacti_b200_attention_fwd": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _f32, _int, _st]),
    "cacti_b200_attention_bwd": (_int, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _f32, _int, _st]),
    "cacti_b200_attention_bwd_prep": (_int, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _f32, _int, _st]),
    "cacti_b200_gemm_strided_batched_tri": (_int, [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _int, _int,
                                                   C.POINTER(_f32), C.POINTER(_f32), _i64, _i64, _i64, _i64, _i64, _i64,
                                                   _i64, _i64, _int, _i64, _int, _int, _p, _sz, _st]),
}

TRI_NONE, TRI_C_LOWER, TRI_A_LOWER, TRI_A_UPPER = 0, 1, 2, 3
OPERAND_A_PADDED, OPERAND_B_PADDED = 1, 2

_lib = None


def header_functions(path: str = HEADER):
    """Names of all functions declared in the public header."""
    src = open(path).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(cacti_b200_[a-z0-9_]+)\s*\(", src)))


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OSError(f"{LIB_PATH} not found: build it with `python -m cacti_b200.build` (no fallback exists)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)          # AttributeError if the symbol is missing
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


class CactiB200Error(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        msg = lib().cacti_b200_error_string(code).decode()
        extra = f" (cudaError {lib().cacti_b200_last_cuda_error()})" if code == ERR_LAUNCH else ""
        super().__init__(f"{where}: error {code}: {msg}{extra}")


def check(code: int, where: str) -> None:
    if code != OK:
        raise CactiB200Error(code, where)
