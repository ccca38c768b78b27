"""ctypes binding of libcacti_b200_host.so (the C++ host shim's flat test ABI)."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "..", "lib", "libcacti_b200_host.so")
_lib = None
_i64, _sz, _p = C.c_int64, C.c_size_t, C.c_void_p


def lib():
    global _lib
    if _lib is None:
        from .. import capi
        capi.lib()                                   # the kernel library must load first; no fallback
        L = C.CDLL(LIB_PATH)
        sig = {
            "cbh_ctx_create": (_p, [C.c_int, _sz, _sz, C.c_int]), "cbh_ctx_destroy": (None, [_p]),
            "cbh_cell_new": (_i64, [_p, _sz, C.c_int]), "cbh_cell_put": (C.c_int, [_p, _i64, _p, _sz]),
            "cbh_cell_get": (C.c_int, [_p, _i64, _p, _sz]), "cbh_cell_unlive": (C.c_int, [_p, _i64]),
            "cbh_cell_resident": (C.c_int, [_p, _i64]), "cbh_pread": (C.c_uint64, [_p, _i64]),
            "cbh_pwrite": (C.c_uint64, [_p, _i64]), "cbh_pin": (None, [_p, _i64]), "cbh_unpin": (None, [_p, _i64]),
            "cbh_in_use": (_sz, [_p]), "cbh_sync": (C.c_int, [_p]), "cbh_stats": (None, [_p, C.POINTER(C.c_long)]),
            "cbh_thunk_rmsnorm_fwd": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, C.c_float, _i64, _i64, C.c_int]),
            "cbh_thunk_add_rmsnorm_fwd": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _i64, _i64, C.c_float, _i64, _i64, C.c_int]),
            "cbh_thunk_softmax_fwd": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _i64, _i64, _i64, C.c_int]),
            "cbh_thunk_softmax_bwd": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _i64, _i64, _i64, _i64, C.c_int]),
            "cbh_thunk_add": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _i64, C.c_int]),
            "cbh_thunk_matmul": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _i64, _i64, _i64, C.c_int, C.c_int, C.c_float, C.c_int]),
            "cbh_cell_free": (C.c_int, [_p, _i64]), "cbh_soft_limit": (_sz, [_p]), "cbh_stream": (_p, [_p]),
            "cbh_parse_vmem_soft_limit": (_sz, [C.c_char_p, _sz, _sz]), "cbh_stats_bytes": (None, [_p, C.POINTER(C.c_longlong)]),
            "cbh_arena_create": (_p, [_sz]), "cbh_arena_destroy": (None, [_p]), "cbh_arena_alloc": (_sz, [_p, _sz, C.c_int]),
            "cbh_arena_free": (None, [_p, _sz]), "cbh_arena_front": (_sz, [_p]), "cbh_arena_back": (_sz, [_p]),
            "cbh_arena_in_use": (_sz, [_p]),
            "cbh_thunk_rmsnorm_bwd": (C.c_int, [_p, C.c_int, C.c_int, _i64, _i64, _i64, _i64, _i64, C.c_float, _i64, _i64, C.c_int, C.c_int]),
            "cbh_thunk_rope_fwd": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, C.c_int]),
            "cbh_thunk_rope_bwd": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, C.c_int]),
            "cbh_thunk_swiglu_fwd": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _i64, C.c_int]),
            "cbh_thunk_swiglu_bwd": (C.c_int, [_p, C.c_int, C.c_int, _i64, _i64, _i64, _i64, _i64, _i64, C.c_int]),
            "cbh_thunk_softmax_nll": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _i64, C.c_int, C.c_float, _i64, _i64, C.c_int, _i64]),
            "cbh_thunk_gather_rows": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, C.c_int, _i64, _i64, _i64, C.c_int, _i64]),
            "cbh_thunk_scatter_add_rows": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, C.c_int, _i64, _i64, _i64, C.c_int, _i64]),
            "cbh_thunk_block_pad": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _i64, _i64, _i64, _i64, C.c_int]),
            "cbh_thunk_block_matmul": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, C.c_int, C.c_int,
                                                 C.c_float, C.c_int, _i64, C.c_int, C.c_int]),
            "cbh_thunk_attention_fwd": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, C.c_float, C.c_int]),
            "cbh_thunk_attention_bwd_prep": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                                                       _i64, C.c_float, C.c_int]),
            "cbh_thunk_attention_bwd": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                                                  _i64, C.c_float, C.c_int]),
            "cbh_thunk_adamw32_step": (C.c_int, [_p, C.c_int, _i64, _i64, _i64, _i64, _i64, _i64, C.c_int, C.c_int, C.c_float, C.c_float,
                                                 C.c_float, C.c_float, C.c_float, C.c_float, C.c_int]),
        }
        for n, (r, a) in sig.items():
            f = getattr(L, n)
            f.restype, f.argtypes = r, a
        _lib = L
    return _lib


APPLY, ACCUMULATE, INITIALIZE = 0, 1, 2
NO_CELL = -1          # an optional cell argument that is not given


class Ctx:
    """One shim context: an arena of `arena_bytes` with a soft limit, on the CUDA or the fake backend."""

    def __init__(self, cuda, arena_bytes, soft_limit=0, sync_each_thunk=False):
        self.L = lib()
        self.h = self.L.cbh_ctx_create(int(cuda), arena_bytes, soft_limit, int(sync_each_thunk))

    def close(self):
        if self.h:
            self.L.cbh_ctx_destroy(self.h)
            self.h = None

    def cell(self, array=None, nbytes=None, stable=False):
        n = array.nbytes if array is not None else nbytes
        c = self.L.cbh_cell_new(self.h, n, int(stable))
        if array is not None:
            assert self.L.cbh_cell_put(self.h, c, array.ctypes.data_as(C.c_void_p), n) == 0
        return c

    def get(self, c, like):
        import numpy as np
        out = np.empty_like(like)
        rc = self.L.cbh_cell_get(self.h, c, out.ctypes.data_as(C.c_void_p), out.nbytes)
        if rc:
            raise RuntimeError("cell has no value")
        return out

    def free(self, c):
        assert self.L.cbh_cell_free(self.h, c) == 0

    def stats(self):
        a = (C.c_long * 6)()
        self.L.cbh_stats(self.h, a)
        b = (C.c_longlong * 3)()
        self.L.cbh_stats_bytes(self.h, b)
        return dict(spills=a[0], drops=a[1], reloads=a[2], oom_retries=a[3], hard_oom=a[4], spill_copies=a[5],
                    spill_bytes=b[0], reload_bytes=b[1], peak_in_use=b[2])
