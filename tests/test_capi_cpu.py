"""CPU checks of the C-ABI library: it loads, exports every declared symbol, and validates arguments
before touching the device (none of these calls launches anything)."""
import ctypes as C
import os
import re

from cacti_b200 import capi


def test_library_exports_every_declared_symbol():
    L = capi.lib()
    declared = capi.header_functions()
    assert len(declared) >= 25
    for name in declared:
        assert hasattr(L, name), name
    assert set(declared) == set(capi.SIGNATURES), set(declared) ^ set(capi.SIGNATURES)
    assert L.cacti_b200_version() >= 100


def test_header_has_no_torch_or_cxx_types():
    src = open(capi.HEADER).read()
    assert "torch" not in src and "at::" not in src and "std::" not in src
    assert 'extern "C"' in src


def test_error_strings():
    L = capi.lib()
    seen = {L.cacti_b200_error_string(c).decode() for c in range(8)}
    assert len(seen) == 8 and "ok" in seen


def test_argument_validation_returns_codes_without_a_device():
    L = capi.lib()
    P = 0x1000   # non-null, never dereferenced: every call below fails validation first
    assert L.cacti_b200_rmsnorm_fwd(P, P, P, 1e-6, -1, 8, capi.R_32F, None) == capi.ERR_INVALID_VALUE
    assert L.cacti_b200_rmsnorm_fwd(0, P, P, 1e-6, 4, 8, capi.R_32F, None) == capi.ERR_INVALID_VALUE
    assert L.cacti_b200_rmsnorm_fwd(P, P, P, 1e-6, 4, 8, 99, None) == capi.ERR_DTYPE
    assert L.cacti_b200_rmsnorm_fwd(P, P, P, 1e-6, 0, 8, capi.R_32F, None) == capi.OK      # empty: no-op
    assert L.cacti_b200_rmsnorm_bwd(P, P, P, P, P, 1e-6, 4, 8, capi.R_16F, capi.R_16F, 0, 0, 0, 0, None) == capi.ERR_WORKSPACE
    assert L.cacti_b200_rmsnorm_bwd(P, P, P, P, P, 1e-6, 4, 8, capi.R_16F, capi.R_16BF, 0, 0, P, 1 << 30, None) == capi.ERR_DTYPE
    assert L.cacti_b200_rmsnorm_bwd(P, P, P, P, P, 1e-6, 4, 8, capi.R_16F, capi.R_16F, 2, 0, P, 1 << 30, None) == capi.ERR_INVALID_VALUE
    assert L.cacti_b200_softmax_fwd(P, P, 4, 8, 7, 1, 1, 0, capi.R_16F, None) == capi.ERR_INVALID_VALUE
    assert L.cacti_b200_softmax_fwd(P, P, 4, 8, capi.MASK_CAUSAL, 0, 8, 0, capi.R_16F, None) == capi.ERR_INVALID_VALUE
    assert L.cacti_b200_softmax_fwd(P, P, 4, 0, capi.MASK_NONE, 1, 1, 0, capi.R_16F, None) == capi.OK
    assert L.cacti_b200_rope_fwd(P, P, P, P, 4, 2, 7, 16, 0, capi.R_16F, None) == capi.ERR_SHAPE    # odd head_dim
    assert L.cacti_b200_rope_fwd(P, P, P, P, 4, 2, 8, 0, 0, capi.R_16F, None) == capi.ERR_INVALID_VALUE
    assert L.cacti_b200_swiglu_fwd(P, P, 0, 16, capi.R_16F, None) == capi.ERR_INVALID_VALUE
    assert L.cacti_b200_swiglu_fwd(P, P, P, 16, 3, None) == capi.ERR_DTYPE
    assert L.cacti_b200_softmax_nll_fwd_bwd(0, 0, P, P, P, 5, 0, 1.0, 4, 8, capi.R_16F, 0, 0, 0, 0, None) == capi.ERR_DTYPE
    assert L.cacti_b200_softmax_nll_fwd_bwd(P, 0, P, P, P, capi.R_32I, 0, 1.0, 4, 8, capi.R_16F, 0, 0, 0, 0, None) == capi.ERR_WORKSPACE
    assert L.cacti_b200_gather_rows(P, P, P, capi.R_32F, 4, 8, 8, capi.R_16F, 0, None) == capi.ERR_DTYPE
    assert L.cacti_b200_scatter_add_rows(P, P, P, capi.R_32I, 4, 8, 8, capi.R_16F, 0, 0, 0, 0, None) == capi.ERR_WORKSPACE
    assert L.cacti_b200_accumulate(P, 0, 4, capi.R_16F, None) == capi.ERR_INVALID_VALUE
    assert L.cacti_b200_tune(b"no_such_knob", 1) == capi.ERR_INVALID_VALUE
    assert L.cacti_b200_tune(b"softmax_threads", 100) == capi.ERR_INVALID_VALUE
    assert L.cacti_b200_tune(b"softmax_threads", 256) == capi.OK


def test_workspace_queries():
    L = capi.lib()
    assert L.cacti_b200_rmsnorm_workspace_bytes(16384, 3200) >= 148 * 3200 * 4
    assert L.cacti_b200_softmax_nll_workspace_bytes(8192) >= 8192 * 4
    assert L.cacti_b200_scatter_add_rows_workspace_bytes(16384, 32000) >= (32001 + 32000 + 16384) * 4


def test_product_does_not_touch_the_oracle():
    """Nothing under cacti_b200/ may import, read or link the oracle."""
    root = os.path.join(os.path.dirname(capi.HERE), "cacti_b200")
    for dp, _, files in os.walk(root):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                src = open(os.path.join(dp, f), errors="ignore").read()
                assert not re.search(r"\boracle\b", src), os.path.join(dp, f)
