"""What a kernel does when one of its bounded waits runs out.

No product kernel can be made to time out without breaking it, so the path is exercised by the library's own
self-test kernel: its threads wait, with a short poll limit, on a barrier that nothing arms (nothing faults, nothing
spins without a limit), give up after slightly different numbers of polls, agree on that at their group barrier and
leave together, releasing the tensor memory they hold.  The host sees the code in the device error word and the
context stays usable: the next matmul (which needs all 512 tensor-memory columns of an SM) runs and is correct.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from cacti_b200 import capi, ops
from oracle import ref_chain as R
from tests.gpu_util import dev, host
from tests.tolerances import assert_close

pytestmark = pytest.mark.gpu


def _device_error():
    err = C.c_uint(99)
    assert capi.lib().cacti_b200_device_error(C.byref(err)) == capi.OK
    return err.value


def test_bounded_wait_runs_out_and_the_context_survives(cuda):
    L = capi.lib()
    torch.cuda.synchronize()
    assert _device_error() == 0
    out = torch.zeros(3, dtype=torch.int32, device=cuda)
    for polls in (1, 64):
        out.zero_()
        assert L.cacti_b200_selftest_bounded_wait(out.data_ptr(), polls, torch.cuda.current_stream().cuda_stream) == capi.OK
        assert out.cpu().tolist() == [1, 1, 1]          # reached its end; both row groups left as one
        assert _device_error() == 5                     # recorded ...
        assert _device_error() == 0                     # ... and cleared by the read
    # 148 CTAs of it at once would have taken every SM's tensor memory had any been leaked
    for _ in range(4):
        assert L.cacti_b200_selftest_bounded_wait(out.data_ptr(), 8, torch.cuda.current_stream().cuda_stream) == capi.OK
    assert _device_error() == 5
    a, b = R.normal(1, (512, 256), np.float16), R.normal(2, (768, 256), np.float16, 0.1)
    c = ops.gemm(dev(a), dev(b), False, True)
    assert_close(host(c), R.ref_gemm(a, b, False, True), "float16", "matmul after a timed-out kernel", floor_frac=1.0)
    assert _device_error() == 0


def test_selftest_rejects_bad_arguments(cuda):
    L = capi.lib()
    out = torch.zeros(3, dtype=torch.int32, device=cuda)
    assert L.cacti_b200_selftest_bounded_wait(0, 8, None) == capi.ERR_INVALID_VALUE
    assert L.cacti_b200_selftest_bounded_wait(out.data_ptr(), 0, None) == capi.ERR_INVALID_VALUE
    assert L.cacti_b200_selftest_bounded_wait(out.data_ptr(), 1 << 20, None) == capi.ERR_INVALID_VALUE
