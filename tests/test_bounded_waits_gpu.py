"""Device-side waits are bounded: a wait on a flag that nothing sets runs out of its poll budget, the kernel returns, the
status word carries the timeout code and the CUDA context stays usable (no trap, no hang)."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_flag_wait_times_out_and_reports():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from pear_b200.ops import lib as kl
    lib = kl.lib()
    flags = torch.zeros(32 * 8, dtype=torch.int32, device="cuda")  # [slot][source rank], nobody ever writes it
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # wait for 4 "ranks" to reach epoch 1 in slot 3 with a budget of 1000 polls (~0.1 ms)
    assert lib.pear_symm_wait(ctypes.c_void_p(flags.data_ptr()), 4, 3, 1, 1000, ctypes.c_void_p(status.data_ptr()), stream) == 0
    torch.cuda.synchronize()
    assert int(status[0]) == 3  # PEAR_ERR_FLAG_TIMEOUT
    # the context is alive: set the flags, wait again with a clean status
    status.zero_()
    flags.view(32, 8)[3, :4] = 1
    assert lib.pear_symm_wait(ctypes.c_void_p(flags.data_ptr()), 4, 3, 1, 1000, ctypes.c_void_p(status.data_ptr()), stream) == 0
    torch.cuda.synchronize()
    assert int(status[0]) == 0 and float((torch.ones(8, device="cuda") * 2).sum()) == 16.0
