"""Robustness of the boundary on the device: a bounded wait that runs out, and two GPUs driven from one process."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(__file__))
import oracle as O  # noqa: E402
import bolt_b200 as B  # noqa: E402
from bolt_b200 import synth  # noqa: E402
from util import dev_zeros, dptr, to_dev, to_host  # noqa: E402

pytestmark = pytest.mark.gpu


def small_gemm(m=256, k=512, n=384, seed=5):
    """packed-weight GEMM with int32 output through the C ABI on the current device -> (got, expected)"""
    A, W = synth.u8(seed, (m, k)), synth.s8(seed + 1, (k, n))
    bdesc = B.tensor2df(B.DT_I8, B.DF_NORMAL, k, n)
    nbytes, rhs = B.matrix_matrix_multiply_transform_rhs_bytes(bdesc)
    d_a, d_w, d_pack = to_dev(A), to_dev(W), dev_zeros(nbytes)
    pdesc = B.matrix_matrix_multiply_transform_rhs(bdesc, dptr(d_w), dptr(d_pack))
    adesc = B.tensor2df(B.DT_U8_Q, B.DF_NORMAL, m, k)
    tb = B.matrix_matrix_multiply_tmp_bytes(adesc, pdesc)
    d_tmp = dev_zeros(tb)
    d_tmp[: 4 * n] = d_pack[rhs: rhs + 4 * n]
    d_c = dev_zeros(4 * m * n)
    B.matrix_matrix_multiply(adesc, dptr(d_a), pdesc, dptr(d_pack), tb, dptr(d_tmp), B.tensor2df(B.DT_I32, B.DF_NORMAL, m, n), dptr(d_c), None)
    code = B.lib().bolt_b200_synchronize()
    return code, to_host(d_c, np.int32, m * n).reshape(m, n), O.port_gemm(A, W, O.port_offsetc(W), None)


def test_a_wait_that_runs_out_is_reported_and_the_library_keeps_working():
    """Every barrier wait in the kernels is bounded.  The self-test entry waits, with a limit of a million cycles
    (half a millisecond), on a barrier nobody arrives on: the kernel returns, the status word says 21,
    synchronize reports it once, and the next GEMM is bit-exact."""
    lib = B.lib()
    B.CHECK_STATUS(lib.bolt_b200_synchronize(), "clean start")
    B.CHECK_STATUS(lib.bolt_b200_selftest_wait_limit(1000000), "launch")
    assert lib.bolt_b200_synchronize() == B.UNKNOWN
    assert lib.bolt_b200_device_status() == 0          # cleared by the report
    code, got, ref = small_gemm()
    assert code == B.SUCCESS and got.tobytes() == ref.tobytes()
    # and the raw status word, read without synchronize
    B.CHECK_STATUS(lib.bolt_b200_selftest_wait_limit(1000), "launch")
    import torch
    torch.cuda.synchronize()
    assert lib.bolt_b200_device_status() == 21
    assert lib.bolt_b200_synchronize() == B.SUCCESS
    assert lib.bolt_b200_selftest_wait_limit(0) == B.NOT_MATCH


def test_two_devices_from_one_process():
    """Kernel attributes (the opt-in to more than 48 KB of shared memory) are per device: after work on device 0,
    the same process switches to device 1 and back.  Also: a pointer that lives on the other GPU is refused."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs in one box")
    lib = B.lib()
    try:
        for dev in (0, 1, 0, 1):
            torch.cuda.set_device(dev)
            B.CHECK_STATUS(lib.bolt_b200_set_device(dev))
            code, got, ref = small_gemm(seed=7 + dev)
            assert code == B.SUCCESS and got.tobytes() == ref.tobytes(), dev
            assert lib.bolt_b200_last_gemm_used_tensor_cores() == 1
        # operands on device 0 while the library is on device 1
        torch.cuda.set_device(0)
        a0 = dev_zeros(256 * 512)
        torch.cuda.set_device(1)
        B.CHECK_STATUS(lib.bolt_b200_set_device(1))
        m, k, n = 256, 512, 384
        bdesc = B.tensor2df(B.DT_I8, B.DF_NORMAL, k, n)
        nbytes, rhs = B.matrix_matrix_multiply_transform_rhs_bytes(bdesc)
        d_w, d_pack = dev_zeros(k * n), dev_zeros(nbytes)
        pdesc = B.matrix_matrix_multiply_transform_rhs(bdesc, dptr(d_w), dptr(d_pack))
        adesc = B.tensor2df(B.DT_U8_Q, B.DF_NORMAL, m, k)
        tb = B.matrix_matrix_multiply_tmp_bytes(adesc, pdesc)
        d_tmp, d_c = dev_zeros(tb), dev_zeros(4 * m * n)
        with pytest.raises(B.BoltError):
            B.matrix_matrix_multiply(adesc, dptr(a0), pdesc, dptr(d_pack), tb, dptr(d_tmp), B.tensor2df(B.DT_I32, B.DF_NORMAL, m, n), dptr(d_c), None)
    finally:
        torch.cuda.set_device(0)
        lib.bolt_b200_set_device(0)
