"""The allocation-free quantize entry point (bolt_b200_quantize_f32_u8_noalloc) against the regular
device-scale path, through the C ABI.

Who needs it: a caller that may not allocate device memory at call time -- a server whose pool
allocator took the whole GPU at start-up, a host that bans allocation on its serving path.  The
entry point keeps its reduction scratch in a fixed array inside the library, shared by all calls,
so the checks run two calls back to back (the second with a different, smaller tensor: whatever
the first call left in the array must not leak into it).

Collected last on purpose (file name): a failure here cannot hide the other tests from a run that
stops at the first failure.  It passes alone in a fresh process and after the rest of the suite.
"""
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


def regular_path(x):
    """existing entry points: scale left on the device, then quantize reading it"""
    lib = B.lib()
    n = x.size
    dx, dq, ds = to_dev(x), dev_zeros(n), dev_zeros(16)
    B.CHECK_STATUS(lib.bolt_b200_absmax_scale_f32(dptr(dx), n, dptr(ds)))
    B.CHECK_STATUS(lib.bolt_b200_quantize_f32_u8_dev(dptr(dx), n, dptr(dq), dptr(ds)))
    return to_host(dq, np.uint8, n), to_host(ds, np.float32, 1)[0]


def noalloc_path(x):
    lib = B.lib()
    n = x.size
    dx, dq, ds = to_dev(x), dev_zeros(n), dev_zeros(16)
    B.CHECK_STATUS(lib.bolt_b200_quantize_f32_u8_noalloc(dptr(dx), n, dptr(dq), dptr(ds)), "quantize_noalloc")
    return to_host(dq, np.uint8, n), to_host(ds, np.float32, 1)[0]


def test_noalloc_matches_regular_path_twice_in_a_row():
    first = synth.normal(901, (4096 * 768 + 13,), 3.0)        # 193 chunks, ragged tail
    second = synth.normal(902, (20000,), 0.05)                # 2 chunks, a much smaller maximum
    for x in (first, second):
        q_new, s_new = noalloc_path(x)
        q_ref, s_ref = regular_path(x)
        assert s_new.tobytes() == s_ref.tobytes()
        assert q_new.tobytes() == q_ref.tobytes()


def test_noalloc_matches_the_cpu_oracle_and_allocates_nothing():
    """Against the scalar restatement of the reference's quantize (dynamic scale = 127 / absmax), and with the
    device's free memory read before and after the second call: the call must not change it."""
    import torch

    lib = B.lib()
    for seed, n, std in ((903, 3 * 1000 * 1000 + 7, 1.5), (904, 70001, 40.0)):
        x = synth.normal(seed, (n,), std)
        q_ref, s_ref = np.zeros(n, np.uint8), np.array([-1.0], np.float32)
        O.port.oracle_quantize_f32_u8(O.ptr(x), n, O.ptr(q_ref), O.ptr(s_ref), 0)
        dx, dq, ds = to_dev(x), dev_zeros(n), dev_zeros(16)
        B.CHECK_STATUS(lib.bolt_b200_quantize_f32_u8_noalloc(dptr(dx), n, dptr(dq), dptr(ds)), "first call")
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        B.CHECK_STATUS(lib.bolt_b200_quantize_f32_u8_noalloc(dptr(dx), n, dptr(dq), dptr(ds)), "second call")
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, (free_before, free_after)
        assert to_host(ds, np.float32, 1).tobytes() == s_ref.tobytes()
        assert to_host(dq, np.uint8, n).tobytes() == q_ref.tobytes()


def test_noalloc_edges():
    lib = B.lib()
    z = np.zeros(1000, np.float32)
    q, s = noalloc_path(z)
    assert s == 1.0 and np.all(q == 128)                       # absmax 0 -> scale 1
    buf = dev_zeros(64)
    too_many = B.NOALLOC_MAX_ELEMENTS + 1
    assert lib.bolt_b200_quantize_f32_u8_noalloc(dptr(buf), too_many, dptr(buf), dptr(buf)) == B.NOT_SUPPORTED
    assert lib.bolt_b200_quantize_f32_u8_noalloc(dptr(buf), 0, dptr(buf), dptr(buf)) == B.NOT_SUPPORTED
    assert lib.bolt_b200_quantize_f32_u8_noalloc(None, 16, dptr(buf), dptr(buf)) == B.NULL_POINTER
