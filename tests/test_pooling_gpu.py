"""GPU parity of the u8 pooling (maximum and the reference's integer mean) through the C ABI: bit for bit against
the reference's outputs (golden fixtures) and, at a ResNet-sized tensor, the oracle."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(__file__))
sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import cases  # noqa: E402
import oracle as O  # noqa: E402
import bolt_b200 as B  # noqa: E402
from bolt_b200 import synth  # noqa: E402
from util import dev_zeros, dptr, hptr, to_dev, to_host  # noqa: E402

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def pool_gpu(case, x, host=False):
    n, c, ih, iw, k, s, p, mean, cip, ceil = case
    oh, ow = cases.pool_out_hw(case)
    in_desc = B.tensor4df(B.DT_U8_Q, B.DF_NCHWC16, n, c, ih, iw)
    out_desc = B.tensor4df(B.DT_U8_Q, B.DF_NCHWC16, n, c, oh, ow)
    pp = B.pooling_param(k, s, p, bool(mean), bool(cip))
    sc = [3.5, -1.0]
    if host:
        y = np.zeros(n * c * oh * ow, np.uint8)
        B.pooling(in_desc, hptr(x), pp, sc, out_desc, hptr(y))
        return y, sc
    dx, dy = to_dev(x), dev_zeros(n * c * oh * ow)
    B.pooling(in_desc, dptr(dx), pp, sc, out_desc, dptr(dy))
    B.CHECK_STATUS(B.lib().bolt_b200_synchronize(), "synchronize")
    return to_host(dy, np.uint8, n * c * oh * ow), sc


@pytest.mark.parametrize("host", [False, True])
def test_pooling_golden(host):
    g = np.load(os.path.join(GOLD, "pooling.npz"))
    for i, case in enumerate(cases.POOL_CASES):
        y, sc = pool_gpu(case, cases.pool_input(i), host)
        assert y.tobytes() == g["p%d" % i].tobytes(), (case, host)
        assert np.array(sc, np.float32).tobytes() == g["p%d_scale" % i].tobytes(), case


def test_pooling_resnet_stem_size_vs_oracle():
    """3 x 3 stride 2 pad 1 maximum on 64 x 112 x 112 (the pooling after ResNet's stem), batch 8; the global 7 x 7 mean"""
    for case in ((8, 64, 112, 112, 3, 2, 1, 0, 0, 0), (8, 2048, 7, 7, 7, 1, 0, 1, 0, 0)):
        n, c, ih, iw, k, s, p, mean, cip, ceil = case
        oh, ow = cases.pool_out_hw(case)
        x = synth.relu_u8(77, (n * c * ih * iw,))
        y, sc = pool_gpu(case, x)
        ref = np.zeros(n * c * oh * ow, np.uint8)
        rs = np.array([3.5, -1.0], np.float32)
        assert O.port.oracle_pooling_u8(n, c, ih, iw, oh, ow, k, k, s, s, p, p, mean, cip, O.ptr(x), O.ptr(ref), O.ptr(rs)) == 0
        assert y.tobytes() == ref.tobytes() and np.array(sc, np.float32).tobytes() == rs.tobytes(), case


def test_pooling_argument_checks():
    lib = B.lib()
    import ctypes as C
    d = dev_zeros(16 * 8 * 8)
    in_desc = B.tensor4df(B.DT_U8_Q, B.DF_NCHWC16, 1, 16, 8, 8)
    out_desc = B.tensor4df(B.DT_U8_Q, B.DF_NCHWC16, 1, 16, 4, 4)
    pp = B.pooling_param(2, 2, 2)            # padding not smaller than the kernel
    assert lib.pooling_cuda_b200(C.byref(in_desc), dptr(d), C.byref(pp), None, C.byref(out_desc), dptr(d)) == B.NOT_SUPPORTED
    pp = B.pooling_param(2, 2, 0)
    bad = B.tensor4df(B.DT_U8_Q, B.DF_NCHWC16, 1, 16, 9, 9)   # windows that start outside the image
    assert lib.pooling_cuda_b200(C.byref(in_desc), dptr(d), C.byref(pp), None, C.byref(bad), dptr(d)) == B.NOT_MATCH
    f32 = B.tensor4df(B.DT_F32, B.DF_NCHWC16, 1, 16, 8, 8)
    assert lib.pooling_cuda_b200(C.byref(f32), dptr(d), C.byref(pp), None, C.byref(out_desc), dptr(d)) == B.NOT_MATCH
