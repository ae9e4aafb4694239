"""GPU parity of the 1-bit convolution (XNOR-Net / DoReFa) through the C ABI: against fixtures made by
the reference's own scalar code (compute/tensor/src/cpu/general/convolution.cpp:141-179,264-285,
compiled by oracle/ref_bnn_shim.cpp; tests/golden/bnn.npz), and on larger shapes against the scalar
restatement of Bolt's ARMv8.2 kernels (oracle_bnn_conv), which test_oracle_pins.py checks against the
same fixtures and against the compiled reference."""
import ctypes as C
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


pack_bits_msb = cases.pack_bits_msb


def bnn_case(seed, n, ic, ih, iw, oc, fh, fw, st, pad, xnor):
    x = synth.normal(seed, (n, ic, ih, iw)).astype(np.float16)
    if not xnor:
        x = (x * np.float16(0.5) + np.float16(0.5)).astype(np.float16)   # DoReFa activations around 0.5
    wf = synth.normal(seed + 1, (oc, ic, fh, fw))
    wbits = pack_bits_msb((wf >= 0).reshape(-1))
    alpha = np.abs(wf).reshape(oc, -1).mean(axis=1).astype(np.float16)      # XNOR-Net scale = mean |W|
    beta = (synth.normal(seed + 2, (oc,), 0.1)).astype(np.float16)
    xin = cases.to_blocked(x.view(np.uint16), 8)
    return xin, wbits, alpha.view(np.uint16), beta.view(np.uint16)


def bnn_gpu(n, ic, ih, iw, oc, fh, fw, st, pad, xnor, xin, wbits, alpha, beta, host=False):
    fdt = B.DT_BIN11 if xnor else B.DT_BIN01
    p = B.conv_param(oc, fh, fw, st, pad)
    in_desc = B.tensor4df(B.DT_F16, B.DF_NCHWC8, n, ic, ih, iw)
    f_desc = B.tensor4df(fdt, B.DF_NCHW, oc, ic, fh, fw)
    oh, ow = (ih + 2 * pad - fh) // st + 1, (iw + 2 * pad - fw) // st + 1
    out_desc = B.tensor4df(B.DT_F16, B.DF_NCHWC8, n, oc, oh, ow)
    alg = B.convolution_infer_forward_algorithm(in_desc, f_desc, out_desc, p, B.DT_F16)
    assert alg == B.CONVOLUTION_ALGORITHM_BNN
    fbytes = B.convolution_transform_filter_bytes(f_desc, p, alg)
    tot = n * oc * oh * ow
    if host:
        ftm = np.zeros(fbytes, np.uint8)
        ftm_desc = B.convolution_transform_filter(f_desc, hptr(wbits), p, alg, hptr(ftm))
        tb = B.convolution_infer_forward_tmp_bytes(in_desc, ftm_desc, out_desc, p, alg)
        tmp, out = np.zeros(tb, np.uint8), np.zeros(tot, np.uint16)
        B.convolution(in_desc, hptr(xin), ftm_desc, hptr(ftm), p, alg, hptr(alpha), hptr(beta), tb, hptr(tmp), out_desc, hptr(out))
        return out
    d_w, d_ftm = to_dev(wbits), dev_zeros(fbytes)
    ftm_desc = B.convolution_transform_filter(f_desc, dptr(d_w), p, alg, dptr(d_ftm))
    assert ftm_desc.df == B.DF_NCHWN16C8
    tb = B.convolution_infer_forward_tmp_bytes(in_desc, ftm_desc, out_desc, p, alg)
    d_x, d_a, d_b, d_tmp, d_out = to_dev(xin), to_dev(alpha), to_dev(beta), dev_zeros(tb), dev_zeros(tot * 2)
    B.convolution(in_desc, dptr(d_x), ftm_desc, dptr(d_ftm), p, alg, dptr(d_a), dptr(d_b), tb, dptr(d_tmp), out_desc, dptr(d_out))
    B.CHECK_STATUS(B.lib().bolt_b200_synchronize(), "synchronize")
    return to_host(d_out, np.uint16, tot)


def bnn_oracle(n, ic, ih, iw, oc, fh, fw, st, pad, xnor, xin, wbits, alpha, beta):
    s = O.BnnShape(n, ic, ih, iw, oc, fh, fw, st, st, pad, pad, pad, pad, int(xnor))
    oh, ow = (ih + 2 * pad - fh) // st + 1, (iw + 2 * pad - fw) // st + 1
    out = np.zeros(n * oc * oh * ow, np.uint16)
    O.port.oracle_bnn_conv(C.byref(s), O.ptr(xin), O.ptr(wbits), O.ptr(alpha), O.ptr(beta), O.ptr(out), None)
    return out


SHAPES = [(1, 8, 5, 5, 8, 3, 3, 1, 1), (2, 32, 7, 6, 32, 3, 3, 1, 1), (1, 64, 9, 9, 72, 3, 3, 2, 1), (2, 40, 6, 6, 16, 1, 1, 1, 0),
          (1, 256, 14, 14, 64, 3, 3, 1, 1), (2, 96, 8, 8, 48, 5, 5, 1, 2)]


@pytest.mark.parametrize("i", range(len(cases.BNN_SHAPES)))
def test_bnn_vs_reference_fixtures(i):
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "bnn.npz"))
    shape = cases.BNN_SHAPES[i]
    for xnor in (0, 1):
        for scaling in (0, 1, 2):
            got = bnn_gpu(*shape, bool(xnor), *cases.bnn_inputs(i, xnor, scaling))
            assert got.tobytes() == g["b%d_%d%d" % (i, xnor, scaling)].tobytes(), (i, xnor, scaling)


@pytest.mark.parametrize("xnor", [True, False])
@pytest.mark.parametrize("shape", SHAPES)
def test_bnn_vs_oracle(shape, xnor):
    data = bnn_case(sum(shape), *shape, xnor)
    got = bnn_gpu(*shape, xnor, *data)
    ref = bnn_oracle(*shape, xnor, *data)
    assert got.tobytes() == ref.tobytes()


def test_bnn_benchmarked_geometry_and_host_pointers():
    """The benchmarked geometry (C 256 -> 256, 28 x 28, 3 x 3, pad 1) at batch 2, both modes."""
    shape = (2, 256, 28, 28, 256, 3, 3, 1, 1)
    for xnor in (True, False):
        data = bnn_case(5, *shape, xnor)
        ref = bnn_oracle(*shape, xnor, *data)
        assert bnn_gpu(*shape, xnor, *data).tobytes() == ref.tobytes()
    small = (1, 32, 7, 6, 32, 3, 3, 1, 1)
    data = bnn_case(6, *small, True)
    assert bnn_gpu(*small, True, *data, host=True).tobytes() == bnn_oracle(*small, True, *data).tobytes()
