"""GPU parity of quantize / requantize / dequantize / bias folding against the golden fixtures
(outputs of the reference) and the oracle, through the C ABI."""
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
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def same_bits(a, b):
    return a.shape == b.shape and a.tobytes() == b.tobytes()


def quant_gpu(src, sdt, qdt, scale, mode=0, host=False):
    n = src.size
    npq = np.uint8 if qdt == B.DT_U8_Q else np.int8
    sc = list(scale)
    if host:
        q = np.zeros(n, npq)
        B.quantize(B.tensor1d(sdt, n), hptr(src), B.tensor1d(qdt, n), hptr(q), sc, mode)
        return q, sc
    d, dq = to_dev(src), dev_zeros(n)
    B.quantize(B.tensor1d(sdt, n), dptr(d), B.tensor1d(qdt, n), dptr(dq), sc, mode)
    return to_host(dq, npq, n), sc


def test_quantize_golden():
    g = np.load(os.path.join(GOLD, "quantize.npz"))
    for i, n in enumerate(cases.QUANT_SIZES):
        x, a, u, b, off = cases.quant_inputs(i)
        for host in (False, True):
            for name, qdt in (("u8", B.DT_U8_Q), ("i8", B.DT_I8)):
                q, s = quant_gpu(x, B.DT_F32, qdt, [-1.0], host=host)
                assert same_bits(q, g["q%d_f32_%s" % (i, name)])
                assert np.float32(s[0]) == g["q%d_f32_%s_scale" % (i, name)][0]
                q, s = quant_gpu(a, B.DT_I32, qdt, [-1.0, 0.37], host=host)
                assert same_bits(q, g["q%d_i32_%s" % (i, name)])
                assert same_bits(np.array(s, np.float32), g["q%d_i32_%s_scale" % (i, name)])
                q, s = quant_gpu(a, B.DT_I32, qdt, [2.0, 0.37], host=host)
                assert same_bits(q, g["q%d_i32s_%s" % (i, name)])
            q, _ = quant_gpu(u, B.DT_U8_Q, B.DT_I8, [0.0], host=host)
            assert same_bits(q, g["q%d_u8i8" % i])
        # dequantize
        for src, sdt, key in ((a, B.DT_I32, "dq_i32"), (u, B.DT_U8_Q, "dq_u8")):
            d, out = to_dev(src), dev_zeros(4 * n)
            B.dequantize(B.tensor1d(sdt, n), dptr(d), 0.37, B.tensor1d(B.DT_F32, n), dptr(out))
            assert same_bits(to_host(out, np.float32, n), g["q%d_%s" % (i, key)])
        # bias folding
        lib = B.lib()
        db, doff, dout = to_dev(b), to_dev(off), dev_zeros(4 * n)
        sc = (C.c_float * 1)(3.0)
        bd, fd = B.tensor1d(B.DT_F32, n), B.tensor2df(B.DT_I8, B.DF_NKNxKx, n, n)
        B.CHECK_STATUS(lib.quantize_bias_offsetC_cuda_b200(dptr(db), C.byref(bd), B.DT_I32, dptr(doff), C.byref(fd), sc, dptr(dout)))
        assert same_bits(to_host(dout, np.int32, n), g["q%d_biasoff" % i])


def test_quantize_modes_and_edges_vs_oracle():
    for n in (1, 31, 1000, 70001):
        for std in (1.0, 0.02, 50.0):
            x = synth.normal(n + 3, (n,), std)
            if n > 31:
                x[5] = 0.0
                x[7] = -np.abs(x).max() * 2      # the maximum is a negative value
            for name, qdt, npq in (("u8", B.DT_U8_Q, np.uint8), ("i8", B.DT_I8, np.int8)):
                for sc0, mode in ((-1.0, 0), (0.5, 0), (3.0, 1), (1e9, 0), (1e9, 1)):
                    q, s = quant_gpu(x, B.DT_F32, qdt, [sc0], mode)
                    qp, sp = np.zeros(n, npq), np.array([sc0], np.float32)
                    fn = O.port.oracle_quantize_f32_u8 if name == "u8" else O.port.oracle_quantize_f32_i8
                    fn(O.ptr(x), n, O.ptr(qp), O.ptr(sp), mode)
                    assert same_bits(q, qp) and np.float32(s[0]) == sp[0], (n, std, name, sc0, mode)
    z = np.zeros(100, np.float32)
    q, s = quant_gpu(z, B.DT_F32, B.DT_U8_Q, [-1.0])
    assert s[0] == 1.0 and np.all(q == 128)      # absmax 0 -> scale 1 (quantize.cpp:63-65)
    q, s = quant_gpu(np.zeros(0, np.float32), B.DT_F32, B.DT_U8_Q, [-1.0])
    assert q.size == 0


def test_requantize_matches_conv_usage():
    """convolution_direct.cpp:2798-2806: ReLU'd int32 -> U8_Q with a dynamic scale; scale[0] comes back."""
    n = 64 * 56 * 56
    a = np.maximum(synth.integers(61, (n,), -30000, 90000), 0).astype(np.int32)
    q, s = quant_gpu(a, B.DT_I32, B.DT_U8_Q, [-1.0, 0.0123])
    qp, sp = np.zeros(n, np.uint8), np.array([-1.0, 0.0123], np.float32)
    O.port.oracle_quantize_i32_u8(O.ptr(a), n, O.ptr(qp), O.ptr(sp))
    assert same_bits(q, qp) and same_bits(np.array(s, np.float32), sp)


def test_device_scale_pipeline_matches_host_scale():
    """Extension: absmax scale left on the device + quantize reading it == the host-scale path."""
    n = 4096 * 768
    x = synth.normal(71, (n,))
    lib = B.lib()
    dx, dq, ds = to_dev(x), dev_zeros(n), dev_zeros(16)
    B.CHECK_STATUS(lib.bolt_b200_absmax_scale_f32(dptr(dx), n, dptr(ds)))
    B.CHECK_STATUS(lib.bolt_b200_quantize_f32_u8_dev(dptr(dx), n, dptr(dq), dptr(ds)))
    q, s = quant_gpu(x, B.DT_F32, B.DT_U8_Q, [-1.0])
    assert to_host(ds, np.float32, 1)[0] == np.float32(s[0])
    assert same_bits(to_host(dq, np.uint8, n), q)
