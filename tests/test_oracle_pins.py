"""Pins the scalar oracle (oracle/bolt_oracle.c) to the reference.

Two anchors: (1) the golden fixtures under tests/golden/ (outputs of the unmodified reference on
seeded inputs) -- always checked; (2) the compiled reference itself (oracle/_ref), when it is
present and the host has avx512_vnni -- a wider sweep in the style of the reference's own cover
tests (compute/blas_enhance/tests/test_mmm.cpp:165-171, test_mvm.cpp:134-172).
"""
import itertools
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import cases  # noqa: E402
import oracle as O  # noqa: E402
from oracle import ptr  # noqa: E402
from bolt_b200 import synth  # noqa: E402

GOLD = os.path.join(os.path.dirname(__file__), "golden")
needs_ref = pytest.mark.skipif(O.ref is None, reason="compiled reference (oracle/_ref) not available on this host")


def same_bits(a, b):
    return a.shape == b.shape and a.tobytes() == b.tobytes()


# ---------------------------------------------------------------- golden fixtures
def test_golden_gemm():
    g = np.load(os.path.join(GOLD, "gemm.npz"))
    for i in range(len(cases.GEMM_SHAPES)):
        for a_t, b_t in cases.gemm_variants(i):
            A, B, Cin = cases.gemm_inputs(i, a_t, b_t)
            off = O.port_offsetc(B, b_t)
            key = "g%d_%d%d" % (i, a_t, b_t)
            assert same_bits(O.port_gemm(A, B, off, None, Cin, a_t, b_t), g[key + "_s32"]), key
            if a_t == 0:
                assert same_bits(O.port_gemm(A, B, off, cases.GEMM_F32_SCALE, None, 0, b_t), g[key + "_f32"]), key
                assert same_bits(O.port_gemm(A, B, off, cases.GEMM_U8_SCALE, None, 0, b_t), g[key + "_u8"]), key


def test_golden_gemv():
    g = np.load(os.path.join(GOLD, "gemv.npz"))
    for i in range(len(cases.GEMV_SHAPES)):
        for w_t in (0, 1):
            W, x, yin = cases.gemv_inputs(i, w_t)
            off = O.port_offsetc(W, not w_t)
            key = "v%d_%d" % (i, w_t)
            assert same_bits(O.port_gemv(W, x, off, None, yin, w_t), g[key + "_s32"]), key
            assert same_bits(O.port_gemv(W, x, off, cases.GEMM_F32_SCALE, None, w_t), g[key + "_f32"]), key
            assert same_bits(O.port_gemv(W, x, off, cases.GEMM_U8_SCALE, None, w_t), g[key + "_u8"]), key


def test_golden_gemv_row():
    g = np.load(os.path.join(GOLD, "gemv_row.npz"))
    for i in range(len(cases.GEMV_ROW_SHAPES)):
        for m_t in (0, 1):
            Mx, v = cases.gemv_row_inputs(i, m_t)
            key = "r%d_%d" % (i, m_t)
            assert same_bits(O.port_gemv_row(Mx, v, None, m_t), g[key + "_s32"]), key
            assert same_bits(O.port_gemv_row(Mx, v, cases.GEMM_F32_SCALE, m_t), g[key + "_f32"]), key
            assert same_bits(O.port_gemv_row(Mx, v, cases.GEMM_U8_SCALE, m_t), g[key + "_u8"]), key


def port_quant(kind, src, dst_dtype, scale, mode=0):
    n = src.size
    q = np.zeros(n, dst_dtype)
    s = np.array(scale, np.float32)
    fn = {"f32u8": O.port.oracle_quantize_f32_u8, "f32i8": O.port.oracle_quantize_f32_i8,
          "i32u8": O.port.oracle_quantize_i32_u8, "i32i8": O.port.oracle_quantize_i32_i8}[kind]
    if kind.startswith("f32"):
        fn(ptr(src), n, ptr(q), ptr(s), mode)
    else:
        fn(ptr(src), n, ptr(q), ptr(s))
    return q, s


def test_golden_quantize():
    g = np.load(os.path.join(GOLD, "quantize.npz"))
    for i, n in enumerate(cases.QUANT_SIZES):
        x, a, u, b, off = cases.quant_inputs(i)
        for name, dst in (("u8", np.uint8), ("i8", np.int8)):
            q, s = port_quant("f32" + name, x, dst, [-1])
            assert same_bits(q, g["q%d_f32_%s" % (i, name)]) and same_bits(s, g["q%d_f32_%s_scale" % (i, name)])
            q, s = port_quant("i32" + name, a, dst, [-1, 0.37])
            assert same_bits(q, g["q%d_i32_%s" % (i, name)]) and same_bits(s, g["q%d_i32_%s_scale" % (i, name)])
            q, s = port_quant("i32" + name, a, dst, [2.0, 0.37])
            assert same_bits(q, g["q%d_i32s_%s" % (i, name)])
        q = np.zeros(n, np.int8)
        O.port.oracle_u8_to_i8(ptr(u), n, ptr(q))
        assert same_bits(q, g["q%d_u8i8" % i])
        f = np.zeros(n, np.float32)
        O.port.oracle_dequantize_i32_f32(ptr(a), n, 0.37, ptr(f))
        assert same_bits(f, g["q%d_dq_i32" % i])
        O.port.oracle_dequantize_u8_f32(ptr(u), n, 0.37, ptr(f))
        assert same_bits(f, g["q%d_dq_u8" % i])
        r = np.zeros(n, np.int32)
        O.port.oracle_bias_offsetc(ptr(b), ptr(off), n, 3.0, ptr(r))
        assert same_bits(r, g["q%d_biasoff" % i])


def test_golden_conv():
    import ctypes as C
    g = np.load(os.path.join(GOLD, "conv.npz"))
    for i, (n, ic, ih, iw, oc, fh, fw, st, pad) in enumerate(cases.CONV_SHAPES):
        for blk, out_u8, relu in cases.conv_variants(i):
            xin, w, bias = cases.conv_inputs(i, blk)
            s = O.ConvShape(n, ic, ih, iw, oc, fh, fw, st, st, pad, pad, pad, pad, 1, 1, blk, 16, relu, out_u8)
            key = "c%d_%d%d%d" % (i, blk, out_u8, relu)
            out = np.zeros(g[key].size, g[key].dtype)
            sc = np.array(cases.CONV_SCALES, np.float32)
            O.port.oracle_conv_int8(C.byref(s), ptr(xin), ptr(w), ptr(bias), None, ptr(out), ptr(sc), None)
            assert same_bits(out, g[key]) and same_bits(sc, g[key + "_scale"]), key
        for key, out_u8, act, with_elt in cases.conv_extra_variants(i):
            blk = 16 if ic % 16 == 0 else 8
            xin, w, bias = cases.conv_inputs(i, blk)
            key = "c%d_%s" % (i, key)
            elt = cases.conv_eltwise(i, g[key].size) if with_elt else None
            s = O.ConvShape(n, ic, ih, iw, oc, fh, fw, st, st, pad, pad, pad, pad, 1, 1, blk, 16, act, out_u8)
            out = np.zeros(g[key].size, g[key].dtype)
            sc = np.array(cases.CONV_SCALES, np.float32)
            O.port.oracle_conv_int8(C.byref(s), ptr(xin), ptr(w), ptr(bias), ptr(elt), ptr(out), ptr(sc), None)
            assert same_bits(out, g[key]) and same_bits(sc, g[key + "_scale"]), key


def test_golden_bnn():
    """The restatement of the 1-bit convolution against outputs of the reference's own scalar code
    (cpu/general/convolution.cpp:141-179,264-285, compiled by oracle/ref_bnn_shim.cpp): thresholds,
    bit order, padding values, tap sums, scale * sum + bias -- both modes, three kinds of scale / bias."""
    g = np.load(os.path.join(GOLD, "bnn.npz"))
    for i, shape in enumerate(cases.BNN_SHAPES):
        for xnor in (0, 1):
            for scaling in (0, 1, 2):
                got = O.port_bnn(shape, xnor, *cases.bnn_inputs(i, xnor, scaling))
                assert same_bits(got, g["b%d_%d%d" % (i, xnor, scaling)]), (i, xnor, scaling)


@pytest.mark.skipif(O.ref_bnn is None, reason="oracle/_ref/libbolt_ref_bnn.so not built")
def test_ref_bnn_sweep():
    """wider than the fixtures: odd sizes, strides, asymmetric images, against the compiled reference"""
    k = 0
    for n, ic, hw, oc, f, st, pad in [(1, 8, 4, 8, 1, 1, 0), (2, 16, 5, 8, 3, 2, 1), (1, 24, 7, 16, 3, 1, 0), (1, 48, 6, 24, 5, 2, 2),
                                      (3, 8, 9, 40, 3, 3, 1), (1, 128, 5, 8, 3, 1, 1)]:
        shape = (n, ic, hw, hw + 1, oc, f, f, st, pad)
        for xnor in (0, 1):
            x = synth.normal(12000 + k, (n, ic, hw, hw + 1)).astype(np.float16)
            wbits = cases.pack_bits_msb(synth.normal(12500 + k, (oc * ic * f * f,)) >= 0)
            scale = (synth.normal(12600 + k, (oc,)) * 0.3).astype(np.float16).view(np.uint16)
            bias = synth.normal(12700 + k, (oc,)).astype(np.float16).view(np.uint16)
            xin = cases.to_blocked(x.view(np.uint16), 8)
            assert same_bits(O.port_bnn(shape, xnor, xin, wbits, scale, bias), O.ref_bnn_conv(shape, xnor, xin, wbits, scale, bias)), shape
            k += 1


def test_bnn_oracle_hand_checkable_cases():
    """Cases whose answers follow directly from the definitions in
    cpu/arm/bnn/convolution_xnor_A76.cpp:67-79,300-374 and convolution_dorefa_A76.cpp:167-199."""
    import ctypes as C
    f16 = lambda v: int(np.float16(v).view(np.uint16))
    n, ic, hw, oc = 1, 8, 3, 8
    ones_w = np.full(oc * ic * 9 // 8, 0xFF, np.uint8)                  # every weight bit set (+1)
    x_pos = np.full(ic * hw * hw, f16(1.0), np.uint16)                   # every activation bit set
    scale, bias = np.full(oc, f16(0.5), np.uint16), np.full(oc, f16(0.25), np.uint16)
    out, sums = np.zeros(oc * hw * hw, np.uint16), np.zeros(oc * hw * hw, np.int32)
    s = O.BnnShape(n, ic, hw, hw, oc, 3, 3, 1, 1, 1, 1, 1, 1, 1)
    O.port.oracle_bnn_conv(C.byref(s), ptr(x_pos), ptr(ones_w), ptr(scale), ptr(bias), ptr(out), ptr(sums))
    sums = sums.reshape(oc // 8, hw, hw, 8)
    # XNOR: valid taps contribute +ic each, padded taps (-1 against +1) contribute -ic each
    assert sums[0, 1, 1, 0] == 9 * ic and sums[0, 0, 0, 0] == 4 * ic - 5 * ic and sums[0, 0, 1, 0] == 6 * ic - 3 * ic
    assert out.reshape(oc // 8, hw, hw, 8)[0, 1, 1, 0] == f16(72 * 0.5 + 0.25)
    s = O.BnnShape(n, ic, hw, hw, oc, 3, 3, 1, 1, 1, 1, 1, 1, 0)
    O.port.oracle_bnn_conv(C.byref(s), ptr(x_pos), ptr(ones_w), ptr(scale), ptr(bias), ptr(out), ptr(sums))
    sums = sums.reshape(oc // 8, hw, hw, 8)
    # DoReFa: popcount(and), padding contributes nothing
    assert sums[0, 1, 1, 0] == 9 * ic and sums[0, 0, 0, 0] == 4 * ic and sums[0, 0, 1, 0] == 6 * ic
    x_thr = np.full(ic * hw * hw, f16(0.49), np.uint16)                  # below 0.5 -> bit 0 in DoReFa, bit 1 in XNOR
    O.port.oracle_bnn_conv(C.byref(s), ptr(x_thr), ptr(ones_w), ptr(scale), ptr(bias), ptr(out), ptr(sums))
    assert not sums.any()
    # fp16 fused multiply-add: one rounding (2049 * 1 + 1 = 2050 exactly; two roundings would give 2048 + 1 -> 2048)
    assert O.port.oracle_f16_fma(f16(2048.0), f16(1.0), f16(1.0)) == f16(2048.0)      # 2049 ties to even 2048
    assert O.port.oracle_f16_fma(f16(1.0009765625), f16(1.0009765625), f16(-1.0)) == int(np.float16(0.001953125 + 2.0 ** -20).view(np.uint16))
    assert O.port.oracle_i32_to_f16(2049) == f16(2048.0) and O.port.oracle_i32_to_f16(2051) == f16(2052.0)


def test_known_answers_u8_saturation():
    """The reference's u8 epilogue reads the rounded sum as unsigned: negatives store 255."""
    assert O.port.oracle_usat8(-800 + 128) == 255
    assert O.port.oracle_usat8(O.port.oracle_cvt_rne(-800 * 0.1) + 128) == 48
    assert O.port.oracle_usat8(80 + 128) == 208
    assert O.port.oracle_cvt_rne(0.5) == 0 and O.port.oracle_cvt_rne(1.5) == 2 and O.port.oracle_cvt_rne(-2.5) == -2
    assert O.port.oracle_cvt_rne(3e9) == -2147483648 and O.port.oracle_cvt_rne(float("nan")) == -2147483648


# ---------------------------------------------------------------- compiled reference
@needs_ref
def test_ref_gemm_cover_sweep():
    bad = 0
    for m, k, n in itertools.product([1, 2, 7, 8, 9, 24, 33], [1, 3, 4, 7, 8, 9, 16, 31, 33], [1, 5, 8, 15, 16, 17, 33, 48, 49, 64]):
        for a_t, b_t, pre in itertools.product((0, 1), (0, 1), (0, 1)):
            seed = (m * 64 + k) * 64 + n
            A = synth.u8(seed, (k, m) if a_t else (m, k))
            B = synth.s8(seed + 1, (n, k) if b_t else (k, n))
            Cin = synth.integers(seed + 2, (m, n), -1000, 1000)
            r = O.ref_gemm(A, B, None, Cin, a_t, b_t, prepack=bool(pre))
            p = O.port_gemm(A, B, O.port_offsetc(B, b_t), None, Cin, a_t, b_t)
            bad += not same_bits(r, p)
    assert bad == 0


@needs_ref
def test_ref_gemm_epilogues():
    for (m, k, n) in [(5, 40, 50), (33, 128, 96), (8, 4100, 16), (128, 768, 768)]:
        A = synth.u8(m + k, (m, k))
        B = synth.s8(m + k + 1, (k, n))
        off = O.port_offsetc(B)
        for sc in ([0.37], [123.4], [-1, 0.001], [-1, 0.01], [-1, 1.0], [-1, 0.0003]):
            if sc[0] < 0:  # one row per call: the reference overruns u8 outputs with M > 1
                r = np.concatenate([O.ref_gemm(A[i:i + 1], B, sc) for i in range(m)])
            else:
                r = O.ref_gemm(A, B, sc)
            assert same_bits(r, O.port_gemm(A, B, off, sc)), (m, k, n, sc)
        Cin = synth.integers(9, (m, n), -100, 100).view(np.float32)
        assert same_bits(O.ref_gemm(A, B, [0.5], Cin), O.port_gemm(A, B, off, [0.5], Cin))


@needs_ref
def test_ref_gemv_sweep():
    for n, k in itertools.product([1, 3, 7, 8, 9, 15, 16, 17, 31, 33, 63, 64, 65, 100, 129], [1, 2, 3, 4, 5, 8, 9, 31, 32, 33, 65, 2049, 2100]):
        for w_t in (0, 1):
            W = synth.s8(n * 4096 + k, (k, n) if w_t else (n, k))
            x = synth.u8(n * 4096 + k + 1, (k,))
            off = O.port_offsetc(W, not w_t)
            yin = synth.integers(5, (n,), -1000, 1000)
            for sc in (None, [0.37], [-1, 0.001], [-1, 0.01]):
                yi = yin if sc is None else None
                assert same_bits(O.ref_gemv(W, x, sc, yi, w_t), O.port_gemv(W, x, off, sc, yi, w_t)), (n, k, w_t, sc)


@needs_ref
def test_ref_quantize_sweep():
    for n in [1, 5, 15, 16, 17, 100, 1000, 4099]:
        for std in (1.0, 0.02, 50.0):
            x = synth.normal(n, (n,), std)
            for name, dst, dt in (("u8", np.uint8, O.DT_U8_Q), ("i8", np.int8, O.DT_I8)):
                for sc0, mode in ((-1, 0), (0.5, 0), (3.0, 1), (1e9, 0)):
                    qr = np.zeros(n, dst)
                    sr = np.array([sc0], np.float32)
                    O.ref.ref_quantize(n, O.DT_F32, ptr(x), dt, ptr(qr), ptr(sr), mode)
                    qp, sp = port_quant("f32" + name, x, dst, [sc0], mode)
                    assert same_bits(qr, qp) and same_bits(sr, sp), (n, std, name, sc0, mode)
        a = synth.integers(n + 7, (n,), -100000, 100000)
        for name, dst, dt in (("u8", np.uint8, O.DT_U8_Q), ("i8", np.int8, O.DT_I8)):
            for sc in ([-1, 0.37], [2.0, 0.37], [-1, -1], [0.001, 5.0]):
                qr = np.zeros(n, dst)
                sr = np.array(sc, np.float32)
                O.ref.ref_quantize(n, O.DT_I32, ptr(a), dt, ptr(qr), ptr(sr), 0)
                qp, sp = port_quant("i32" + name, a, dst, sc)
                assert same_bits(qr, qp) and same_bits(sr, sp), (n, name, sc)


def test_golden_matmul():
    """The restatement of the matmul operator, built from the scalar primitives, against the reference's outputs."""
    g = np.load(os.path.join(GOLD, "matmul.npz"))
    for name in cases.MATMUL_CASES:
        C, scale = O.port_matmul(*cases.matmul_inputs(name))
        assert C.shape == g[name].shape and C.tobytes() == g[name].tobytes(), name
        assert np.float32(scale).tobytes() == g[name + "_scale"].tobytes(), name


@needs_ref
def test_ref_matmul_sweep():
    """small shapes around the kernels' edge sizes, fp32 and dynamically quantized outputs"""
    F, U = O.DT_F32, O.DT_U8_Q
    for m, k, n in itertools.product([1, 2, 17, 48], [3, 64, 100], [1, 16, 49]):
        for ta, tb in ((0, 0), (1, 1)):
            A = synth.normal(m * 100 + k, (2, k, m) if ta else (2, m, k))
            B = synth.normal(n * 100 + k + 1, (2, n, k) if tb else (2, k, n))
            for c_dt, c_scale in ((F, -1.0), (U, -1.0)):
                args = (A, F, -1.0, ta, B, F, -1.0, tb, None, c_dt, c_scale)
                rc, Cr, sr = O.ref_matmul(*args)
                Cp, sp = O.port_matmul(*args)
                assert rc == 0 and Cr.tobytes() == Cp.tobytes() and np.float32(sr) == np.float32(sp), (m, k, n, ta, tb, c_dt)


def _port_pool(i):
    case = cases.POOL_CASES[i]
    n, c, ih, iw, k, s, p, mean, cip, ceil = case
    oh, ow = cases.pool_out_hw(case)
    x = cases.pool_input(i)
    y = np.zeros(n * c * oh * ow, np.uint8)
    sc = np.array([3.5, -1.0], np.float32)
    rc = O.port.oracle_pooling_u8(n, c, ih, iw, oh, ow, k, k, s, s, p, p, mean, cip, ptr(x), ptr(y), ptr(sc))
    return rc, y, sc


def test_golden_pooling():
    g = np.load(os.path.join(GOLD, "pooling.npz"))
    for i in range(len(cases.POOL_CASES)):
        rc, y, sc = _port_pool(i)
        assert rc == 0 and y.tobytes() == g["p%d" % i].tobytes() and sc.tobytes() == g["p%d_scale" % i].tobytes(), cases.POOL_CASES[i]
    # a mean window whose values all lie below the zero point stores 255 (logical shift of a negative product)
    x = np.full(16 * 4 * 4, 100, np.uint8)
    y = np.zeros(16 * 2 * 2, np.uint8)
    sc = np.array([1.0, 0.0], np.float32)
    assert O.port.oracle_pooling_u8(1, 16, 4, 4, 2, 2, 2, 2, 2, 2, 0, 0, 1, 0, ptr(x), ptr(y), ptr(sc)) == 0
    assert (y == 255).all()
