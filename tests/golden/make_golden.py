"""Generates tests/golden/*.npz from the UNMODIFIED reference (oracle/_ref/libbolt_ref.so and
oracle/_ref/libbolt_ref_bnn.so, built from the Bolt sources by `make -C oracle ref BOLT_ROOT=...`).  Run in a container that has the reference tree
and an avx512_vnni CPU:

    python tests/golden/make_golden.py

Inputs come from tests/golden/cases.py (seeded, reproducible anywhere); the fixtures hold only the
reference's outputs, so the checks that use them need neither the reference tree nor AVX512.
The u8 GEMM outputs are produced one row (M = 1) per call: for M > 1 the reference's AVX512
kernel strides u8 rows by 4N bytes and overruns its output
(compute/blas_enhance/src/cpu/x86/int8/avx512/mmm_avx512_vnni.cpp:1468,1473).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)
import cases  # noqa: E402
import oracle as O  # noqa: E402
from oracle import ptr  # noqa: E402

assert O.ref is not None, "needs oracle/_ref/libbolt_ref.so and an avx512_vnni host"
assert O.ref_bnn is not None, "needs oracle/_ref/libbolt_ref_bnn.so (make -C oracle ref BOLT_ROOT=...)"


def gemm_outputs():
    out = {}
    for i in range(len(cases.GEMM_SHAPES)):
        m = cases.GEMM_SHAPES[i][0]
        for a_t, b_t in cases.gemm_variants(i):
            A, B, Cin = cases.gemm_inputs(i, a_t, b_t)
            key = "g%d_%d%d" % (i, a_t, b_t)
            out[key + "_s32"] = O.ref_gemm(A, B, None, Cin, a_t, b_t)
            if a_t == 0:
                out[key + "_f32"] = O.ref_gemm(A, B, cases.GEMM_F32_SCALE, None, a_t, b_t)
                rows = [O.ref_gemm(A[r:r + 1], B, cases.GEMM_U8_SCALE, None, 0, b_t) for r in range(m)]
                out[key + "_u8"] = np.concatenate(rows)
    return out


def gemv_outputs():
    out = {}
    for i in range(len(cases.GEMV_SHAPES)):
        for w_t in (0, 1):
            W, x, yin = cases.gemv_inputs(i, w_t)
            key = "v%d_%d" % (i, w_t)
            out[key + "_s32"] = O.ref_gemv(W, x, None, yin, w_t)
            out[key + "_f32"] = O.ref_gemv(W, x, cases.GEMM_F32_SCALE, None, w_t)
            out[key + "_u8"] = O.ref_gemv(W, x, cases.GEMM_U8_SCALE, None, w_t)
    return out


def quant_outputs():
    out = {}
    for i, n in enumerate(cases.QUANT_SIZES):
        x, a, u, b, off = cases.quant_inputs(i)
        for name, dst, dt in (("u8", np.uint8, O.DT_U8_Q), ("i8", np.int8, O.DT_I8)):
            q = np.zeros(n, dst)
            s = np.array([-1], np.float32)
            O.ref.ref_quantize(n, O.DT_F32, ptr(x), dt, ptr(q), ptr(s), 0)
            out["q%d_f32_%s" % (i, name)], out["q%d_f32_%s_scale" % (i, name)] = q, s.copy()
            q = np.zeros(n, dst)
            s = np.array([-1, 0.37], np.float32)
            O.ref.ref_quantize(n, O.DT_I32, ptr(a), dt, ptr(q), ptr(s), 0)
            out["q%d_i32_%s" % (i, name)], out["q%d_i32_%s_scale" % (i, name)] = q, s.copy()
            q = np.zeros(n, dst)
            s = np.array([2.0, 0.37], np.float32)
            O.ref.ref_quantize(n, O.DT_I32, ptr(a), dt, ptr(q), ptr(s), 0)
            out["q%d_i32s_%s" % (i, name)] = q
        q = np.zeros(n, np.int8)
        O.ref.ref_quantize(n, O.DT_U8_Q, ptr(u), O.DT_I8, ptr(q), None, 0)
        out["q%d_u8i8" % i] = q
        s = np.array([0.37], np.float32)
        ap = np.zeros(n + 64, np.int32)
        ap[:n] = a
        f = np.zeros(n + 64, np.float32)  # padded: the reference writes a whole vector when n < 16
        O.ref.ref_dequantize(n, O.DT_I32, ptr(ap), ptr(s), ptr(f))
        out["q%d_dq_i32" % i] = f[:n].copy()
        f = np.zeros(n, np.float32)
        O.ref.ref_dequantize(n, O.DT_U8_Q, ptr(u), ptr(s), ptr(f))
        out["q%d_dq_u8" % i] = f
        r = np.zeros(n, np.int32)
        O.ref.ref_bias_offsetc(n, ptr(b), ptr(off), 3.0, ptr(r))
        out["q%d_biasoff" % i] = r
    return out


def conv_outputs():
    import ctypes as C
    out = {}
    for i, (n, ic, ih, iw, oc, fh, fw, st, pad) in enumerate(cases.CONV_SHAPES):
        oh, ow = (ih + 2 * pad - fh) // st + 1, (iw + 2 * pad - fw) // st + 1
        tot = n * oc * oh * ow
        for blk, out_u8, relu in cases.conv_variants(i):
            xin, w, bias = cases.conv_inputs(i, blk)
            pl = O.ref.ref_conv_plan(n, ic, ih, iw, oc, fh, fw, st, pad, blk, 16, out_u8, relu, ptr(w))
            assert pl
            res = np.zeros(tot + 64, np.uint8 if out_u8 else np.float32)
            sc = np.array(cases.CONV_SCALES, np.float32)
            assert O.ref.ref_conv_run(pl, ptr(xin.copy()), None, ptr(bias), ptr(res), ptr(sc)) == 0
            O.ref.ref_conv_free(pl)
            key = "c%d_%d%d%d" % (i, blk, out_u8, relu)
            out[key], out[key + "_scale"] = res[:tot].copy(), sc.copy()
        # u8 output with a residual input (fp32 staging + F32 -> U8_Q), and activation modes other than ReLU
        for key, out_u8, act, with_elt in cases.conv_extra_variants(i):
            xin, w, bias = cases.conv_inputs(i, 16 if ic % 16 == 0 else 8)
            blk = 16 if ic % 16 == 0 else 8
            elt = cases.conv_eltwise(i, tot) if with_elt else None
            pl = O.ref.ref_conv_plan(n, ic, ih, iw, oc, fh, fw, st, pad, blk, 16, out_u8, act, ptr(w))
            assert pl
            res = np.zeros(tot + 64, np.uint8 if out_u8 else np.float32)
            sc = np.array(cases.CONV_SCALES, np.float32)
            assert O.ref.ref_conv_run(pl, ptr(xin.copy()), ptr(elt), ptr(bias), ptr(res), ptr(sc)) == 0
            O.ref.ref_conv_free(pl)
            out["c%d_%s" % (i, key)], out["c%d_%s_scale" % (i, key)] = res[:tot].copy(), sc.copy()
    return out


def gemv_row_outputs():
    out = {}
    for i in range(len(cases.GEMV_ROW_SHAPES)):
        for m_t in (0, 1):
            Mx, v = cases.gemv_row_inputs(i, m_t)
            key = "r%d_%d" % (i, m_t)
            out[key + "_s32"] = O.ref_gemv_row(Mx, v, None, m_t)
            out[key + "_f32"] = O.ref_gemv_row(Mx, v, cases.GEMM_F32_SCALE, m_t)
            out[key + "_u8"] = O.ref_gemv_row(Mx, v, cases.GEMM_U8_SCALE, m_t)
    return out


def bnn_outputs():
    """the reference's scalar 1-bit convolution (cpu/general/convolution.cpp:141-179,264-285), both modes"""
    out = {}
    for i, shape in enumerate(cases.BNN_SHAPES):
        for xnor in (0, 1):
            for scaling in (0, 1, 2):
                xin, wbits, scale, bias = cases.bnn_inputs(i, xnor, scaling)
                out["b%d_%d%d" % (i, xnor, scaling)] = O.ref_bnn_conv(shape, xnor, xin, wbits, scale, bias)
    return out


def matmul_outputs():
    """the reference's matmul operator (compute/tensor/src/matmul.cpp) on its x86 int8 branch"""
    out = {}
    for name in cases.MATMUL_CASES:
        rc, C, scale = O.ref_matmul(*cases.matmul_inputs(name))
        assert rc == 0, name
        out[name] = C
        out[name + "_scale"] = np.float32(scale)
    return out


def pool_outputs():
    """the reference's u8 pooling (cpu/x86/int8/avx512/pooling_int8.cpp)"""
    import ctypes as C
    O.ref.ref_pooling_u8.argtypes = [C.c_uint32] * 12 + [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    out = {}
    for i, case in enumerate(cases.POOL_CASES):
        n, c, ih, iw, k, s, p, mean, cip, ceil = case
        oh, ow = cases.pool_out_hw(case)
        x = cases.pool_input(i)
        y = np.zeros(n * c * oh * ow, np.uint8)
        sc = np.array([3.5, -1.0], np.float32)
        rc = O.ref.ref_pooling_u8(n, c, ih, iw, oh, ow, k, k, s, s, p, p, mean, cip, ptr(x), ptr(y), ptr(sc))
        assert rc == 0, case
        out["p%d" % i] = y
        out["p%d_scale" % i] = sc
    return out


def main():
    np.savez_compressed(os.path.join(HERE, "pooling.npz"), **pool_outputs())
    np.savez_compressed(os.path.join(HERE, "matmul.npz"), **matmul_outputs())
    np.savez_compressed(os.path.join(HERE, "bnn.npz"), **bnn_outputs())
    np.savez_compressed(os.path.join(HERE, "gemv_row.npz"), **gemv_row_outputs())
    np.savez_compressed(os.path.join(HERE, "conv.npz"), **conv_outputs())
    np.savez_compressed(os.path.join(HERE, "gemm.npz"), **gemm_outputs())
    np.savez_compressed(os.path.join(HERE, "gemv.npz"), **gemv_outputs())
    np.savez_compressed(os.path.join(HERE, "quantize.npz"), **quant_outputs())
    for f in ("gemm.npz", "gemv.npz", "gemv_row.npz", "quantize.npz", "conv.npz", "matmul.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
