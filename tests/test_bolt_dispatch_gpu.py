"""Bolt's own entry points with Arch = CUDA_B200.

integration/build_dispatch.py compiles the reference's dispatchers (blas_enhance/src/mmm.cpp, mvm.cpp,
tensor/src/quantize.cpp, dequantize.cpp, convolution.cpp) with the CUDA_B200 branches a maintainer would add,
against libbolt_b200.so.  These tests call the symbols of that library -- `matrix_matrix_multiply`,
`matrix_vector_multiply`, `quantize`, `dequantize`, `convolution` -- exactly as the reference's unit tests do
(compute/blas_enhance/tests/test_mmm.cpp:69-91, test_mvm.cpp, compute/tensor/tests/test_convolution_int8.cpp),
and compare with the golden outputs of the reference's x86 path and with the oracle, bit for bit.
"""
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

GOLD = os.path.join(os.path.dirname(__file__), "golden")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DISPATCH = os.path.join(ROOT, "integration", "_build", "libbolt_dispatch_b200.so")
ARCH = 11  # CUDA_B200 in the patched common/uni/include/sys.h
TD = B.TensorDesc


def bolt():
    if not os.path.exists(DISPATCH):
        pytest.skip("integration/_build/libbolt_dispatch_b200.so is not built (python integration/build_dispatch.py BOLT_ROOT)")
    B.load(build_if_missing=False)
    L = C.CDLL(DISPATCH)
    u32p, vp, f32p = C.POINTER(C.c_uint32), C.c_void_p, C.POINTER(C.c_float)
    sig = {
        "matrix_matrix_multiply_tmp_bytes": [TD, TD, u32p, C.c_int],
        "matrix_matrix_multiply_transform_rhs_bytes": [TD, u32p, u32p, C.c_int],
        "matrix_matrix_multiply_transform_rhs": [TD, vp, C.POINTER(TD), vp, C.c_int],
        "matrix_matrix_multiply": [TD, vp, TD, vp, C.c_uint32, vp, TD, vp, f32p, C.c_int],
        "matrix_vector_multiply_tmp_bytes": [TD, TD, u32p, C.c_int],
        "matrix_vector_multiply_transform_weight_bytes": [TD, u32p, C.c_int],
        "matrix_vector_multiply_transform_weight": [TD, vp, C.POINTER(TD), vp, C.c_int],
        "matrix_vector_multiply": [TD, vp, TD, vp, C.c_uint32, vp, TD, vp, f32p, C.c_int],
        "shim_quantize": [C.POINTER(TD), vp, C.POINTER(TD), vp, f32p],
        "shim_dequantize": [C.POINTER(TD), vp, f32p, C.POINTER(TD), vp, C.POINTER(TD), vp],
        "shim_conv_output_size": [C.POINTER(TD), C.POINTER(TD), C.POINTER(B.ConvolutionParamSpec), C.POINTER(TD), C.c_int],
        "shim_conv_prepare": [C.POINTER(TD), C.POINTER(TD), vp, C.POINTER(TD), C.POINTER(B.ConvolutionParamSpec),
                              C.POINTER(B.ActivationParamSpec), C.c_int, C.POINTER(C.c_int), u32p, vp, C.POINTER(TD), u32p],
        "shim_convolution": [C.POINTER(TD), vp, C.POINTER(TD), vp, C.POINTER(TD), vp, C.POINTER(B.ConvolutionParamSpec),
                             C.c_int, f32p, C.POINTER(TD), vp, C.c_uint32, vp, C.POINTER(TD), vp,
                             C.POINTER(B.ActivationParamSpec)],
    }
    sig["shim_matmul"] = [C.POINTER(TD), vp, C.c_float, C.c_int, C.POINTER(TD), vp, C.c_float, C.c_int, C.c_uint32, vp, C.c_int, f32p,
                          vp, C.POINTER(TD), vp, C.c_uint32]
    for name, args in sig.items():
        f = getattr(L, name)
        f.argtypes, f.restype = args, C.c_int
    L.shim_arch_name.restype = C.c_char_p
    return L


def ok(code, what):
    B.CHECK_STATUS(code, what)


def fscale(values):
    return None if values is None else (C.c_float * len(values))(*values)


def test_dispatch_library_knows_the_new_arch():
    L = bolt()
    assert L.shim_arch_cuda_b200() == ARCH
    assert L.shim_arch_name() == b"CUDA_B200"
    # byte counts are host arithmetic: Bolt's symbol reaches libbolt_b200.so without a GPU
    nb, off = C.c_uint32(), C.c_uint32()
    ok(L.matrix_matrix_multiply_transform_rhs_bytes(B.tensor2df(B.DT_I8, B.DF_NORMAL, 768, 3072), C.byref(nb), C.byref(off), ARCH), "rhs bytes")
    assert (nb.value, off.value) == B.matrix_matrix_multiply_transform_rhs_bytes(B.tensor2df(B.DT_I8, B.DF_NORMAL, 768, 3072))
    assert off.value == 768 * 3072 and nb.value >= off.value + 4 * 3072


def mmm_through_bolt(L, A, Bm, scale, Cin, a_t, b_t, transform, host):
    """test_mmm.cpp:mmmTestKernel, UT_ARCH = CUDA_B200"""
    m, k = (A.shape[1], A.shape[0]) if a_t else A.shape
    n = Bm.shape[0] if b_t else Bm.shape[1]
    a_desc = B.tensor2df(B.DT_U8_Q, B.DF_TRANSPOSE, k, m) if a_t else B.tensor2df(B.DT_U8_Q, B.DF_NORMAL, m, k)
    b_desc = B.tensor2df(B.DT_I8, B.DF_TRANSPOSE, n, k) if b_t else B.tensor2df(B.DT_I8, B.DF_NORMAL, k, n)
    cdt = B.DT_I32 if scale is None else (B.DT_U8_Q if scale[0] < 0 else B.DT_F32)
    npdt = {B.DT_I32: np.int32, B.DT_F32: np.float32, B.DT_U8_Q: np.uint8}[cdt]
    c_desc = B.tensor2df(cdt, B.DF_NORMAL, m, n)
    Cbuf = np.zeros((m, n), npdt) if Cin is None else np.ascontiguousarray(Cin).copy()
    keep = []

    def buf(a):
        if host:
            keep.append(a)
            return a, hptr(a)
        t = to_dev(a) if a.dtype != np.uint8 or a.ndim != 1 or a.any() else dev_zeros(a.size)
        keep.append(t)
        return t, dptr(t)

    _, pA = buf(A)
    _, pB = buf(Bm)
    trans_desc, p_trans, offset, trans = b_desc, pB, 0, None
    if transform:
        nb, off = C.c_uint32(), C.c_uint32()
        ok(L.matrix_matrix_multiply_transform_rhs_bytes(b_desc, C.byref(nb), C.byref(off), ARCH), "rhs bytes")
        offset = off.value
        trans, p_trans = buf(np.zeros(nb.value, np.uint8))
        trans_desc = TD()
        ok(L.matrix_matrix_multiply_transform_rhs(b_desc, pB, C.byref(trans_desc), p_trans, ARCH), "transform rhs")
    nbt = C.c_uint32()
    ok(L.matrix_matrix_multiply_tmp_bytes(a_desc, trans_desc, C.byref(nbt), ARCH), "tmp bytes")
    tmp, p_tmp = buf(np.zeros(max(nbt.value, 16), np.uint8))
    if transform:
        tmp[: 4 * n] = trans[offset: offset + 4 * n]   # test_mmm.cpp:83-85
    cb, pC = buf(Cbuf)
    ok(L.matrix_matrix_multiply(a_desc, pA, trans_desc, p_trans, nbt.value, p_tmp, c_desc, pC, fscale(scale), ARCH), "mmm")
    ok(B.lib().bolt_b200_synchronize(), "synchronize")
    if host:
        if transform:
            B.lib().bolt_b200_release_weight(p_trans)
        return Cbuf
    return to_host(cb, npdt, m * n).reshape(m, n)


@pytest.mark.gpu
@pytest.mark.parametrize("host", [False, True])
def test_bolt_matrix_matrix_multiply_golden(host):
    L = bolt()
    g = np.load(os.path.join(GOLD, "gemm.npz"))
    for i in range(len(cases.GEMM_SHAPES)):
        for a_t, b_t in cases.gemm_variants(i):
            A, Bm, Cin = cases.gemm_inputs(i, a_t, b_t)
            key = "g%d_%d%d" % (i, a_t, b_t)
            for transform in (True, False):
                got = mmm_through_bolt(L, A, Bm, None, Cin, a_t, b_t, transform, host)
                assert got.tobytes() == g[key + "_s32"].tobytes(), (key, transform, host)
            if a_t == 0:
                got = mmm_through_bolt(L, A, Bm, cases.GEMM_F32_SCALE, None, 0, b_t, True, host)
                assert got.tobytes() == g[key + "_f32"].tobytes(), key
                got = mmm_through_bolt(L, A, Bm, cases.GEMM_U8_SCALE, None, 0, b_t, True, host)
                assert got.tobytes() == g[key + "_u8"].tobytes(), key


@pytest.mark.gpu
def test_bolt_matrix_matrix_multiply_headline_shape_vs_oracle():
    """M 4096 (batch 32 x 128 tokens), K 768, N 768: the BERT-base projection, packed weight, int32 accumulate."""
    L = bolt()
    m, k, n = 512, 768, 768
    A, Bm = synth.u8(11, (m, k)), synth.s8(12, (k, n))
    Cin = synth.s8(13, (m, n)).astype(np.int32)
    got = mmm_through_bolt(L, A, Bm, None, Cin, 0, 0, True, False)
    ref = O.port_gemm(A, Bm, O.port_offsetc(Bm), None) + Cin
    assert got.tobytes() == ref.astype(np.int32).tobytes()
    assert B.lib().bolt_b200_last_gemm_used_tensor_cores() == 1


@pytest.mark.gpu
@pytest.mark.parametrize("host", [False, True])
def test_bolt_matrix_vector_multiply(host):
    """test_mvm.cpp: packed and on-the-fly weights, int32 result on top of the incoming values"""
    L = bolt()
    for row, col, t in ((33, 65, 0), (768, 768, 0), (100, 48, 1), (1000, 2048, 0)):
        W = synth.s8(row * 7 + col, (col, row) if t else (row, col))
        v = synth.u8(row + col, (col,))
        Wn = np.ascontiguousarray(W.T) if t else W
        y0 = np.arange(row, dtype=np.int32) - 5
        # (rows of the last partial group of 16 overwrite instead of accumulating, in the reference as here)
        ref = O.port_gemv(Wn, v, O.port_offsetc(Wn, True), None, y0)
        m_desc = B.tensor2df(B.DT_I8, B.DF_TRANSPOSE, col, row) if t else B.tensor2df(B.DT_I8, B.DF_NORMAL, row, col)
        v_desc, r_desc = B.tensor1d(B.DT_U8_Q, col), B.tensor1d(B.DT_I32, row)
        for transform in (True, False):
            keep = []

            def buf(a):
                if host:
                    keep.append(a)
                    return a, hptr(a)
                tt = to_dev(a) if a.any() else dev_zeros(a.size * a.itemsize)
                keep.append(tt)
                return tt, dptr(tt)

            _, pW = buf(W)
            _, pv = buf(v)
            desc, p_mat = m_desc, pW
            nbt = C.c_uint32()
            if transform:
                nb = C.c_uint32()
                ok(L.matrix_vector_multiply_transform_weight_bytes(m_desc, C.byref(nb), ARCH), "weight bytes")
                packed, p_mat = buf(np.zeros(nb.value, np.uint8))
                desc = TD()
                ok(L.matrix_vector_multiply_transform_weight(m_desc, pW, C.byref(desc), p_mat, ARCH), "transform weight")
            ok(L.matrix_vector_multiply_tmp_bytes(desc, v_desc, C.byref(nbt), ARCH), "tmp bytes")
            tmp, p_tmp = buf(np.zeros(nbt.value + 64, np.uint8))
            if transform:
                o = ((row + 15) // 16 * 16) * ((col + 7) // 8 * 8)
                tmp[: 4 * row] = packed[o: o + 4 * row]     # test_mvm.cpp: offsetC travels in tmp
            y, py = buf(y0.copy())
            ok(L.matrix_vector_multiply(desc, p_mat, v_desc, pv, nbt.value, p_tmp, r_desc, py, None, ARCH), "mvm")
            ok(B.lib().bolt_b200_synchronize(), "synchronize")
            got = y if host else to_host(y, np.int32, row)
            if host and transform:
                B.lib().bolt_b200_release_weight(p_mat)
            assert np.array_equal(got, ref), (row, col, t, transform, host)


@pytest.mark.gpu
def test_bolt_quantize_and_dequantize():
    """tensor/src/quantize.cpp and dequantize.cpp: a Tensor over the caller's buffer, ArchInfo.arch = CUDA_B200"""
    L = bolt()
    g = np.load(os.path.join(GOLD, "quantize.npz"))
    for i, n in enumerate(cases.QUANT_SIZES):
        x, a, u, b, off = cases.quant_inputs(i)
        for host in (False, True):
            for name, qdt, npq in (("u8", B.DT_U8_Q, np.uint8), ("i8", B.DT_I8, np.int8)):
                q = np.zeros(n, npq)
                d_desc, q_desc = B.tensor1d(B.DT_F32, n), B.tensor1d(qdt, n)
                s = (C.c_float * 1)(-1.0)
                if host:
                    ok(L.shim_quantize(C.byref(d_desc), hptr(x), C.byref(q_desc), hptr(q), s), "quantize")
                    got = q
                else:
                    dx, dq = to_dev(x), dev_zeros(n)
                    ok(L.shim_quantize(C.byref(d_desc), dptr(dx), C.byref(q_desc), dptr(dq), s), "quantize")
                    ok(B.lib().bolt_b200_synchronize(), "synchronize")
                    got = to_host(dq, npq, n)
                assert got.tobytes() == g["q%d_f32_%s" % (i, name)].tobytes(), (i, host, name)
                assert np.float32(s[0]).tobytes() == np.float32(g["q%d_f32_%s_scale" % (i, name)]).tobytes()
            for src, sdt, key in ((a, B.DT_I32, "dq_i32"), (u, B.DT_U8_Q, "dq_u8")):
                q_desc, d_desc, b_desc = B.tensor1d(sdt, n), B.tensor1d(B.DT_F32, n), B.tensor1d(B.DT_F32, 0)
                s = (C.c_float * 1)(0.37)
                out = np.zeros(n, np.float32)
                if host:
                    ok(L.shim_dequantize(C.byref(q_desc), hptr(src), s, C.byref(b_desc), None, C.byref(d_desc), hptr(out)), "dequantize")
                    got = out
                else:
                    d, do = to_dev(src), dev_zeros(4 * n)
                    ok(L.shim_dequantize(C.byref(q_desc), dptr(d), s, C.byref(b_desc), None, C.byref(d_desc), dptr(do)), "dequantize")
                    ok(B.lib().bolt_b200_synchronize(), "synchronize")
                    got = to_host(do, np.float32, n)
                assert got.tobytes() == g["q%d_%s" % (i, key)].tobytes(), (i, host, key)


DF_OF = {16: B.DF_NCHWC16, 8: B.DF_NCHWC8}


def conv_through_bolt(L, shape, xin, w, bias, blk, out_u8, relu, scales, eltwise=None):
    """test_convolution_int8.cpp's call sequence: output size, algorithm, packed-filter bytes, packing, tmp bytes, run"""
    n, ic, ih, iw, oc, fh, fw, st, pad = shape
    p = B.conv_param(oc, fh, fw, st, pad, 1, bool(relu))
    act = B.ActivationParamSpec()
    act.mode = int(relu)
    in_desc = B.tensor4df(B.DT_U8_Q, DF_OF[blk], n, ic, ih, iw)
    f_desc = B.tensor4df(B.DT_I8, B.DF_NCHW, oc, ic, fh, fw)
    target = B.DT_U8_Q if out_u8 else B.DT_F32
    out_desc = TD()
    ok(L.shim_conv_output_size(C.byref(in_desc), C.byref(f_desc), C.byref(p), C.byref(out_desc), target), "output size")
    assert out_desc.dt == target and out_desc.df == (B.DF_NCHWC16 if out_u8 and oc != 8 else B.DF_NCHWC8)
    oh, ow = out_desc.dims[1], out_desc.dims[0]
    alg, fbytes, tbytes = C.c_int(), C.c_uint32(), C.c_uint32()
    ftm_desc = TD()
    ok(L.shim_conv_prepare(C.byref(in_desc), C.byref(f_desc), None, C.byref(out_desc), C.byref(p), C.byref(act), target,
                           C.byref(alg), C.byref(fbytes), None, C.byref(ftm_desc), C.byref(tbytes)), "sizes")
    d_w, d_ftm = to_dev(w), dev_zeros(fbytes.value)
    ok(L.shim_conv_prepare(C.byref(in_desc), C.byref(f_desc), dptr(d_w), C.byref(out_desc), C.byref(p), C.byref(act), target,
                           C.byref(alg), C.byref(fbytes), dptr(d_ftm), C.byref(ftm_desc), C.byref(tbytes)), "prepare")
    tot = n * oc * oh * ow
    d_x, d_b, d_tmp, d_out = to_dev(xin), to_dev(bias), dev_zeros(tbytes.value), dev_zeros(tot * 4)
    d_e = None if eltwise is None else to_dev(eltwise)
    b_desc = B.tensor1d(B.DT_F32, oc)
    sc = (C.c_float * 3)(*scales)
    ok(L.shim_convolution(C.byref(in_desc), dptr(d_x), C.byref(out_desc), None if d_e is None else dptr(d_e),
                          C.byref(ftm_desc), dptr(d_ftm), C.byref(p), alg.value, sc, C.byref(b_desc), dptr(d_b),
                          tbytes.value, dptr(d_tmp), C.byref(out_desc), dptr(d_out), C.byref(act)), "convolution")
    ok(B.lib().bolt_b200_synchronize(), "synchronize")
    return to_host(d_out, np.uint8 if out_u8 else np.float32, tot), list(sc)


@pytest.mark.gpu
def test_bolt_convolution_golden():
    L = bolt()
    g = np.load(os.path.join(GOLD, "conv.npz"))
    for i, shape in enumerate(cases.CONV_SHAPES):
        for blk, out_u8, relu in cases.conv_variants(i):
            xin, w, bias = cases.conv_inputs(i, blk)
            got, sc = conv_through_bolt(L, shape, xin, w, bias, blk, out_u8, relu, cases.CONV_SCALES)
            key = "c%d_%d%d%d" % (i, blk, out_u8, relu)
            assert got.tobytes() == g[key].tobytes(), key
            assert np.array(sc, np.float32).tobytes() == g[key + "_scale"].tobytes(), key
        for name, out_u8, actm, with_elt in cases.conv_extra_variants(i):
            if not with_elt:
                continue
            blk = 16 if shape[1] % 16 == 0 else 8
            xin, w, bias = cases.conv_inputs(i, blk)
            key = "c%d_%s" % (i, name)
            elt = cases.conv_eltwise(i, g[key].size)
            got, sc = conv_through_bolt(L, shape, xin, w, bias, blk, out_u8, actm, cases.CONV_SCALES, eltwise=elt)
            assert got.tobytes() == g[key].tobytes(), key


@pytest.mark.gpu
def test_bolt_matmul_golden():
    """tensor/src/matmul.cpp with ArchInfo.arch = CUDA_B200: output size, tmp bytes and the run through Bolt's own
    functions, scales carried by the Tensors"""
    L = bolt()
    g = np.load(os.path.join(GOLD, "matmul.npz"))
    for name in cases.MATMUL_CASES:
        A, a_dt, a_s, ta, Bm, b_dt, b_s, tb, bias, c_dt, c_s = cases.matmul_inputs(name)
        a_desc, b_desc = B.tensor_nd(a_dt, A.shape), B.tensor_nd(b_dt, Bm.shape)
        d_a, d_b = to_dev(A), to_dev(Bm)
        d_bias = None if bias is None else to_dev(bias)
        n_out = g[name].size
        d_c, d_tmp = dev_zeros(4 * n_out), dev_zeros(1 << 22)
        cs, cd = C.c_float(c_s), TD()
        ok(L.shim_matmul(C.byref(a_desc), dptr(d_a), a_s, ta, C.byref(b_desc), dptr(d_b), b_s, tb, 0 if bias is None else bias.size,
                         None if bias is None else dptr(d_bias), c_dt, C.byref(cs), dptr(d_c), C.byref(cd), dptr(d_tmp), 1 << 22), name)
        ok(B.lib().bolt_b200_synchronize(), "synchronize")
        got = to_host(d_c, g[name].dtype, n_out)
        assert tuple(reversed(list(cd.dims[: cd.nDims]))) == g[name].shape, name
        assert got.tobytes() == g[name].tobytes(), name
        assert np.float32(cs.value).tobytes() == g[name + "_scale"].tobytes(), name
