"""GPU parity of the GEMM / GEMV path, through the C ABI, in the shape of the reference's own
tests (compute/blas_enhance/tests/test_mmm.cpp, test_mvm.cpp): build descs, query the byte
counts, pre-pack (or not), copy offsetC into tmp, multiply, compare bit for bit."""
import ctypes as C
import itertools
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
NP_OF = {B.DT_I32: np.int32, B.DT_F32: np.float32, B.DT_U8_Q: np.uint8}


def out_dt(scale):
    return B.DT_I32 if scale is None else (B.DT_U8_Q if scale[0] < 0 else B.DT_F32)


def mmm_gpu(A, Bm, scale=None, Cin=None, a_t=False, b_t=False, transform=True, host=False):
    """test_mmm.cpp:mmmTestKernel on CUDA_B200; host=True passes host pointers (staged path)."""
    m, k = (A.shape[1], A.shape[0]) if a_t else A.shape
    n = Bm.shape[0] if b_t else Bm.shape[1]
    a_desc = B.tensor2df(B.DT_U8_Q, B.DF_TRANSPOSE, k, m) if a_t else B.tensor2df(B.DT_U8_Q, B.DF_NORMAL, m, k)
    b_desc = B.tensor2df(B.DT_I8, B.DF_TRANSPOSE, n, k) if b_t else B.tensor2df(B.DT_I8, B.DF_NORMAL, k, n)
    cdt = out_dt(scale)
    c_desc = B.tensor2df(cdt, B.DF_NORMAL, m, n)
    npdt = NP_OF[cdt]
    Cbuf = np.zeros((m, n), npdt) if Cin is None else np.ascontiguousarray(Cin).copy()
    keep = []

    def mk(a):
        if host:
            keep.append(a)
            return hptr(a)
        t = to_dev(a)
        keep.append(t)
        return dptr(t)

    pA, pB = mk(A), mk(Bm)
    trans_desc, p_trans, offset = b_desc, pB, 0
    trans_host = None
    if transform:
        nbytes, offset = B.matrix_matrix_multiply_transform_rhs_bytes(b_desc)
        if host:
            trans_host = np.zeros(nbytes, np.uint8)
            p_trans = hptr(trans_host)
        else:
            t = dev_zeros(nbytes)
            keep.append(t)
            p_trans = dptr(t)
        trans_desc = B.matrix_matrix_multiply_transform_rhs(b_desc, pB, p_trans)
        assert trans_desc.df == B.DF_NKNxKx
    nbytes_tmp = B.matrix_matrix_multiply_tmp_bytes(a_desc, trans_desc)
    if host:
        tmp = np.zeros(nbytes_tmp, np.uint8)
        if transform:
            tmp[: 4 * n] = trans_host[offset: offset + 4 * n]   # test_mmm.cpp:83-85
        p_tmp, pC = hptr(tmp), hptr(Cbuf)
    else:
        tmp = dev_zeros(nbytes_tmp)
        if transform:
            tmp[: 4 * n] = keep[-1][offset: offset + 4 * n]
        dC = to_dev(Cbuf)
        p_tmp, pC = dptr(tmp), dptr(dC)
    B.matrix_matrix_multiply(a_desc, pA, trans_desc, p_trans, nbytes_tmp, p_tmp, c_desc, pC, scale)
    B.CHECK_STATUS(B.lib().bolt_b200_synchronize(), "synchronize")
    if host:
        if transform:
            B.lib().bolt_b200_release_weight(p_trans)
        return Cbuf
    return to_host(dC, npdt, m * n).reshape(m, n)


def same_bits(a, b):
    return a.shape == b.shape and a.tobytes() == b.tobytes()


def test_mmm_golden_all_variants():
    g = np.load(os.path.join(GOLD, "gemm.npz"))
    for i in range(len(cases.GEMM_SHAPES)):
        for a_t, b_t in cases.gemm_variants(i):
            A, Bm, Cin = cases.gemm_inputs(i, a_t, b_t)
            key = "g%d_%d%d" % (i, a_t, b_t)
            for transform in (True, False):
                assert same_bits(mmm_gpu(A, Bm, None, Cin, a_t, b_t, transform), g[key + "_s32"]), (key, transform)
            if a_t == 0:
                assert same_bits(mmm_gpu(A, Bm, cases.GEMM_F32_SCALE, None, 0, b_t), g[key + "_f32"]), key
                assert same_bits(mmm_gpu(A, Bm, cases.GEMM_U8_SCALE, None, 0, b_t), g[key + "_u8"]), key


def test_mmm_cover_sweep_vs_oracle():
    """test_mmm.cpp:165-171 sweeps m,k,n in [1,33]; a thinned grid of the same range, 8 variants each."""
    rng = [1, 2, 3, 8, 15, 16, 17, 32, 33]
    bad = []
    for m, k, n in itertools.product(rng, rng, rng):
        for a_t, b_t, transform in itertools.product((0, 1), (0, 1), (True, False)):
            if (m + k + n + a_t + b_t) % 3:   # thin the grid: ~1/3 of 5832 cases
                continue
            seed = (m * 64 + k) * 64 + n
            A = synth.u8(seed, (k, m) if a_t else (m, k))
            Bm = synth.s8(seed + 1, (n, k) if b_t else (k, n))
            Cin = synth.integers(seed + 2, (m, n), -1000, 1000)
            ref = O.port_gemm(A, Bm, O.port_offsetc(Bm, b_t), None, Cin, a_t, b_t)
            if not same_bits(mmm_gpu(A, Bm, None, Cin, a_t, b_t, transform), ref):
                bad.append((m, k, n, a_t, b_t, transform))
    assert not bad, bad[:10]


TC_SHAPES = [(128, 32, 32), (128, 256, 128), (128, 256, 1024), (256, 512, 256), (100, 72, 80), (129, 257, 144),
             (128, 768, 768), (1, 768, 768), (16, 1024, 512), (300, 200, 4112), (512, 96, 2048)]


@pytest.mark.parametrize("m,n,k", TC_SHAPES)
def test_mmm_tensor_core_shapes(m, n, k):
    """K % 16 == 0, A row-major: the tcgen05 kernel.  All three epilogues, accumulate-into-C."""
    A = synth.u8(m + n + k, (m, k))
    Bm = synth.s8(m + n + k + 1, (k, n))
    off = O.port_offsetc(Bm)
    Cin = synth.integers(3, (m, n), -1000, 1000)
    got = mmm_gpu(A, Bm, None, Cin)
    assert B.lib().bolt_b200_last_gemm_used_tensor_cores() == 1
    assert same_bits(got, O.port_gemm(A, Bm, off, None, Cin))
    for sc in ([0.37], [-1, 0.002], [-1, 1.0]):
        assert same_bits(mmm_gpu(A, Bm, sc), O.port_gemm(A, Bm, off, sc)), sc
    Cbits = synth.integers(4, (m, n), -100, 100).view(np.float32)
    assert same_bits(mmm_gpu(A, Bm, [0.5], Cbits), O.port_gemm(A, Bm, off, [0.5], Cbits))


def test_mmm_small_projection_dynamic_quant_fp32_out():
    """The CPU-runnable case: A fp32 [128,768] ~N(0,1) -> dynamic U8_Q, B ~N(0,0.02) -> I8 per tensor,
    pre-packed, fp32 dequantized output; fp32 output within 1e-5 relative (here: bit-equal)."""
    m, k, n = 128, 768, 768
    Af = synth.normal(1, (m, k))
    Bf = synth.normal(2, (k, n), 0.02)
    # oracle
    sa, sb = np.array([-1], np.float32), np.array([-1], np.float32)
    qa, qb = np.zeros(m * k, np.uint8), np.zeros(k * n, np.int8)
    O.port.oracle_quantize_f32_u8(O.ptr(Af), m * k, O.ptr(qa), O.ptr(sa), 0)
    O.port.oracle_quantize_f32_i8(O.ptr(Bf), k * n, O.ptr(qb), O.ptr(sb), 0)
    scaleO = np.float32(sa[0]) * np.float32(sb[0])
    ref = O.port_gemm(qa.reshape(m, k), qb.reshape(k, n), O.port_offsetc(qb.reshape(k, n)), [float(scaleO)])
    # device
    dAf, dBf = to_dev(Af), to_dev(Bf)
    dqa, dqb = dev_zeros(m * k), dev_zeros(k * n)
    s1, s2 = [-1.0], [-1.0]
    B.quantize(B.tensor2df(B.DT_F32, B.DF_NORMAL, m, k), dptr(dAf), B.tensor2df(B.DT_U8_Q, B.DF_NORMAL, m, k), dptr(dqa), s1)
    B.quantize(B.tensor2df(B.DT_F32, B.DF_NORMAL, k, n), dptr(dBf), B.tensor2df(B.DT_I8, B.DF_NORMAL, k, n), dptr(dqb), s2)
    assert np.float32(s1[0]) == sa[0] and np.float32(s2[0]) == sb[0]
    got = mmm_gpu(to_host(dqa, np.uint8, m * k).reshape(m, k), to_host(dqb, np.int8, k * n).reshape(k, n),
                  [float(np.float32(s1[0]) * np.float32(s2[0]))])
    assert same_bits(got, ref)
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=0)


def test_mmm_full_size_rows_sample():
    """Config-2 shape at full size: raw int32 against an exact float64 product, and a sample of rows
    against the oracle through the fused u8 epilogue."""
    m, k, n = 4096, 768, 3072
    A = synth.u8(11, (m, k))
    Bm = synth.s8(12, (k, n))
    off = O.port_offsetc(Bm)
    got = mmm_gpu(A, Bm)
    exact = (A.astype(np.float64) @ Bm.astype(np.float64)).astype(np.int64) + off
    assert np.array_equal(got.astype(np.int64), exact)
    gu8 = mmm_gpu(A, Bm, [-1, 0.0005])
    rows = synth.integers(13, (48,), 0, m)
    assert same_bits(gu8[rows], O.port_gemm(A[rows], Bm, off, [-1, 0.0005]))


def test_mmm_linearity_large():
    """Size-independent property: C(A1) + C(A2) - C(0) == C(A1 + A2) for u8 inputs that do not overflow."""
    m, k, n = 1024, 2048, 1024
    A1 = synth.u8(21, (m, k)) >> 1
    A2 = synth.u8(22, (m, k)) >> 1
    Bm = synth.s8(23, (k, n))
    c1, c2 = mmm_gpu(A1, Bm).astype(np.int64), mmm_gpu(A2, Bm).astype(np.int64)
    c0 = mmm_gpu(np.zeros_like(A1), Bm).astype(np.int64)
    c12 = mmm_gpu((A1 + A2).astype(np.uint8), Bm).astype(np.int64)
    assert np.array_equal(c1 + c2 - c0, c12)


def test_mmm_host_pointers_and_weight_twin():
    """Host buffers (what an unchanged Bolt engine passes): staged in, result staged out; the packed
    weight written to host memory keeps a device twin that later calls find by address."""
    A, Bm, Cin = cases.gemm_inputs(7, 0, 0)
    off = O.port_offsetc(Bm)
    assert same_bits(mmm_gpu(A, Bm, None, Cin, host=True), O.port_gemm(A, Bm, off, None, Cin))
    assert same_bits(mmm_gpu(A, Bm, None, Cin, transform=False, host=True), O.port_gemm(A, Bm, off, None, Cin))
    assert same_bits(mmm_gpu(A, Bm, [-1, 0.004], host=True), O.port_gemm(A, Bm, off, [-1, 0.004]))
    m, k, n = 256, 512, 384
    A, Bm = synth.u8(31, (m, k)), synth.s8(32, (k, n))
    assert same_bits(mmm_gpu(A, Bm, [0.37], host=True), O.port_gemm(A, Bm, O.port_offsetc(Bm), [0.37]))


def test_empty_and_errors():
    lib = B.lib()
    a = B.tensor2df(B.DT_U8_Q, B.DF_NORMAL, 0, 8)
    b = B.tensor2df(B.DT_I8, B.DF_NKNxKx, 8, 4)
    c = B.tensor2df(B.DT_I32, B.DF_NORMAL, 0, 4)
    buf = dev_zeros(256)
    assert lib.b200_matrix_matrix_multiply(a, dptr(buf), b, dptr(buf), 64, dptr(buf), c, dptr(buf), None, B.CUDA_B200) == B.SUCCESS
    a = B.tensor2df(B.DT_U8_Q, B.DF_NORMAL, 4, 8)
    c = B.tensor2df(B.DT_I32, B.DF_NORMAL, 4, 4)
    assert lib.b200_matrix_matrix_multiply(a, dptr(buf), b, dptr(buf), 64, None, c, dptr(buf), None, B.CUDA_B200) == B.NULL_POINTER
    f = B.tensor2df(B.DT_F32, B.DF_NORMAL, 4, 8)
    fb = B.tensor2df(B.DT_F32, B.DF_NORMAL, 8, 4)
    assert lib.b200_matrix_matrix_multiply(f, dptr(buf), fb, dptr(buf), 64, dptr(buf), c, dptr(buf), None, B.CUDA_B200) == B.NOT_SUPPORTED


def test_gemm_ex_per_channel_and_per_token():
    """Extension (no Bolt counterpart): per-channel / per-token scales.  Accumulators are pinned by
    the cases above; the epilogue is checked against its definition and, with uniform scales,
    against the reference's per-tensor result bit for bit."""
    m, k, n = 200, 256, 176
    A, Bm = synth.u8(41, (m, k)), synth.s8(42, (k, n))
    off = O.port_offsetc(Bm)
    acc = O.port_gemm(A, Bm, off)
    lib = B.lib()
    bdesc = B.tensor2df(B.DT_I8, B.DF_NORMAL, k, n)
    nbytes, rhs = B.matrix_matrix_multiply_transform_rhs_bytes(bdesc)
    dB, dP, dA = to_dev(Bm), dev_zeros(nbytes), to_dev(A)
    B.matrix_matrix_multiply_transform_rhs(bdesc, dptr(dB), dptr(dP))
    sA, sB, so = np.float32(3.7), np.float32(211.0), np.float32(0.9)
    col = (np.abs(synth.normal(43, (n,))) + np.float32(50)).astype(np.float32)
    row = (np.abs(synth.normal(44, (m,))) + np.float32(2)).astype(np.float32)
    dcol, drow = to_dev(col), to_dev(row)

    def run(out_dt, use_row, use_col):
        ep = B.GemmEpilogue()
        ep.out_dt, ep.accumulate, ep.out_scale, ep.sA, ep.sB = out_dt, 0, float(so), float(sA), float(sB)
        ep.row_scale = dptr(drow) if use_row else None
        ep.col_scale = dptr(dcol) if use_col else None
        dC = dev_zeros(m * n * 4)
        B.CHECK_STATUS(lib.bolt_b200_gemm_u8s8_ex(n, m, k, dptr(dA), dptr(dP), dptr(dP, rhs), dptr(dC), C.byref(ep)))
        return to_host(dC, NP_OF[out_dt], m * n).reshape(m, n)

    for use_row, use_col in itertools.product((False, True), (False, True)):
        ra = row[:, None] if use_row else np.full((m, 1), sA, np.float32)
        cb = col[None, :] if use_col else np.full((1, n), sB, np.float32)
        prod = (ra * cb).astype(np.float32)
        f_fac = (np.float32(1.0) / prod).astype(np.float32)
        u_fac = (so / prod).astype(np.float32)
        exp_f = (acc.astype(np.float32) * f_fac).astype(np.float32)
        assert same_bits(run(B.DT_F32, use_row, use_col), exp_f), (use_row, use_col)
        r = np.rint((acc.astype(np.float32) * u_fac).astype(np.float32)).astype(np.int64) + 128
        exp_u = np.where(r < 0, 255, np.minimum(r, 255)).astype(np.uint8)
        assert same_bits(run(B.DT_U8_Q, use_row, use_col), exp_u), (use_row, use_col)
    # uniform scales == the reference's per-tensor epilogues
    assert same_bits(run(B.DT_F32, False, False), O.port_gemm(A, Bm, off, [float(sA * sB)]))
    assert same_bits(run(B.DT_U8_Q, False, False), O.port_gemm(A, Bm, off, [-1, float(so / (sA * sB))]))
    assert same_bits(run(B.DT_I32, False, False), acc)


# ------------------------------------------------------------------------------------ GEMV
def mvm_gpu(W, x, scale=None, yin=None, w_t=False, transform=True, host=False):
    """test_mvm.cpp:mvmTestKernel on CUDA_B200."""
    n, k = W.shape[::-1] if w_t else W.shape
    m_desc = B.tensor2df(B.DT_I8, B.DF_TRANSPOSE, k, n) if w_t else B.tensor2df(B.DT_I8, B.DF_NORMAL, n, k)
    v_desc = B.tensor1d(B.DT_U8_Q, k)
    rdt = out_dt(scale)
    r_desc = B.tensor1d(rdt, n)
    npdt = NP_OF[rdt]
    y = np.zeros(n, npdt) if yin is None else yin.copy()
    al = lambda v, a: (v + a - 1) // a * a
    if host:
        pW, px, py = hptr(W), hptr(x), hptr(y)
        trans_desc, p_trans = m_desc, pW
        if transform:
            nb = B.matrix_vector_multiply_transform_weight_bytes(m_desc)
            th = np.zeros(nb, np.uint8)
            p_trans = hptr(th)
            trans_desc = B.matrix_vector_multiply_transform_weight(m_desc, pW, p_trans)
        nbt = B.matrix_vector_multiply_tmp_bytes(trans_desc, v_desc)
        tmp = np.zeros(nbt + 64, np.uint8)
        if transform:
            o = al(n, 16) * al(k, 8)
            tmp[: 4 * n] = th[o: o + 4 * n]          # test_mvm.cpp:85
        B.matrix_vector_multiply(trans_desc, p_trans, v_desc, px, nbt, hptr(tmp), r_desc, py, scale)
        if transform:
            B.lib().bolt_b200_release_weight(p_trans)
        return y
    dW, dx, dy = to_dev(W), to_dev(x), to_dev(y)
    trans_desc, p_trans = m_desc, dptr(dW)
    if transform:
        nb = B.matrix_vector_multiply_transform_weight_bytes(m_desc)
        dT = dev_zeros(nb)
        p_trans = dptr(dT)
        trans_desc = B.matrix_vector_multiply_transform_weight(m_desc, dptr(dW), p_trans)
        assert trans_desc.df == B.DF_NKN32K4
    nbt = B.matrix_vector_multiply_tmp_bytes(trans_desc, v_desc)
    tmp = dev_zeros(nbt + 64)
    if transform:
        o = al(n, 16) * al(k, 8)
        tmp[: 4 * n] = dT[o: o + 4 * n]
    B.matrix_vector_multiply(trans_desc, p_trans, v_desc, dptr(dx), nbt, dptr(tmp), r_desc, dptr(dy), scale)
    B.CHECK_STATUS(B.lib().bolt_b200_synchronize(), "synchronize")
    return to_host(dy, npdt, n)


def test_mvm_golden():
    g = np.load(os.path.join(GOLD, "gemv.npz"))
    for i in range(len(cases.GEMV_SHAPES)):
        for w_t in (0, 1):
            W, x, yin = cases.gemv_inputs(i, w_t)
            key = "v%d_%d" % (i, w_t)
            for transform in (True, False):
                assert same_bits(mvm_gpu(W, x, None, yin, w_t, transform), g[key + "_s32"]), (key, transform)
            assert same_bits(mvm_gpu(W, x, cases.GEMM_F32_SCALE, None, w_t), g[key + "_f32"]), key
            assert same_bits(mvm_gpu(W, x, cases.GEMM_U8_SCALE, None, w_t), g[key + "_u8"]), key
    W, x, yin = cases.gemv_inputs(5, 0)
    assert same_bits(mvm_gpu(W, x, None, yin, host=True), g["v5_0_s32"])
    assert same_bits(mvm_gpu(W, x, None, yin, transform=False, host=True), g["v5_0_s32"])


def test_mvm_cover_sweep_vs_oracle():
    """test_mvm.cpp:134-172 sweeps m,k in [1,65]."""
    bad = []
    for n, k in itertools.product([1, 2, 7, 8, 9, 16, 31, 33, 48, 64, 65], [1, 3, 4, 8, 15, 16, 17, 32, 64, 65]):
        for w_t in (0, 1):
            W = synth.s8(n * 4096 + k, (k, n) if w_t else (n, k))
            x = synth.u8(n * 4096 + k + 1, (k,))
            yin = synth.integers(5, (n,), -1000, 1000)
            off = O.port_offsetc(W, not w_t)
            for sc in (None, [0.37], [-1, 0.01]):
                yi = yin if sc is None else None
                if not same_bits(mvm_gpu(W, x, sc, yi, w_t), O.port_gemv(W, x, off, sc, yi, w_t)):
                    bad.append((n, k, w_t, sc))
    assert not bad, bad[:10]


def test_mvm_large_vs_oracle():
    """An FFN-shaped slice: K = 8192, N = 4096 (1/7 of the FFN's 28672 columns), all epilogues."""
    n, k = 4096, 8192
    W, x = synth.s8(51, (n, k)), synth.u8(52, (k,))
    off = O.port_offsetc(W, True)
    for sc in (None, [0.37], [-1, 0.0004]):
        assert same_bits(mvm_gpu(W, x, sc), O.port_gemv(W, x, off, sc)), sc


# ------------------------------------------------------- u8 matrix x s8 vector (matmul's GEMV)
def mvm_row_gpu(Mx, v, scale=None, m_t=False, host=False):
    n, k = Mx.shape[::-1] if m_t else Mx.shape
    m_desc = B.tensor2df(B.DT_U8_Q, B.DF_TRANSPOSE, k, n) if m_t else B.tensor2df(B.DT_U8_Q, B.DF_NORMAL, n, k)
    v_desc = B.tensor1d(B.DT_I8, k)
    rdt = out_dt(scale)
    r_desc = B.tensor1d(rdt, n)
    npdt = NP_OF[rdt]
    nbt = B.matrix_vector_multiply_tmp_bytes(m_desc, v_desc)
    if host:
        y, tmp = np.zeros(n, npdt), np.zeros(nbt + 64, np.uint8)
        B.matrix_vector_multiply(m_desc, hptr(Mx), v_desc, hptr(v), nbt, hptr(tmp), r_desc, hptr(y), scale)
        return y
    dM, dv, dy, tmp = to_dev(Mx), to_dev(v), dev_zeros(n * 4), dev_zeros(nbt + 64)
    B.matrix_vector_multiply(m_desc, dptr(dM), v_desc, dptr(dv), nbt, dptr(tmp), r_desc, dptr(dy), scale)
    B.CHECK_STATUS(B.lib().bolt_b200_synchronize(), "synchronize")
    return to_host(dy, npdt, n)


def test_mvm_row_golden_and_sweep():
    g = np.load(os.path.join(GOLD, "gemv_row.npz"))
    for i in range(len(cases.GEMV_ROW_SHAPES)):
        for m_t in (0, 1):
            Mx, v = cases.gemv_row_inputs(i, m_t)
            key = "r%d_%d" % (i, m_t)
            assert same_bits(mvm_row_gpu(Mx, v, None, m_t), g[key + "_s32"]), key
            assert same_bits(mvm_row_gpu(Mx, v, cases.GEMM_F32_SCALE, m_t), g[key + "_f32"]), key
            assert same_bits(mvm_row_gpu(Mx, v, cases.GEMM_U8_SCALE, m_t), g[key + "_u8"]), key
    Mx, v = cases.gemv_row_inputs(5, 0)
    assert same_bits(mvm_row_gpu(Mx, v, None, host=True), g["r5_0_s32"])
    bad = []
    for n, k in itertools.product([1, 2, 5, 8, 13, 16, 33, 64, 65], [1, 4, 15, 16, 48, 100, 512]):
        for m_t in (0, 1):
            Mx, v = synth.u8(n * 977 + k, (k, n) if m_t else (n, k)), synth.s8(n * 31 + k, (k,))
            for sc in (None, [0.37], [-1, 0.002], [-1, 0.05]):
                if not same_bits(mvm_row_gpu(Mx, v, sc, m_t), O.port_gemv_row(Mx, v, sc, m_t)):
                    bad.append((n, k, m_t, sc))
    assert not bad, bad[:10]
    Mx, v = synth.u8(1, (2048, 4096)), synth.s8(2, (4096,))
    assert same_bits(mvm_row_gpu(Mx, v, [-1, 0.0005]), O.port_gemv_row(Mx, v, [-1, 0.0005]))


@pytest.mark.parametrize("n,per_token", [(256, True), (512, True), (768, False), (288, True), (96, False)])
def test_gemm_scatter_into_wider_matrices(n, per_token):
    """The scatter epilogue on one GPU: a [M, n] product stored at column 128 of two [M, 1024] matrices (the fused
    all-gather of the N-split, with both destinations local).  The columns must equal the plain u8 GEMM, everything
    else must stay as it was.  n a multiple of 256: boxes of 128-byte rows assembled by the four warps of a lane
    quadrant; other n: one 32-byte-row box per warp."""
    import torch

    m, k, ld, col0 = 300, 512, 1024, 128
    A, W = synth.u8(61, (m, k)), synth.s8(62, (k, n))
    bdesc = B.tensor2df(B.DT_I8, B.DF_NORMAL, k, n)
    nbytes, rhs = B.matrix_matrix_multiply_transform_rhs_bytes(bdesc)
    d_a, d_w, d_pack = to_dev(A), to_dev(W), dev_zeros(nbytes)
    B.matrix_matrix_multiply_transform_rhs(bdesc, dptr(d_w), dptr(d_pack))
    sB = (np.abs(synth.normal(63, (n,))) * 300 + 900).astype(np.float32)
    rs = (np.abs(synth.normal(64, (m,))) * 10 + 30).astype(np.float32)
    d_sb, d_rs = to_dev(sB), to_dev(rs)
    ep = B.GemmEpilogue()
    ep.out_dt, ep.accumulate, ep.out_scale, ep.sA, ep.sB = B.DT_U8_Q, 0, 40.0, 35.0, 1.0
    ep.row_scale, ep.col_scale = (dptr(d_rs) if per_token else None), dptr(d_sb)
    plain = dev_zeros(m * n)
    B.CHECK_STATUS(B.lib().bolt_b200_gemm_u8s8_ex(n, m, k, dptr(d_a), dptr(d_pack), dptr(d_pack, rhs), dptr(plain), C.byref(ep)))
    wide = [torch.full((m * ld,), 7, dtype=torch.uint8, device="cuda") for _ in range(2)]
    sc = B.Scatter()
    sc.n_dest, sc.ld, sc.col0 = 2, ld, col0
    sc.dest[0], sc.dest[1] = wide[0].data_ptr(), wide[1].data_ptr()
    for _ in range(2):   # twice: the staging boxes are reused across launches
        B.CHECK_STATUS(B.lib().bolt_b200_gemm_u8s8_scatter(n, m, k, dptr(d_a), dptr(d_pack), dptr(d_pack, rhs), C.byref(ep), C.byref(sc)))
    B.CHECK_STATUS(B.lib().bolt_b200_synchronize(), "synchronize")
    assert B.lib().bolt_b200_last_gemm_used_tensor_cores() == 1
    want = np.full((m, ld), 7, np.uint8)
    want[:, col0:col0 + n] = to_host(plain, np.uint8, m * n).reshape(m, n)
    assert len(np.unique(want[:, col0:col0 + n])) > 50      # a result with content, not a saturated one
    for wd in wide:
        assert np.array_equal(wd.cpu().numpy().reshape(m, ld), want)
    # refused: a column offset that is not a multiple of 32, a destination count beyond 8
    sc.col0 = 100
    assert B.lib().bolt_b200_gemm_u8s8_scatter(n, m, k, dptr(d_a), dptr(d_pack), dptr(d_pack, rhs), C.byref(ep), C.byref(sc)) == B.NOT_SUPPORTED
    sc.col0, sc.n_dest = col0, 9
    assert B.lib().bolt_b200_gemm_u8s8_scatter(n, m, k, dptr(d_a), dptr(d_pack), dptr(d_pack, rhs), C.byref(ep), C.byref(sc)) == B.NOT_SUPPORTED


def test_gemm_scatter_long_k_pairs():
    """K = 4096 and M = 512: the CTA-pair kernel with the 128-byte-row scatter"""
    import torch

    m, k, n, ld, col0 = 512, 4096, 512, 1024, 512
    A, W = synth.u8(71, (m, k)), synth.s8(72, (k, n))
    bdesc = B.tensor2df(B.DT_I8, B.DF_NORMAL, k, n)
    nbytes, rhs = B.matrix_matrix_multiply_transform_rhs_bytes(bdesc)
    d_a, d_w, d_pack = to_dev(A), to_dev(W), dev_zeros(nbytes)
    B.matrix_matrix_multiply_transform_rhs(bdesc, dptr(d_w), dptr(d_pack))
    sB = (np.abs(synth.normal(73, (n,))) * 300 + 900).astype(np.float32)
    d_sb = to_dev(sB)
    ep = B.GemmEpilogue()
    ep.out_dt, ep.accumulate, ep.out_scale, ep.sA, ep.sB = B.DT_U8_Q, 0, 40.0, 100.0, 1.0
    ep.row_scale, ep.col_scale = None, dptr(d_sb)
    plain = dev_zeros(m * n)
    B.CHECK_STATUS(B.lib().bolt_b200_gemm_u8s8_ex(n, m, k, dptr(d_a), dptr(d_pack), dptr(d_pack, rhs), dptr(plain), C.byref(ep)))
    wide = torch.full((m * ld,), 9, dtype=torch.uint8, device="cuda")
    sc = B.Scatter()
    sc.n_dest, sc.ld, sc.col0 = 1, ld, col0
    sc.dest[0] = wide.data_ptr()
    B.CHECK_STATUS(B.lib().bolt_b200_gemm_u8s8_scatter(n, m, k, dptr(d_a), dptr(d_pack), dptr(d_pack, rhs), C.byref(ep), C.byref(sc)))
    B.CHECK_STATUS(B.lib().bolt_b200_synchronize(), "synchronize")
    want = np.full((m, ld), 9, np.uint8)
    want[:, col0:col0 + n] = to_host(plain, np.uint8, m * n).reshape(m, n)
    assert np.array_equal(wide.cpu().numpy().reshape(m, ld), want)
