"""TEST INFRASTRUCTURE ONLY -- the CPU checker for the CUDA library.

``oracle.port``   : ctypes handle on ``libbolt_oracle.so`` (scalar C restatement of the
                    reference arithmetic, ``bolt_oracle.c``); builds it with gcc on first use.
``oracle.ref``    : ctypes handle on ``_ref/libbolt_ref.so`` (the reference's own x86
                    AVX512-VNNI sources compiled with ``ref_shim.cpp``) or ``None`` when
                    the library is absent or the host CPU lacks avx512_vnni.
``oracle.ref_bnn``: ctypes handle on ``_ref/libbolt_ref_bnn.so`` (the reference's scalar 1-bit
                    convolution compiled with ``ref_bnn_shim.cpp``) or ``None`` when absent.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of
``bench.py`` may import this package.  The product package ``bolt_b200`` never does.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_c = ctypes
_u32, _i32, _f32p = _c.c_uint32, _c.c_int, _c.POINTER(_c.c_float)
_vp, _u64 = _c.c_void_p, _c.c_uint64


def build_port():
    """Compile the scalar restatement (a second or two of gcc)."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "all"])


def build_ref(bolt_root=None):
    """Compile the reference's own int8 sources (and its scalar 1-bit convolution) from a mounted
    huawei-noah/bolt tree: `bolt_root`, else the BOLT_ROOT environment variable."""
    bolt_root = bolt_root or os.environ.get("BOLT_ROOT")
    if not bolt_root or not os.path.isdir(bolt_root):
        return False
    subprocess.check_call(["make", "-s", "-C", _HERE, "ref", "BOLT_ROOT=" + bolt_root])
    return True


def host_has_avx512_vnni():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return "avx512_vnni" in line.split()
    except OSError:
        pass
    return False


def ptr(a):
    """Raw pointer of a numpy array (or None)."""
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_vp)


class ConvShape(_c.Structure):
    _fields_ = [(k, _u32) for k in (
        "n", "ic", "ih", "iw", "oc", "fh", "fw", "stride_h", "stride_w", "pad_t", "pad_b",
        "pad_l", "pad_r", "dil_h", "dil_w", "cin_block", "cout_block", "relu", "out_u8")]


class BnnShape(_c.Structure):
    _fields_ = [(k, _u32) for k in (
        "n", "ic", "ih", "iw", "oc", "fh", "fw", "stride_h", "stride_w", "pad_t", "pad_b",
        "pad_l", "pad_r", "xnor")]


def _load_port():
    so = os.path.join(_HERE, "libbolt_oracle.so")
    src = os.path.join(_HERE, "bolt_oracle.c")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        build_port()
    lib = _c.CDLL(so)
    lib.oracle_cvt_rne.restype = _c.c_int32
    lib.oracle_cvt_rne.argtypes = [_c.c_float]
    lib.oracle_usat8.restype = _c.c_uint8
    lib.oracle_usat8.argtypes = [_c.c_int32]
    lib.oracle_offsetc.argtypes = [_vp, _u32, _u32, _i32, _vp]
    lib.oracle_gemm_u8s8.argtypes = [_u32, _u32, _u32, _vp, _i32, _vp, _i32, _vp, _vp, _vp]
    lib.oracle_gemv_s8u8.argtypes = [_u32, _u32, _vp, _i32, _vp, _vp, _vp, _vp]
    lib.oracle_gemv_u8s8_row.argtypes = [_u32, _u32, _vp, _i32, _vp, _vp, _vp]
    lib.oracle_scale_f32.restype = _c.c_float
    lib.oracle_scale_f32.argtypes = [_vp, _u64]
    lib.oracle_scale_i32.restype = _c.c_float
    lib.oracle_scale_i32.argtypes = [_vp, _u64]
    lib.oracle_quantize_f32_u8.argtypes = [_vp, _u64, _vp, _vp, _i32]
    lib.oracle_quantize_f32_i8.argtypes = [_vp, _u64, _vp, _vp, _i32]
    lib.oracle_quantize_i32_u8.argtypes = [_vp, _u64, _vp, _vp]
    lib.oracle_quantize_i32_i8.argtypes = [_vp, _u64, _vp, _vp]
    lib.oracle_u8_to_i8.argtypes = [_vp, _u64, _vp]
    lib.oracle_bias_offsetc.argtypes = [_vp, _vp, _u32, _c.c_float, _vp]
    lib.oracle_dequantize_i32_f32.argtypes = [_vp, _u64, _c.c_float, _vp]
    lib.oracle_dequantize_u8_f32.argtypes = [_vp, _u64, _c.c_float, _vp]
    lib.oracle_pooling_u8.argtypes = [_u32] * 12 + [_i32, _i32, _vp, _vp, _vp]
    if hasattr(lib, "oracle_conv_int8"):
        lib.oracle_conv_out_hw.argtypes = [_c.POINTER(ConvShape), _vp, _vp]
        lib.oracle_conv_int8.argtypes = [_c.POINTER(ConvShape), _vp, _vp, _vp, _vp, _vp, _vp, _vp]
    if hasattr(lib, "oracle_bnn_conv"):
        lib.oracle_bnn_conv.argtypes = [_c.POINTER(BnnShape), _vp, _vp, _vp, _vp, _vp, _vp]
        lib.oracle_f32_to_f16.restype = _c.c_uint16
        lib.oracle_f32_to_f16.argtypes = [_c.c_float]
        lib.oracle_f16_to_f32.restype = _c.c_float
        lib.oracle_f16_to_f32.argtypes = [_c.c_uint16]
        lib.oracle_f16_fma.restype = _c.c_uint16
        lib.oracle_f16_fma.argtypes = [_c.c_uint16] * 3
        lib.oracle_i32_to_f16.restype = _c.c_uint16
        lib.oracle_i32_to_f16.argtypes = [_c.c_int32]
    return lib


def _load_ref():
    so = os.path.join(_HERE, "_ref", "libbolt_ref.so")
    if not os.path.exists(so) or not host_has_avx512_vnni():
        return None
    lib = _c.CDLL(so)
    lib.ref_set_threads.argtypes = [_i32]
    lib.ref_get_threads.restype = _i32
    lib.ref_gemm_plan.restype = _vp
    lib.ref_gemm_plan.argtypes = [_u32, _u32, _u32, _i32, _i32, _vp, _i32]
    lib.ref_gemm_run.argtypes = [_vp, _vp, _vp, _vp, _vp]
    lib.ref_gemm_offsetc.argtypes = [_vp, _vp]
    lib.ref_gemm_free.argtypes = [_vp]
    lib.ref_gemm_unpacked.argtypes = [_u32, _u32, _u32, _i32, _i32, _vp, _vp, _vp, _i32, _vp]
    lib.ref_gemv_plan.restype = _vp
    lib.ref_gemv_plan.argtypes = [_u32, _u32, _i32, _vp, _i32]
    lib.ref_gemv_run.argtypes = [_vp, _vp, _vp, _vp, _vp]
    lib.ref_gemv_free.argtypes = [_vp]
    lib.ref_gemv_row.argtypes = [_u32, _u32, _i32, _vp, _vp, _vp, _i32, _vp]
    lib.ref_quantize.argtypes = [_u32, _i32, _vp, _i32, _vp, _vp, _i32]
    lib.ref_dequantize.argtypes = [_u32, _i32, _vp, _vp, _vp]
    lib.ref_bias_offsetc.argtypes = [_u32, _vp, _vp, _c.c_float, _vp]
    lib.ref_conv_plan.restype = _vp
    lib.ref_conv_plan.argtypes = [_u32] * 9 + [_i32] * 4 + [_vp]
    lib.ref_conv_run.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp]
    lib.ref_conv_free.argtypes = [_vp]
    return lib


def _load_ref_bnn():
    so = os.path.join(_HERE, "_ref", "libbolt_ref_bnn.so")
    if not os.path.exists(so):
        return None
    try:
        lib = _c.CDLL(so)
    except OSError:
        return None
    lib.ref_bnn_conv.argtypes = [_u32] * 13 + [_i32] + [_vp] * 5
    return lib


port = _load_port()
ref = _load_ref()
ref_bnn = _load_ref_bnn()

DT_I8, DT_I32, DT_F32, DT_U8_Q = 1, 3, 6, 10
_OUT_DT = {0: np.int32, 1: np.float32, 2: np.uint8}


# ---- convenience wrappers used by the tests (numpy in, numpy out) -----------------------
def _scale_arr(scale):
    return None if scale is None else np.ascontiguousarray(np.asarray(scale, dtype=np.float32))


def out_kind(scale):
    if scale is None:
        return 0
    return 2 if scale[0] < 0 else 1


def port_gemm(A, B, offsetC, scale=None, C_in=None, a_t=False, b_t=False):
    """A u8 [M,K] (or [K,M] if a_t), B s8 [K,N] (or [N,K] if b_t)."""
    M, K = (A.shape[1], A.shape[0]) if a_t else A.shape
    N = B.shape[0] if b_t else B.shape[1]
    kind = out_kind(scale)
    C = np.zeros((M, N), _OUT_DT[kind]) if C_in is None else C_in.copy()
    s = _scale_arr(scale)
    port.oracle_gemm_u8s8(M, N, K, ptr(A), int(a_t), ptr(B), int(b_t), ptr(offsetC), ptr(C), ptr(s))
    return C


def port_offsetc(B, b_t=False):
    N, K = B.shape if b_t else B.shape[::-1]
    out = np.zeros(N, np.int32)
    port.oracle_offsetc(ptr(B), K, N, int(b_t), ptr(out))
    return out


def port_gemv(W, x, offsetC, scale=None, y_in=None, w_t=False):
    N, K = W.shape[::-1] if w_t else W.shape
    kind = out_kind(scale)
    y = np.zeros(N, _OUT_DT[kind]) if y_in is None else y_in.copy()
    s = _scale_arr(scale)
    port.oracle_gemv_s8u8(N, K, ptr(W), int(w_t), ptr(x), ptr(offsetC), ptr(y), ptr(s))
    return y


def ref_gemm(A, B, scale=None, C_in=None, a_t=False, b_t=False, offsetC=None, prepack=True):
    M, K = (A.shape[1], A.shape[0]) if a_t else A.shape
    N = B.shape[0] if b_t else B.shape[1]
    kind = out_kind(scale)
    C = np.zeros((M, N), _OUT_DT[kind]) if C_in is None else C_in.copy()
    s = _scale_arr(scale)
    if not prepack:
        assert offsetC is None
        rc = ref.ref_gemm_unpacked(M, N, K, int(a_t), int(b_t), ptr(A), ptr(B), ptr(C), kind, ptr(s))
        assert rc == 0
        return C
    pl = ref.ref_gemm_plan(M, N, K, int(a_t), int(b_t), ptr(B), kind)
    assert pl
    rc = ref.ref_gemm_run(pl, ptr(A), ptr(C), ptr(s), ptr(offsetC))
    ref.ref_gemm_free(pl)
    assert rc == 0
    return C


def ref_gemv(W, x, scale=None, y_in=None, w_t=False, offsetC=None):
    N, K = W.shape[::-1] if w_t else W.shape
    kind = out_kind(scale)
    y = np.zeros(N, _OUT_DT[kind]) if y_in is None else y_in.copy()
    s = _scale_arr(scale)
    pl = ref.ref_gemv_plan(N, K, int(w_t), ptr(W), kind)
    assert pl
    rc = ref.ref_gemv_run(pl, ptr(x), ptr(y), ptr(s), ptr(offsetC))
    ref.ref_gemv_free(pl)
    assert rc == 0
    return y


def port_gemv_row(Mx, v, scale=None, m_t=False):
    """Mx u8 [N,K] (or [K,N] if m_t), v s8 [K]"""
    N, K = Mx.shape[::-1] if m_t else Mx.shape
    y = np.zeros(N, _OUT_DT[out_kind(scale)])
    s = _scale_arr(scale)
    port.oracle_gemv_u8s8_row(N, K, ptr(Mx), int(m_t), ptr(v), ptr(y), ptr(s))
    return y


def ref_gemv_row(Mx, v, scale=None, m_t=False):
    N, K = Mx.shape[::-1] if m_t else Mx.shape
    kind = out_kind(scale)
    y = np.zeros(N + 64, _OUT_DT[kind])
    s = _scale_arr(scale)
    rc = ref.ref_gemv_row(N, K, int(m_t), ptr(Mx), ptr(v), ptr(y), kind, ptr(s))
    assert rc == 0
    return y[:N].copy()


def _bnn_out_elems(shape):
    n, ic, ih, iw, oc, fh, fw, st, pad = shape
    return n * oc * ((ih + 2 * pad - fh) // st + 1) * ((iw + 2 * pad - fw) // st + 1)


def port_bnn(shape, xnor, xin, wbits, scale, bias):
    """shape (n, ic, ih, iw, oc, fh, fw, stride, pad); xin / scale / bias: binary16 bit patterns;
    returns binary16 bit patterns, NCHWc8."""
    n, ic, ih, iw, oc, fh, fw, st, pad = shape
    s = BnnShape(n, ic, ih, iw, oc, fh, fw, st, st, pad, pad, pad, pad, int(xnor))
    out = np.zeros(_bnn_out_elems(shape), np.uint16)
    port.oracle_bnn_conv(_c.byref(s), ptr(xin), ptr(wbits), ptr(scale), ptr(bias), ptr(out), None)
    return out


def ref_bnn_conv(shape, xnor, xin, wbits, scale, bias):
    """the same through the reference's own scalar code (cpu/general/convolution.cpp)"""
    n, ic, ih, iw, oc, fh, fw, st, pad = shape
    out = np.zeros(_bnn_out_elems(shape), np.uint16)
    rc = ref_bnn.ref_bnn_conv(n, ic, ih, iw, oc, fh, fw, st, st, pad, pad, pad, pad, int(xnor), ptr(xin), ptr(wbits),
                              ptr(scale), ptr(bias), ptr(out))
    assert rc == 0
    return out


# ---- the matmul operator (compute/tensor/src/matmul.cpp:303-557, x86 int8 branch) -------------------
_NP_OF_DT = {DT_F32: np.float32, DT_U8_Q: np.uint8, DT_I8: np.int8}


def _quant_operand(x, dt_in, scale_in, dt_want):
    """matmul.cpp:401-421: an operand that is not of the wanted type is quantized (whole tensor, one scale)"""
    if dt_in == dt_want:
        return x, np.float32(scale_in)
    assert dt_in == DT_F32
    q = np.zeros(x.size, np.uint8 if dt_want == DT_U8_Q else np.int8)
    s = np.array([scale_in], np.float32)
    fn = port.oracle_quantize_f32_u8 if dt_want == DT_U8_Q else port.oracle_quantize_f32_i8
    fn(ptr(np.ascontiguousarray(x.reshape(-1))), x.size, ptr(q), ptr(s), 0)
    return q.reshape(x.shape), s[0]


def port_matmul(A, a_dt, a_scale, tA, B, b_dt, b_scale, tB, bias, c_dt, c_scale):
    """Restatement of the operator from the scalar primitives.  A, B: numpy arrays of rank >= 2 (outermost
    first).  Returns (C, scale of C after the call)."""
    a2 = A.shape[-2:][::-1] if tA else A.shape[-2:]
    b2 = B.shape[-2:][::-1] if tB else B.shape[-2:]
    M, K = a2
    K2, N = b2
    assert K == K2
    nd = max(A.ndim, B.ndim)
    ash = (1,) * (nd - A.ndim) + A.shape
    bsh = (1,) * (nd - B.ndim) + B.shape
    batch = tuple(max(x, y) for x, y in zip(ash[:-2], bsh[:-2]))
    is_mvm = M == 1 or N == 1
    qa_dt, qb_dt = (DT_I8, DT_U8_Q) if is_mvm else (DT_U8_Q, DT_I8)
    qA, sA = _quant_operand(A, a_dt, a_scale, qa_dt)
    qB, sB = _quant_operand(B, b_dt, b_scale, qb_dt)
    scaleO = np.float32(np.float32(1) * sA) * sB
    static_u8 = c_dt == DT_U8_Q and c_scale > 0
    if static_u8:
        scale = [-1.0, float(np.float32(c_scale) / scaleO)]
        prod_dt = np.uint8
    else:
        scale = [float(scaleO)]
        prod_dt = np.float32
    qA = qA.reshape(ash)
    qB = qB.reshape(bsh)
    out = np.zeros(batch + (M, N), prod_dt)
    if bias is not None:
        flat = out.reshape(-1).view(np.uint8)
        bb = np.ascontiguousarray(bias).view(np.uint8)
        flat[:] = np.tile(bb, flat.size // bb.size)
    for idx in np.ndindex(*batch):
        ia = tuple(i if i < d else 0 for i, d in zip(idx, ash[:-2]))
        ib = tuple(i if i < d else 0 for i, d in zip(idx, bsh[:-2]))
        a, b = np.ascontiguousarray(qA[ia]), np.ascontiguousarray(qB[ib])
        c_in = out[idx]
        if M == 1:
            # the u8 matrix is B seen as [N, K]; stored [K, N] unless transposeB
            y = np.ascontiguousarray(c_in.reshape(-1)).copy()
            s = _scale_arr(scale)
            port.oracle_gemv_u8s8_row(N, K, ptr(b), int(not tB), ptr(np.ascontiguousarray(a.reshape(-1))), ptr(y), ptr(s))
            out[idx] = y.reshape(M, N)
        elif N == 1:
            # the s8 matrix is A seen as [M, K]
            offc = port_offsetc(a, not tA)
            y = port_gemv(a, np.ascontiguousarray(b.reshape(-1)), offc, scale, np.ascontiguousarray(c_in.reshape(-1)), w_t=bool(tA))
            out[idx] = y.reshape(M, N)
        else:
            offc = port_offsetc(b, bool(tB))
            cin = c_in if prod_dt is np.uint8 else c_in.view(np.int32)
            r = port_gemm(a, b, offc, scale, np.ascontiguousarray(cin), a_t=bool(tA), b_t=bool(tB))
            out[idx] = r if prod_dt is np.uint8 else r.view(np.float32)
    if c_dt == DT_U8_Q and not static_u8:
        q = np.zeros(out.size, np.uint8)
        s = np.array([c_scale], np.float32)
        port.oracle_quantize_f32_u8(ptr(np.ascontiguousarray(out.reshape(-1))), out.size, ptr(q), ptr(s), 0)
        return q.reshape(out.shape), float(s[0])
    return out, float(c_scale)


def ref_matmul(A, a_dt, a_scale, tA, B, b_dt, b_scale, tB, bias, c_dt, c_scale):
    """The reference's own `matmul` (through ref_matmul_shim.cpp).  Returns (status, C, scale of C)."""
    f = ref.ref_matmul
    f.argtypes = [_i32, _u32, _vp, _c.c_float, _i32, _vp, _i32, _u32, _vp, _c.c_float, _i32, _vp, _u32, _vp,
                  _i32, _c.c_float, _vp, _u64, _vp, _vp, _vp]
    ad = (_u32 * A.ndim)(*A.shape)
    bd = (_u32 * B.ndim)(*B.shape)
    a2 = A.shape[-2:][::-1] if tA else A.shape[-2:]
    b2 = B.shape[-2:][::-1] if tB else B.shape[-2:]
    nd = max(A.ndim, B.ndim)
    batch = tuple(max(x, y) for x, y in zip((1,) * (nd - A.ndim) + A.shape[:-2], (1,) * (nd - B.ndim) + B.shape[:-2]))
    n_out = int(np.prod(batch + (a2[0], b2[1])))
    buf = np.zeros(n_out * 4 + 256, np.uint8)
    cnd, cdims, cs = _u32(), (_u32 * 8)(), _c.c_float()
    rc = f(a_dt, A.ndim, ad, a_scale, int(tA), ptr(A), b_dt, B.ndim, bd, b_scale, int(tB), ptr(B),
           0 if bias is None else bias.size, ptr(bias), c_dt, c_scale, ptr(buf), buf.size, _c.byref(cnd), cdims, _c.byref(cs))
    if rc != 0:
        return rc, None, None
    shape = tuple(cdims[i] for i in range(cnd.value))
    npdt = np.float32 if c_dt == DT_F32 else np.uint8
    return 0, buf[: n_out * np.dtype(npdt).itemsize].view(npdt).reshape(shape).copy(), float(cs.value)
