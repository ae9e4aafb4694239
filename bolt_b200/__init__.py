"""bolt_b200 -- Bolt's quantized-inference hot path on NVIDIA B200, behind Bolt's own operator API.

The product is ``lib/libbolt_b200.so`` (hand-written CUDA for sm_100a, C ABI in
``include/bolt_b200.h``).  This package is the thin Python host side: it loads the library with
ctypes and mirrors the names of Bolt's C/C++ interface (``TensorDesc``, ``tensor2df``,
``matrix_matrix_multiply`` ...) so that tests and benchmarks read like Bolt's own
(compute/blas_enhance/tests/test_mmm.cpp, test_mvm.cpp).

There is no CPU fallback: importing works without a GPU (so that the symbol table can be
checked), but every compute entry point needs the CUDA library and a B200.
"""
import ctypes as C
import os

from . import build as _build

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libbolt_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "bolt_b200.h")

# ---- enums (include/bolt_b200.h; values are Bolt's) ----------------------------------------
SUCCESS, NULL_POINTER, NOT_MATCH, NOT_FOUND, ALLOC_FAILED = 0, 1, 2, 3, 4
NOT_IMPLEMENTED, NOT_SUPPORTED, UNKNOWN = 50, 51, 99
CPU_GENERAL, X86_AVX512, CUDA_B200 = 1, 9, 11
DT_U8, DT_I8, DT_U32, DT_I32, DT_F16, DT_F32 = 0, 1, 2, 3, 4, 6
DT_BIN01, DT_BIN11, DT_F32_8Q, DT_U8_Q = 7, 8, 9, 10
DF_NCHW, DF_NCHWC8, DF_NCHWN16C8, DF_TRANSPOSE, DF_NORMAL = 0, 2, 9, 13, 14
DF_NK, DF_NKN32K4, DF_NKNxKx, DF_NCHWC16, DF_NCHWC2NxC4 = 17, 21, 39, 41, 42
ACTIVATION_NULL, ACTIVATION_RELU = 0, 1
NOALLOC_MAX_ELEMENTS = 67108864  # BOLT_B200_NOALLOC_MAX_ELEMENTS
CONVOLUTION_ALGORITHM_POINTWISE, CONVOLUTION_ALGORITHM_DIRECT = 0, 1
CONVOLUTION_ALGORITHM_BNN, CONVOLUTION_ALGORITHM_NULL = 6, 9

_EE_NAMES = {0: "SUCCESS", 1: "NULL_POINTER", 2: "NOT_MATCH", 3: "NOT_FOUND", 4: "ALLOC_FAILED",
             50: "NOT_IMPLEMENTED", 51: "NOT_SUPPORTED", 52: "GCL_ERROR", 53: "FILE_ERROR", 99: "UNKNOWN"}


class BoltError(RuntimeError):
    """A non-SUCCESS EE code (Bolt's CHECK_STATUS would log it and exit)."""

    def __init__(self, code, what=""):
        self.code = code
        super().__init__("%s returned %s" % (what, _EE_NAMES.get(code, code)))


def CHECK_STATUS(code, what=""):
    if code != SUCCESS:
        raise BoltError(code, what)


class TensorDesc(C.Structure):
    """common/uni/include/tensor_desc.h:93-100; dims[0] is the innermost extent."""
    _pack_ = 8
    _fields_ = [("dt", C.c_uint32), ("df", C.c_uint32), ("nDims", C.c_uint32), ("dims", C.c_uint32 * 20)]

    def __repr__(self):
        return "TensorDesc(dt=%d, df=%d, dims=%s)" % (self.dt, self.df, list(self.dims[: self.nDims]))


def tensor4df(dt, df, n, c, h, w):
    d = TensorDesc()
    d.dt, d.df, d.nDims = dt, df, 4
    d.dims[0], d.dims[1], d.dims[2], d.dims[3] = w, h, c, n
    return d


def tensor2df(dt, df, rows, cols):
    d = tensor4df(dt, df, 1, 1, rows, cols)
    d.nDims = 2
    return d


def tensor1d(dt, length):
    d = tensor4df(dt, DF_NCHW, 1, 1, 1, length)
    d.nDims = 1
    return d


class ActivationParamSpec(C.Structure):
    _pack_ = 8
    _fields_ = [("mode", C.c_uint32), ("value", C.c_float * 4)]


class ConvolutionParamSpec(C.Structure):
    _pack_ = 8
    _fields_ = [(k, C.c_uint32) for k in (
        "num_outputs", "kernel_t", "kernel_h", "kernel_w", "stride_t", "stride_h", "stride_w",
        "pad_before", "pad_after", "pad_top", "pad_bottom", "pad_left", "pad_right", "group",
        "dilatedRate_t", "dilatedRate_h", "dilatedRate_w", "num_outputs_origin", "convolution_type",
        "dw_activation_type", "pw_activation_type")] + [("activation_spec", C.c_float * 2)] + [
        (k, C.c_uint32) for k in ("round_mode", "output_pad_t", "output_pad_h", "output_pad_w")]


class PoolingParamSpec(C.Structure):
    """parameter_spec.h:285-301"""
    _pack_ = 8
    _fields_ = [(k, C.c_uint32) for k in ("kernel_t", "kernel_h", "kernel_w", "stride_t", "stride_h", "stride_w", "pad_before",
                                          "pad_after", "pad_top", "pad_bottom", "pad_left", "pad_right", "round_mode", "mode")] + [
        ("count_include_pad", C.c_bool)]


POOLING_MAX, POOLING_MEAN = 0, 1


class Scatter(C.Structure):
    _fields_ = [("n_dest", C.c_uint32), ("dest", C.c_void_p * 8), ("ld", C.c_uint32), ("col0", C.c_uint32)]


class ConvExt(C.Structure):
    """bolt_b200_conv_ext"""
    _fields_ = [("output_scale", C.c_float), ("filter_scales", C.c_void_p)]


class GemmEpilogue(C.Structure):
    """bolt_b200_gemm_epilogue"""
    _fields_ = [("out_dt", C.c_uint32), ("accumulate", C.c_int), ("out_scale", C.c_float),
                ("sA", C.c_float), ("sB", C.c_float), ("d_sA", C.c_void_p),
                ("row_scale", C.c_void_p), ("col_scale", C.c_void_p), ("col_factor", C.c_void_p),
                ("prefetch", C.c_void_p), ("prefetch_bytes", C.c_size_t)]


_vp, _u32, _u32p, _f32p = C.c_void_p, C.c_uint32, C.POINTER(C.c_uint32), C.POINTER(C.c_float)
_TDp = C.POINTER(TensorDesc)

# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "bolt_b200_set_device": (C.c_int, [C.c_int]),
    "bolt_b200_use_para": (C.c_int, [_vp]),
    "bolt_b200_i8_mma_rate": (C.c_int, [C.c_uint32, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "bolt_b200_selftest_wait_limit": (C.c_int, [C.c_uint32]),
    "bolt_b200_gemm_u8s8_scatter": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, _vp, _vp, _vp, _vp, _vp]),
    "bolt_b200_ipc_export": (C.c_int, [_vp, _vp]),
    "bolt_b200_ipc_import": (C.c_int, [_vp, C.POINTER(C.c_void_p)]),
    "bolt_b200_ipc_close": (C.c_int, [_vp]),
    "pooling_cuda_b200": (C.c_int, [_TDp, _vp, C.POINTER(PoolingParamSpec), _vp, _TDp, _vp]),
    "matmul_infer_output_size_cuda_b200": (C.c_int, [_TDp, C.c_int, _TDp, C.c_int, _TDp]),
    "matmul_infer_forward_tmp_bytes_cuda_b200": (C.c_int, [_TDp, C.c_int, _TDp, C.c_int, _TDp, C.c_float, C.POINTER(C.c_uint32)]),
    "matmul_cuda_b200": (C.c_int, [_TDp, C.c_int, _vp, C.c_float, _TDp, C.c_int, _vp, C.c_float, _TDp, _vp, C.c_uint32, _vp,
                                   _TDp, _vp, C.POINTER(C.c_float)]),
    "bolt_b200_set_stream": (C.c_int, [_vp]),
    "bolt_b200_synchronize": (C.c_int, []),
    "bolt_b200_device_status": (C.c_int, []),
    "bolt_b200_set_pointer_mode": (C.c_int, [C.c_int]),
    "bolt_b200_malloc": (_vp, [C.c_size_t]),
    "bolt_b200_free": (None, [_vp]),
    "bolt_b200_memcpy_h2d": (C.c_int, [_vp, _vp, C.c_size_t]),
    "bolt_b200_memcpy_d2h": (C.c_int, [_vp, _vp, C.c_size_t]),
    "bolt_b200_release_weight": (C.c_int, [_vp]),
    "bolt_b200_launch_count": (C.c_uint64, []),
    "bolt_b200_last_gemm_used_tensor_cores": (C.c_int, []),
    "matrix_matrix_multiply_transform_rhs_bytes_cuda_b200": (C.c_int, [_u32, _u32, _u32, _u32, _u32p, _u32p]),
    "matrix_matrix_multiply_transform_rhs_cuda_b200": (C.c_int, [_TDp, _vp, _TDp, _vp]),
    "matrix_matrix_multiply_tmp_bytes_cuda_b200": (C.c_int, [_u32] * 3 + [_u32] * 4 + [_u32p]),
    "mmm_cuda_b200": (C.c_int, [_u32, _u32, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _f32p]),
    "bolt_b200_gemm_u8s8_ex": (C.c_int, [_u32, _u32, _u32, _vp, _vp, _vp, _vp, C.POINTER(GemmEpilogue)]),
    "bolt_b200_quantize_f32_u8_dev": (C.c_int, [_vp, C.c_uint64, _vp, _vp]),
    "bolt_b200_col_factor": (C.c_int, [C.c_float, C.c_float, _vp, C.c_float, _vp, _u32, _vp]),
    "matrix_vector_multiply_transform_weight_bytes_cuda_b200": (C.c_int, [_u32, _u32, _u32, _u32, _u32p]),
    "matrix_vector_multiply_transform_weight_cuda_b200": (C.c_int, [_TDp, _vp, _TDp, _vp, _vp]),
    "matrix_vector_multiply_tmp_bytes_cuda_b200": (C.c_int, [_u32, _u32, _u32, _u32, _u32p]),
    "mvm_cuda_b200": (C.c_int, [_u32, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _f32p]),
    "quantize_cuda_b200": (C.c_int, [_TDp, _vp, _TDp, _vp, _f32p, C.c_int]),
    "quantize_bias_offsetC_cuda_b200": (C.c_int, [_vp, _TDp, _u32, _vp, _TDp, _f32p, _vp]),
    "dequantize_cuda_b200": (C.c_int, [_TDp, _vp, _f32p, _TDp, _vp, _TDp, _vp]),
    "bolt_b200_absmax_scale_f32": (C.c_int, [_vp, C.c_uint64, _vp]),
    "bolt_b200_quantize_f32_u8_noalloc": (C.c_int, [_vp, C.c_uint64, _vp, _vp]),
    "convolution_infer_output_size_cuda_b200": (
        C.c_int, [_TDp, _TDp, C.POINTER(ConvolutionParamSpec), _TDp, _u32]),
    "convolution_infer_forward_algorithm_cuda_b200": (
        C.c_int, [_TDp, _TDp, _TDp, C.POINTER(ConvolutionParamSpec), _u32, _u32p, _u32]),
    "convolution_transform_filter_bytes_cuda_b200": (
        C.c_int, [_TDp, C.POINTER(ConvolutionParamSpec), _u32, _u32p]),
    "convolution_transform_filter_cuda_b200": (
        C.c_int, [_TDp, _vp, C.POINTER(ConvolutionParamSpec), _u32, _TDp, _vp]),
    "convolution_infer_forward_tmp_bytes_cuda_b200": (
        C.c_int, [_TDp, _TDp, _TDp, C.POINTER(ConvolutionParamSpec), _u32, _u32p]),
    "convolution_cuda_b200": (
        C.c_int, [_TDp, _vp, _vp, _TDp, _vp, C.POINTER(ConvolutionParamSpec), _u32, _TDp, _vp, _TDp, _vp,
                  _u32, _vp, _TDp, _vp, C.POINTER(ActivationParamSpec)]),
    "bolt_b200_convolution_ex": (
        C.c_int, [_TDp, _vp, _vp, _TDp, _vp, C.POINTER(ConvolutionParamSpec), _u32, _TDp, _vp, _TDp, _vp,
                  _u32, _vp, _TDp, _vp, C.POINTER(ActivationParamSpec), C.POINTER(ConvExt)]),
    "b200_matrix_matrix_multiply_tmp_bytes": (C.c_int, [TensorDesc, TensorDesc, _u32p, _u32]),
    "b200_matrix_matrix_multiply": (
        C.c_int, [TensorDesc, _vp, TensorDesc, _vp, _u32, _vp, TensorDesc, _vp, _f32p, _u32]),
    "b200_matrix_matrix_multiply_rhs_format": (_u32, [_u32]),
    "b200_matrix_matrix_multiply_transform_rhs_bytes": (C.c_int, [TensorDesc, _u32p, _u32p, _u32]),
    "b200_matrix_matrix_multiply_transform_rhs": (C.c_int, [TensorDesc, _vp, _TDp, _vp, _u32]),
    "b200_matrix_vector_multiply_tmp_bytes": (C.c_int, [TensorDesc, TensorDesc, _u32p, _u32]),
    "b200_matrix_vector_multiply": (
        C.c_int, [TensorDesc, _vp, TensorDesc, _vp, _u32, _vp, TensorDesc, _vp, _f32p, _u32]),
    "b200_matrix_vector_multiply_weight_format": (_u32, [_u32]),
    "b200_matrix_vector_multiply_transform_weight_bytes": (C.c_int, [TensorDesc, _u32p, _u32]),
    "b200_matrix_vector_multiply_transform_weight": (C.c_int, [TensorDesc, _vp, _TDp, _vp, _u32]),
}

_lib = None


def load(build_if_missing=True):
    """Load libbolt_b200.so (building it first if it is not there).  Raises if it cannot."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        if not build_if_missing:
            raise RuntimeError("libbolt_b200.so is missing; run `python -m bolt_b200.build`")
        _build.build()
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def lib():
    return load()


def _scale_ptr(scale):
    """Bolt's `const F32 *scale`: None -> NULL, else a float array kept alive by the caller."""
    if scale is None:
        return None, None
    arr = (C.c_float * len(scale))(*scale)
    return arr, C.cast(arr, _f32p)


# ---- Bolt-named wrappers over the operator-level entry points ---------------------------------
def matrix_matrix_multiply_tmp_bytes(aDesc, bDesc, arch=CUDA_B200):
    n = C.c_uint32(0)
    CHECK_STATUS(lib().b200_matrix_matrix_multiply_tmp_bytes(aDesc, bDesc, C.byref(n), arch),
                 "matrix_matrix_multiply_tmp_bytes")
    return n.value


def matrix_matrix_multiply_transform_rhs_bytes(desc, arch=CUDA_B200):
    b, r = C.c_uint32(0), C.c_uint32(0)
    CHECK_STATUS(lib().b200_matrix_matrix_multiply_transform_rhs_bytes(desc, C.byref(b), C.byref(r), arch),
                 "matrix_matrix_multiply_transform_rhs_bytes")
    return b.value, r.value


def matrix_matrix_multiply_transform_rhs(desc, src, dst, arch=CUDA_B200):
    out = TensorDesc()
    CHECK_STATUS(lib().b200_matrix_matrix_multiply_transform_rhs(desc, src, C.byref(out), dst, arch),
                 "matrix_matrix_multiply_transform_rhs")
    return out


def matrix_matrix_multiply(aDesc, A, bDesc, B, nbytes, tmp, cDesc, Cptr, scale=None, arch=CUDA_B200):
    keep, sp = _scale_ptr(scale)
    CHECK_STATUS(lib().b200_matrix_matrix_multiply(aDesc, A, bDesc, B, nbytes, tmp, cDesc, Cptr, sp, arch),
                 "matrix_matrix_multiply")


def matrix_vector_multiply_tmp_bytes(mDesc, vDesc, arch=CUDA_B200):
    n = C.c_uint32(0)
    CHECK_STATUS(lib().b200_matrix_vector_multiply_tmp_bytes(mDesc, vDesc, C.byref(n), arch),
                 "matrix_vector_multiply_tmp_bytes")
    return n.value


def matrix_vector_multiply_transform_weight_bytes(desc, arch=CUDA_B200):
    n = C.c_uint32(0)
    CHECK_STATUS(lib().b200_matrix_vector_multiply_transform_weight_bytes(desc, C.byref(n), arch),
                 "matrix_vector_multiply_transform_weight_bytes")
    return n.value


def matrix_vector_multiply_transform_weight(desc, src, dst, arch=CUDA_B200):
    out = TensorDesc()
    CHECK_STATUS(lib().b200_matrix_vector_multiply_transform_weight(desc, src, C.byref(out), dst, arch),
                 "matrix_vector_multiply_transform_weight")
    return out


def matrix_vector_multiply(mDesc, M, vDesc, v, nbytes, tmp, rDesc, r, scale=None, arch=CUDA_B200):
    keep, sp = _scale_ptr(scale)
    CHECK_STATUS(lib().b200_matrix_vector_multiply(mDesc, M, vDesc, v, nbytes, tmp, rDesc, r, sp, arch),
                 "matrix_vector_multiply")


def quantize(dDesc, data, qDesc, qData, scale, mode=0):
    """quantize_x86-shaped: `scale` is a list read and updated in place (1 or 2 floats)."""
    arr = (C.c_float * max(2, len(scale)))(*scale)
    CHECK_STATUS(lib().quantize_cuda_b200(C.byref(dDesc), data, C.byref(qDesc), qData, C.cast(arr, _f32p), mode),
                 "quantize")
    for i in range(len(scale)):
        scale[i] = arr[i]


def dequantize(qDesc, qData, scale, dDesc, dData):
    arr = (C.c_float * 1)(scale)
    b = tensor1d(DT_F32, 0)
    CHECK_STATUS(lib().dequantize_cuda_b200(C.byref(qDesc), qData, C.cast(arr, _f32p), C.byref(b), None,
                                            C.byref(dDesc), dData), "dequantize")


# ---- pooling (u8, NCHWc16) ------------------------------------------------------------------------------
def pooling_param(kernel, stride, pad, mean=False, count_include_pad=False):
    p = PoolingParamSpec()
    p.kernel_t, p.kernel_h, p.kernel_w = 1, kernel, kernel
    p.stride_t, p.stride_h, p.stride_w = 1, stride, stride
    p.pad_top = p.pad_bottom = p.pad_left = p.pad_right = pad
    p.round_mode = 0
    p.mode = POOLING_MEAN if mean else POOLING_MAX
    p.count_include_pad = bool(count_include_pad)
    return p


def pooling(inputDesc, input_ptr, p, scale, outputDesc, output_ptr):
    """scale: list [input scale, output scale]; the output scale is written back"""
    arr = (C.c_float * 2)(*scale)
    CHECK_STATUS(lib().pooling_cuda_b200(C.byref(inputDesc), input_ptr, C.byref(p), C.cast(arr, _vp), C.byref(outputDesc), output_ptr),
                 "pooling")
    scale[0], scale[1] = arr[0], arr[1]


# ---- matmul (compute/tensor/include/tensor_computing.h: matmul_infer_output_size, _tmp_bytes, matmul) -----
def tensor_nd(dt, shape):
    """desc of a row-major array of `shape` (outermost first); Bolt keeps the innermost extent in dims[0]"""
    d = TensorDesc()
    d.dt, d.nDims = dt, len(shape)
    d.df = DF_NORMAL if len(shape) == 2 else DF_NCHW
    for i, s in enumerate(reversed(shape)):
        d.dims[i] = s
    return d


def matmul_infer_output_size(aDesc, transposeA, bDesc, transposeB):
    c = TensorDesc()
    CHECK_STATUS(lib().matmul_infer_output_size_cuda_b200(C.byref(aDesc), int(transposeA), C.byref(bDesc), int(transposeB),
                                                          C.byref(c)), "matmul_infer_output_size")
    return c


def matmul_infer_forward_tmp_bytes(aDesc, transposeA, bDesc, transposeB, cDesc, c_scale):
    n = C.c_uint32(0)
    CHECK_STATUS(lib().matmul_infer_forward_tmp_bytes_cuda_b200(C.byref(aDesc), int(transposeA), C.byref(bDesc), int(transposeB),
                                                                C.byref(cDesc), c_scale, C.byref(n)), "matmul tmp_bytes")
    return n.value


def matmul(aDesc, transposeA, A, a_scale, bDesc, transposeB, Bp, b_scale, bias_desc, bias, tmp_bytes, tmp, cDesc, Cp, c_scale):
    """returns the output tensor's scale after the call (Tensor::get_scale of C)"""
    s = C.c_float(c_scale)
    bd = bias_desc if bias_desc is not None else tensor1d(DT_F32, 0)
    CHECK_STATUS(lib().matmul_cuda_b200(C.byref(aDesc), int(transposeA), A, a_scale, C.byref(bDesc), int(transposeB), Bp, b_scale,
                                        C.byref(bd), bias, tmp_bytes, tmp, C.byref(cDesc), Cp, C.byref(s)), "matmul")
    return s.value


# ---- convolution (compute/tensor/include/tensor_computing.h:26-64) --------------------------
def conv_param(oc, fh, fw, stride=1, pad=0, dilation=1, relu=False):
    """ConvolutionParamSpec for a plain 2-D convolution (group 1)."""
    p = ConvolutionParamSpec()
    p.num_outputs = p.num_outputs_origin = oc
    p.kernel_t, p.kernel_h, p.kernel_w = 1, fh, fw
    p.stride_t, p.stride_h, p.stride_w = 1, stride, stride
    p.pad_top = p.pad_bottom = p.pad_left = p.pad_right = pad
    p.group = 1
    p.dilatedRate_t, p.dilatedRate_h, p.dilatedRate_w = 1, dilation, dilation
    p.pw_activation_type = ACTIVATION_RELU if relu else ACTIVATION_NULL
    return p


def convolution_infer_output_size(inputDesc, filterDesc, p, target_dt):
    """compute/tensor/src/convolution.cpp:28-145 for the CPU layouts: output format NCHWc16 for a
    u8 target with more than 8 output channels, NCHWc8 otherwise (:98-103)."""
    out = TensorDesc()
    CHECK_STATUS(lib().convolution_infer_output_size_cuda_b200(C.byref(inputDesc), C.byref(filterDesc), C.byref(p),
                                                               C.byref(out), target_dt), "convolution_infer_output_size")
    return out


def convolution_infer_forward_algorithm(inputDesc, filterDesc, outputDesc, p, target_dt):
    alg = C.c_uint32(CONVOLUTION_ALGORITHM_NULL)
    CHECK_STATUS(lib().convolution_infer_forward_algorithm_cuda_b200(
        C.byref(inputDesc), C.byref(filterDesc), C.byref(outputDesc), C.byref(p), 1, C.byref(alg), target_dt),
        "convolution_infer_forward_algorithm")
    return alg.value


def convolution_transform_filter_bytes(filterDesc, p, alg):
    n = C.c_uint32(0)
    CHECK_STATUS(lib().convolution_transform_filter_bytes_cuda_b200(C.byref(filterDesc), C.byref(p), alg, C.byref(n)),
                 "convolution_transform_filter_bytes")
    return n.value


def convolution_transform_filter(filterDesc, filter_ptr, p, alg, dst_ptr):
    out = TensorDesc()
    CHECK_STATUS(lib().convolution_transform_filter_cuda_b200(C.byref(filterDesc), filter_ptr, C.byref(p), alg,
                                                              C.byref(out), dst_ptr), "convolution_transform_filter")
    return out


def convolution_infer_forward_tmp_bytes(inputDesc, ftmDesc, outputDesc, p, alg):
    n = C.c_uint32(0)
    CHECK_STATUS(lib().convolution_infer_forward_tmp_bytes_cuda_b200(
        C.byref(inputDesc), C.byref(ftmDesc), C.byref(outputDesc), C.byref(p), alg, C.byref(n)),
        "convolution_infer_forward_tmp_bytes")
    return n.value


def convolution(inputDesc, input_ptr, ftmDesc, filter_ptr, p, alg, scale, bias_ptr, tmp_bytes, tmp_ptr, outputDesc,
                output_ptr, relu=False, eltwise_ptr=None, output_scale=None, filter_scales_ptr=None):
    """`scale`: for int8 a 3-float list {input, output, filter} updated in place (convolution_cpu.hpp:142-157);
    for 1-bit filters a device/host pointer to the fp16 per-channel scales.  `relu`: bool, or an activation
    mode number.  output_scale / filter_scales_ptr: the extension of bolt_b200_convolution_ex."""
    act = ActivationParamSpec()
    act.mode = int(relu) if not isinstance(relu, bool) else (ACTIVATION_RELU if relu else ACTIVATION_NULL)
    sd, bd = tensor1d(DT_F32, 3), tensor1d(DT_F32, outputDesc.dims[2])
    if isinstance(scale, list):
        arr = (C.c_float * len(scale))(*scale)
        sp = C.cast(arr, C.c_void_p)
    else:
        arr, sp = None, scale
    if output_scale is None and filter_scales_ptr is None:
        CHECK_STATUS(lib().convolution_cuda_b200(C.byref(inputDesc), input_ptr, eltwise_ptr, C.byref(ftmDesc), filter_ptr,
                                                 C.byref(p), alg, C.byref(sd), sp, C.byref(bd), bias_ptr, tmp_bytes, tmp_ptr,
                                                 C.byref(outputDesc), output_ptr, C.byref(act)), "convolution")
    else:
        ext = ConvExt()
        ext.output_scale = 0.0 if output_scale is None else float(output_scale)
        ext.filter_scales = filter_scales_ptr
        CHECK_STATUS(lib().bolt_b200_convolution_ex(C.byref(inputDesc), input_ptr, eltwise_ptr, C.byref(ftmDesc), filter_ptr,
                                                    C.byref(p), alg, C.byref(sd), sp, C.byref(bd), bias_ptr, tmp_bytes,
                                                    tmp_ptr, C.byref(outputDesc), output_ptr, C.byref(act), C.byref(ext)),
                     "convolution_ex")
    if arr is not None:
        for i in range(len(scale)):
            scale[i] = arr[i]
