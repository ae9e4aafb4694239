"""The C-ABI library loads without a GPU and exports every symbol include/bolt_b200.h declares;
the byte-count and format entry points (pure host arithmetic) follow the reference's formulas."""
import ctypes as C
import os

import pytest
import re

import bolt_b200 as B


def declared_functions():
    text = open(B.HEADER_PATH).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = text[text.index('extern "C"'):]
    names = re.findall(r"\b(?:EE|int|void|void \*|uint64_t|DataFormat)\s*\*?\s*([A-Za-z_][A-Za-z0-9_]*)\s*\(", text)
    return sorted(set(names))


def test_every_declared_symbol_is_exported():
    lib = B.load()
    names = declared_functions()
    assert len(names) >= 35
    for n in names:
        assert hasattr(lib, n), "libbolt_b200.so lacks %s" % n
        assert n in B.SIGNATURES, "python binding table lacks %s" % n
    assert sorted(B.SIGNATURES) == names


def test_struct_layouts_match_bolt():
    assert C.sizeof(B.TensorDesc) == 92          # common/uni/include/tensor_desc.h:93-100
    assert C.sizeof(B.ConvolutionParamSpec) == 108
    assert C.sizeof(B.ActivationParamSpec) == 20


def test_gemm_byte_counts():
    """mmm_avx512_vnni.cpp:22-58"""
    lib = B.load()
    b, r = C.c_uint32(), C.c_uint32()
    for N, K in [(768, 768), (3072, 768), (33, 17), (1, 1), (28672, 8192)]:
        assert lib.matrix_matrix_multiply_transform_rhs_bytes_cuda_b200(N, K, B.DT_I8, B.DF_NORMAL, C.byref(b), C.byref(r)) == 0
        al = lambda x, a: (x + a - 1) // a * a
        assert r.value == al(N, 16) * al(K, 8)
        assert b.value == r.value + 4 * N + 64
        assert lib.matrix_matrix_multiply_transform_rhs_bytes_cuda_b200(N, K, B.DT_I8, B.DF_NKNxKx, C.byref(b), C.byref(r)) == 0
        assert (b.value, r.value) == (0, 0)
    d = B.tensor2df(B.DT_I8, B.DF_TRANSPOSE, 48, 40)   # [N=48, K=40]
    assert B.matrix_matrix_multiply_transform_rhs_bytes(d) == (48 * 40 + 4 * 48 + 64, 48 * 40)
    assert lib.b200_matrix_matrix_multiply_rhs_format(B.DT_I8) == B.DF_NKNxKx
    assert lib.b200_matrix_vector_multiply_weight_format(B.DT_I8) == B.DF_NKN32K4
    assert lib.b200_matrix_vector_multiply_weight_format(B.DT_U8_Q) == B.DF_NK


def test_gemv_byte_counts():
    """cpu/x86/mvm.cpp:23-41"""
    d = B.tensor2df(B.DT_I8, B.DF_NORMAL, 100, 33)
    assert B.matrix_vector_multiply_transform_weight_bytes(d) == 100 * 4 + 112 * 40 + 32
    d.df = B.DF_NKN32K4
    assert B.matrix_vector_multiply_transform_weight_bytes(d) == 400


def test_wrong_arch_and_type_are_refused():
    lib = B.load()
    n = C.c_uint32()
    a = B.tensor2df(B.DT_U8_Q, B.DF_NORMAL, 4, 8)
    b = B.tensor2df(B.DT_I8, B.DF_NORMAL, 8, 4)
    assert lib.b200_matrix_matrix_multiply_tmp_bytes(a, b, C.byref(n), B.X86_AVX512) == B.NOT_SUPPORTED
    assert lib.b200_matrix_matrix_multiply_tmp_bytes(a, b, C.byref(n), B.CUDA_B200) == B.SUCCESS
    f = B.tensor2df(B.DT_F32, B.DF_NORMAL, 8, 4)
    assert lib.b200_matrix_matrix_multiply_transform_rhs_bytes(f, C.byref(n), C.byref(n), B.CUDA_B200) == B.NOT_SUPPORTED
    # argument checks of mmm.cpp:161-197 come before anything touches the device
    c = B.tensor2df(B.DT_I32, B.DF_NORMAL, 4, 4)
    assert lib.b200_matrix_matrix_multiply(a, None, b, None, 0, None, c, None, None, B.CUDA_B200) == B.NULL_POINTER
    bad = B.tensor2df(B.DT_I32, B.DF_NORMAL, 5, 4)
    buf = C.create_string_buffer(256)
    p = C.cast(buf, C.c_void_p)
    assert lib.b200_matrix_matrix_multiply(a, p, b, p, 64, p, bad, p, None, B.CUDA_B200) == B.NOT_MATCH


def test_convolution_geometry_is_checked_before_any_launch():
    """An output descriptor that does not follow from input, filter, stride and padding is refused with
    NOT_MATCH by the byte-count entry points (host arithmetic only), for the int8 and the 1-bit path."""
    lib = B.load()
    n = C.c_uint32()
    p = B.conv_param(16, 3, 3, 1, 1)
    x = B.tensor4df(B.DT_U8_Q, B.DF_NCHWC16, 2, 16, 8, 8)
    f = B.tensor4df(B.DT_I8, B.DF_NCHWC2NxC4, 16, 16, 3, 3)
    good = B.tensor4df(B.DT_F32, B.DF_NCHWC8, 2, 16, 8, 8)
    assert lib.convolution_infer_forward_tmp_bytes_cuda_b200(C.byref(x), C.byref(f), C.byref(good), C.byref(p), 1, C.byref(n)) == B.SUCCESS
    for bad in (B.tensor4df(B.DT_F32, B.DF_NCHWC8, 2, 16, 9, 8), B.tensor4df(B.DT_F32, B.DF_NCHWC8, 2, 16, 8, 12),
                B.tensor4df(B.DT_F32, B.DF_NCHWC8, 3, 16, 8, 8)):
        assert lib.convolution_infer_forward_tmp_bytes_cuda_b200(C.byref(x), C.byref(f), C.byref(bad), C.byref(p), 1, C.byref(n)) == B.NOT_MATCH
    xb = B.tensor4df(B.DT_F16, B.DF_NCHWC8, 2, 32, 8, 8)
    fb = B.tensor4df(B.DT_BIN11, B.DF_NCHWN16C8, 16, 32, 3, 3)
    pb = B.conv_param(16, 3, 3, 1, 1)
    ok = B.tensor4df(B.DT_F16, B.DF_NCHWC8, 2, 16, 8, 8)
    assert lib.convolution_infer_forward_tmp_bytes_cuda_b200(C.byref(xb), C.byref(fb), C.byref(ok), C.byref(pb), 6, C.byref(n)) == B.SUCCESS
    for bad in (B.tensor4df(B.DT_F16, B.DF_NCHWC8, 2, 16, 10, 8), B.tensor4df(B.DT_F16, B.DF_NCHWC8, 1, 16, 8, 8)):
        assert lib.convolution_infer_forward_tmp_bytes_cuda_b200(C.byref(xb), C.byref(fb), C.byref(bad), C.byref(pb), 6, C.byref(n)) == B.NOT_MATCH


def test_infer_output_size_rule():
    """convolution.cpp:28-108"""
    x = B.tensor4df(B.DT_U8_Q, B.DF_NCHWC16, 2, 64, 56, 56)
    f = B.tensor4df(B.DT_I8, B.DF_NCHW, 128, 64, 3, 3)
    o = B.convolution_infer_output_size(x, f, B.conv_param(128, 3, 3, 2, 1), B.DT_U8_Q)
    assert list(o.dims[:4]) == [28, 28, 128, 2] and o.df == B.DF_NCHWC16 and o.dt == B.DT_U8_Q
    o = B.convolution_infer_output_size(x, f, B.conv_param(128, 3, 3, 1, 0, 2), B.DT_F32)
    assert list(o.dims[:4]) == [52, 52, 128, 2] and o.df == B.DF_NCHWC8
    f8 = B.tensor4df(B.DT_I8, B.DF_NCHW, 8, 64, 1, 1)
    assert B.convolution_infer_output_size(x, f8, B.conv_param(8, 1, 1), B.DT_U8_Q).df == B.DF_NCHWC8
    f12 = B.tensor4df(B.DT_I8, B.DF_NCHW, 12, 64, 1, 1)
    try:
        B.convolution_infer_output_size(x, f12, B.conv_param(12, 1, 1), B.DT_U8_Q)
        assert False
    except B.BoltError as e:
        assert e.code == B.NOT_SUPPORTED


def _abi_values(tmp_path, extra):
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / ("abi" + str(len(extra))))
    subprocess.check_call(["g++", "-std=c++11", "-w", "-I", os.path.join(root, "include")] + extra +
                          [os.path.join(root, "integration", "abi_print.cpp"), "-o", exe])
    return subprocess.check_output([exe]).decode()


def test_header_types_match_bolts_headers(tmp_path):
    """Sizes, field offsets and enumerator values of everything that crosses the C ABI: the stand-in typedefs of
    include/bolt_b200.h against the values printed by the same program built on Bolt's own headers
    (common/uni/include: sys.h, error.h, tensor_desc.h, parameter_spec.h), kept in golden/abi_values.txt."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(root, "tests", "golden", "abi_values.txt")) as f:
        pinned = f.read()
    assert _abi_values(tmp_path, []) == pinned
    bolt_root = os.environ.get("BOLT_ROOT") or os.path.join(os.path.dirname(root), "reference")
    uni = os.path.join(bolt_root, "common", "uni", "include")
    if os.path.isdir(uni):
        # the fixture itself is still what Bolt's headers say
        assert _abi_values(tmp_path, ["-include", "cstdint", "-DBOLT_B200_WITH_BOLT_HEADERS", "-I", uni]) == pinned
    # the ctypes mirrors used by the Python host side
    import bolt_b200 as B
    vals = dict(line.split(" = ") for line in pinned.strip().splitlines())
    assert C.sizeof(B.TensorDesc) == int(vals["sizeof(TensorDesc)"])
    assert C.sizeof(B.ConvolutionParamSpec) == int(vals["sizeof(ConvolutionParamSpec)"])
    assert C.sizeof(B.ActivationParamSpec) == int(vals["sizeof(ActivationParamSpec)"])
    assert B.ConvolutionParamSpec.round_mode.offset == int(vals["offsetof(ConvolutionParamSpec, round_mode)"])
    for name in ("DT_U8_Q", "DT_I8", "DT_I32", "DT_F32", "DT_BIN01", "DT_BIN11", "DF_NCHWC8", "DF_NCHWC16", "DF_NKN32K4",
                 "DF_NKNxKx", "DF_NCHWC2NxC4", "DF_TRANSPOSE", "DF_NORMAL", "CONVOLUTION_ALGORITHM_POINTWISE",
                 "CONVOLUTION_ALGORITHM_DIRECT", "CONVOLUTION_ALGORITHM_BNN"):
        assert getattr(B, name) == int(vals[name]), name


def test_matmul_output_size_is_host_arithmetic():
    """matmul_infer_output_size_cpu (matmul.cpp:42-99): transposes, broadcast batch dimensions, rank alignment"""
    F = B.DT_F32
    cases_ = [(((2, 3, 40, 64), 0, (2, 3, 64, 24), 0), (2, 3, 40, 24)), (((2, 3, 64, 40), 1, (2, 3, 24, 64), 1), (2, 3, 40, 24)),
              (((2, 3, 40, 64), 0, (1, 1, 64, 24), 0), (2, 3, 40, 24)), (((2, 3, 40, 64), 0, (64, 24), 0), (2, 3, 40, 24)),
              (((1, 33, 50), 0, (5, 50, 17), 0), (5, 33, 17))]
    for (a, ta, b, tb), want in cases_:
        c = B.matmul_infer_output_size(B.tensor_nd(F, a), ta, B.tensor_nd(F, b), tb)
        assert tuple(reversed(list(c.dims[: c.nDims]))) == want, (a, b)
    with pytest.raises(B.BoltError):
        B.matmul_infer_output_size(B.tensor_nd(F, (4, 8, 16)), 0, B.tensor_nd(F, (4, 17, 8)), 0)
    with pytest.raises(B.BoltError):
        B.matmul_infer_output_size(B.tensor_nd(F, (3, 8, 16)), 0, B.tensor_nd(F, (4, 16, 8)), 0)   # batch 3 against 4
