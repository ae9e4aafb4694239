"""GPU parity of the int8 matmul operator (both operands quantized per call, B packed on the fly for every batch)
through the C ABI, in the shape of compute/tensor/tests/test_matmul_int8.cpp (infer the output size, query the
tmp bytes, run): bit for bit against the reference's outputs (golden fixtures) and, at larger sizes, the oracle."""
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
NP_OF = {B.DT_F32: np.float32, B.DT_U8_Q: np.uint8}


def matmul_gpu(A, a_dt, a_scale, ta, Bm, b_dt, b_scale, tb, bias, c_dt, c_scale, host=False):
    a_desc, b_desc = B.tensor_nd(a_dt, A.shape), B.tensor_nd(b_dt, Bm.shape)
    c_desc = B.matmul_infer_output_size(a_desc, ta, b_desc, tb)
    c_desc.dt = c_dt
    shape = tuple(reversed(list(c_desc.dims[: c_desc.nDims])))
    n_out = int(np.prod(shape))
    tmp_bytes = B.matmul_infer_forward_tmp_bytes(a_desc, ta, b_desc, tb, c_desc, c_scale)
    bias_desc = None if bias is None else B.tensor1d(B.DT_F32, bias.size)
    if host:
        out = np.zeros(n_out, NP_OF[c_dt])
        tmp = np.zeros(tmp_bytes, np.uint8)
        s = B.matmul(a_desc, ta, hptr(A), a_scale, b_desc, tb, hptr(Bm), b_scale, bias_desc, None if bias is None else hptr(bias),
                     tmp_bytes, hptr(tmp), c_desc, hptr(out), c_scale)
        return out.reshape(shape), s
    d_a, d_b, d_tmp, d_c = to_dev(A), to_dev(Bm), dev_zeros(tmp_bytes), dev_zeros(n_out * 4)
    d_bias = None if bias is None else to_dev(bias)
    d_c.fill_(0x5A)     # the operator must not depend on what the output held
    s = B.matmul(a_desc, ta, dptr(d_a), a_scale, b_desc, tb, dptr(d_b), b_scale, bias_desc, None if bias is None else dptr(d_bias),
                 tmp_bytes, dptr(d_tmp), c_desc, dptr(d_c), c_scale)
    B.CHECK_STATUS(B.lib().bolt_b200_synchronize(), "synchronize")
    return to_host(d_c, NP_OF[c_dt], n_out).reshape(shape), s


@pytest.mark.parametrize("host", [False, True])
def test_matmul_golden(host):
    g = np.load(os.path.join(GOLD, "matmul.npz"))
    for name in cases.MATMUL_CASES:
        C, scale = matmul_gpu(*cases.matmul_inputs(name), host=host)
        assert C.shape == g[name].shape and C.tobytes() == g[name].tobytes(), (name, host)
        assert np.float32(scale).tobytes() == g[name + "_scale"].tobytes(), name


def test_matmul_static_u8_output_vs_oracle():
    """u8 output requantized inside the product with the output tensor's scale (matmul.cpp:383-386,429-431).  The
    reference stores such a result's rows 4N bytes apart; the rows themselves are pinned one at a time in the GEMM
    fixtures, and the operator here writes them densely."""
    F, U = B.DT_F32, B.DT_U8_Q
    A, Bm = synth.normal(1, (3, 40, 64)), synth.normal(2, (3, 64, 24))
    for c_scale in (0.5, 2.0, 40.0):
        args = (A, F, -1.0, 0, Bm, F, -1.0, 0, None, U, c_scale)
        C, s = matmul_gpu(*args)
        Cp, sp = O.port_matmul(*args)
        assert C.tobytes() == Cp.tobytes() and np.float32(s) == np.float32(sp), c_scale


def test_matmul_attention_shapes_vs_oracle():
    """BERT-base attention at batch 2: scores = Q K^T ([24, 128, 64] x [24, 128, 64]^T) and context = P V, on the
    tensor cores, fp32 and dynamically requantized outputs."""
    F, U = B.DT_F32, B.DT_U8_Q
    q, k = synth.normal(11, (2, 12, 128, 64)), synth.normal(12, (2, 12, 128, 64))
    pr, v = np.abs(synth.normal(13, (2, 12, 128, 128), 0.1)), synth.normal(14, (2, 12, 128, 64))
    for args in ((q, F, -1.0, 0, k, F, -1.0, 1, None, F, -1.0), (pr, F, -1.0, 0, v, F, -1.0, 0, None, F, -1.0),
                 (pr, F, -1.0, 0, v, F, -1.0, 0, None, U, -1.0)):
        C, s = matmul_gpu(*args)
        Cp, sp = O.port_matmul(*args)
        assert C.tobytes() == Cp.tobytes() and np.float32(s) == np.float32(sp)
    assert B.lib().bolt_b200_last_gemm_used_tensor_cores() == 1


def test_matmul_argument_checks():
    F = B.DT_F32
    a_desc, b_desc = B.tensor_nd(F, (4, 8, 16)), B.tensor_nd(F, (4, 17, 8))
    with pytest.raises(B.BoltError):
        B.matmul_infer_output_size(a_desc, 0, b_desc, 0)                       # inner extents differ
    b_desc = B.tensor_nd(F, (4, 16, 8))
    c_desc = B.matmul_infer_output_size(a_desc, 0, b_desc, 0)
    assert list(c_desc.dims[:3]) == [8, 8, 4]
    lib = B.lib()
    import ctypes as C
    n = C.c_uint32()
    # fp32 tensors without a quantization flag: not the int8 operator
    assert lib.matmul_infer_forward_tmp_bytes_cuda_b200(C.byref(a_desc), 0, C.byref(b_desc), 0, C.byref(c_desc), 0.0, C.byref(n)) == B.NOT_SUPPORTED
    need = B.matmul_infer_forward_tmp_bytes(a_desc, 0, b_desc, 0, c_desc, -1.0)
    d = dev_zeros(4 * 8 * 16 * 4)
    s = C.c_float(-1.0)
    bd = B.tensor1d(F, 0)
    assert lib.matmul_cuda_b200(C.byref(a_desc), 0, dptr(d), -1.0, C.byref(b_desc), 0, dptr(d), -1.0, C.byref(bd), None, need - 1, dptr(d),
                                C.byref(c_desc), dptr(d), C.byref(s)) == B.NOT_MATCH       # tmp too small
