"""GPU parity of the int8 convolution through the C ABI, in the shape of the reference's
compute/tensor/tests/test_convolution_int8.cpp (infer algorithm, transform the filter, query tmp,
run) -- but bit for bit against the reference's outputs (golden fixtures) and the oracle, where the
reference's own test only bounds the distance to an fp32 convolution by 8."""
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
DF_OF = {16: B.DF_NCHWC16, 8: B.DF_NCHWC8, 0: B.DF_NCHW}


def conv_gpu(shape, xin, w, bias, in_block, out_u8, relu, scales, eltwise=None, host=False, dilation=1,
             output_scale=None, filter_scales=None, in_f32=False):
    """relu: bool or an activation mode number.  output_scale / filter_scales: bolt_b200_convolution_ex."""
    n, ic, ih, iw, oc, fh, fw, st, pad = shape
    p = B.conv_param(oc, fh, fw, st, pad, dilation, bool(relu))
    in_desc = B.tensor4df(B.DT_F32 if in_f32 else B.DT_U8_Q, DF_OF[in_block], n, ic, ih, iw)
    f_desc = B.tensor4df(B.DT_I8, B.DF_NCHW, oc, ic, fh, fw)
    target = B.DT_U8_Q if out_u8 else B.DT_F32
    out_desc = B.convolution_infer_output_size(in_desc, f_desc, p, target)
    oh, ow = out_desc.dims[1], out_desc.dims[0]
    alg = B.convolution_infer_forward_algorithm(in_desc, f_desc, out_desc, p, target)
    assert alg == (B.CONVOLUTION_ALGORITHM_POINTWISE if fh == 1 and fw == 1 else B.CONVOLUTION_ALGORITHM_DIRECT)
    fbytes = B.convolution_transform_filter_bytes(f_desc, p, alg)
    tot = n * oc * oh * ow
    npdt = np.uint8 if out_u8 else np.float32
    sc = list(scales)
    if host:
        ftm = np.zeros(fbytes, np.uint8)
        ftm_desc = B.convolution_transform_filter(f_desc, hptr(w), p, alg, hptr(ftm))
        tb = B.convolution_infer_forward_tmp_bytes(in_desc, ftm_desc, out_desc, p, alg)
        tmp, out = np.zeros(tb, np.uint8), np.zeros(tot, npdt)
        B.convolution(in_desc, hptr(xin), ftm_desc, hptr(ftm), p, alg, sc, hptr(bias), tb, hptr(tmp), out_desc, hptr(out),
                      relu, None if eltwise is None else hptr(eltwise), output_scale,
                      None if filter_scales is None else hptr(filter_scales))
        B.lib().bolt_b200_release_weight(hptr(ftm))
        return out, sc, (oh, ow)
    d_w, d_ftm = to_dev(w), dev_zeros(fbytes)
    ftm_desc = B.convolution_transform_filter(f_desc, dptr(d_w), p, alg, dptr(d_ftm))
    assert ftm_desc.df == B.DF_NCHWC2NxC4
    tb = B.convolution_infer_forward_tmp_bytes(in_desc, ftm_desc, out_desc, p, alg)
    d_x, d_b, d_tmp, d_out = to_dev(xin), to_dev(bias), dev_zeros(tb), dev_zeros(tot * 4)
    d_e = None if eltwise is None else to_dev(eltwise)
    d_fs = None if filter_scales is None else to_dev(filter_scales)
    B.convolution(in_desc, dptr(d_x), ftm_desc, dptr(d_ftm), p, alg, sc, dptr(d_b), tb, dptr(d_tmp), out_desc, dptr(d_out),
                  relu, None if d_e is None else dptr(d_e), output_scale, None if d_fs is None else dptr(d_fs))
    B.CHECK_STATUS(B.lib().bolt_b200_synchronize(), "synchronize")
    return to_host(d_out, npdt, tot), sc, (oh, ow)


def oracle_conv(shape, xin, w, bias, in_block, out_u8, relu, scales, eltwise=None, dilation=1):
    n, ic, ih, iw, oc, fh, fw, st, pad = shape
    s = O.ConvShape(n, ic, ih, iw, oc, fh, fw, st, st, pad, pad, pad, pad, dilation, dilation, in_block, 16, int(relu), int(out_u8))
    oh, ow = C.c_uint32(), C.c_uint32()
    O.port.oracle_conv_out_hw(C.byref(s), C.byref(oh), C.byref(ow))
    out = np.zeros(n * oc * oh.value * ow.value, np.uint8 if out_u8 else np.float32)
    sc = np.array(scales, np.float32)
    O.port.oracle_conv_int8(C.byref(s), O.ptr(xin), O.ptr(w), O.ptr(bias), O.ptr(eltwise), O.ptr(out), O.ptr(sc), None)
    return out, sc


def test_conv_golden():
    g = np.load(os.path.join(GOLD, "conv.npz"))
    for i, shape in enumerate(cases.CONV_SHAPES):
        for blk, out_u8, relu in cases.conv_variants(i):
            xin, w, bias = cases.conv_inputs(i, blk)
            got, sc, _ = conv_gpu(shape, xin, w, bias, blk, out_u8, relu, cases.CONV_SCALES)
            key = "c%d_%d%d%d" % (i, blk, out_u8, relu)
            assert got.tobytes() == g[key].tobytes(), key
            assert np.array(sc, np.float32).tobytes() == g[key + "_scale"].tobytes(), key
        # the u8 output of a layer with a residual input, activation modes other than ReLU
        for name, out_u8, act, with_elt in cases.conv_extra_variants(i):
            blk = 16 if shape[1] % 16 == 0 else 8
            xin, w, bias = cases.conv_inputs(i, blk)
            key = "c%d_%s" % (i, name)
            elt = cases.conv_eltwise(i, g[key].size) if with_elt else None
            got, sc, _ = conv_gpu(shape, xin, w, bias, blk, out_u8, act, cases.CONV_SCALES, eltwise=elt)
            assert got.tobytes() == g[key].tobytes(), key
            assert np.array(sc, np.float32).tobytes() == g[key + "_scale"].tobytes(), key


def test_conv_u8_output_ignores_incoming_output_scale():
    """Bolt's engine leaves a calibrated scale in scale[1] on every run (convolution_cpu.hpp:150-156); the x86
    path overwrites it (convolution_direct.cpp:2687,2798-2806).  Same bytes and the same returned scale as
    the reference's dynamic path, whatever scale[1] holds on entry."""
    g = np.load(os.path.join(GOLD, "conv.npz"))
    for i in (1, 2):
        shape = cases.CONV_SHAPES[i]
        blk = 16
        xin, w, bias = cases.conv_inputs(i, blk)
        got, sc, _ = conv_gpu(shape, xin, w, bias, blk, 1, True, [cases.CONV_SCALES[0], 9.5, cases.CONV_SCALES[2]])
        key = "c%d_%d%d%d" % (i, blk, 1, 1)
        assert got.tobytes() == g[key].tobytes(), key
        assert np.array(sc, np.float32).tobytes() == g[key + "_scale"].tobytes(), key


# The 22 ResNet-50-shaped layers after the stem at a small batch: every kernel size / stride / channel width
RESNET_LAYERS = [(2, 64, 56, 56, 64, 1, 1, 1, 0), (2, 64, 56, 56, 64, 3, 3, 1, 1), (1, 64, 56, 56, 256, 1, 1, 1, 0),
                 (1, 256, 56, 56, 64, 1, 1, 1, 0), (1, 256, 56, 56, 128, 1, 1, 1, 0), (1, 128, 56, 56, 128, 3, 3, 2, 1),
                 (1, 256, 56, 56, 512, 1, 1, 2, 0),
                 (2, 128, 28, 28, 128, 3, 3, 1, 1), (2, 128, 28, 28, 512, 1, 1, 1, 0), (2, 512, 28, 28, 128, 1, 1, 1, 0),
                 (1, 512, 28, 28, 256, 1, 1, 1, 0), (2, 256, 28, 28, 256, 3, 3, 2, 1), (1, 512, 28, 28, 1024, 1, 1, 2, 0),
                 (2, 256, 14, 14, 256, 3, 3, 1, 1), (3, 256, 14, 14, 1024, 1, 1, 1, 0), (3, 1024, 14, 14, 256, 1, 1, 1, 0),
                 (2, 1024, 14, 14, 512, 1, 1, 1, 0), (2, 512, 14, 14, 512, 3, 3, 2, 1), (2, 1024, 14, 14, 2048, 1, 1, 2, 0),
                 (3, 512, 7, 7, 512, 3, 3, 1, 1), (9, 512, 7, 7, 2048, 1, 1, 1, 0), (3, 2048, 7, 7, 512, 1, 1, 1, 0)]


@pytest.mark.parametrize("shape", RESNET_LAYERS)
def test_conv_resnet_layers_vs_oracle(shape):
    n, ic, ih, iw, oc, fh, fw, st, pad = shape
    x = synth.relu_u8(ic + oc + ih, (n, ic, ih, iw))
    w = (synth.normal(ic * 3 + oc, (oc, ic, fh, fw), 0.05) * 127 / 0.2).clip(-127, 127).round().astype(np.int8)
    bias = synth.normal(9, (oc,), 0.1)
    for blk in (8, 16):
        xin = cases.to_blocked(x, blk)
        for out_u8 in (0, 1):
            got, sc, _ = conv_gpu(shape, xin, w, bias, blk, out_u8, True, [31.75, -1.0, 635.0])
            ref, sr = oracle_conv(shape, xin, w, bias, blk, out_u8, True, [31.75, -1.0, 635.0])
            assert got.tobytes() == ref.tobytes(), (shape, blk, out_u8)
            assert np.array(sc, np.float32).tobytes() == sr.tobytes()


def test_conv_eltwise_dilation_plain_nchw_and_host_pointers():
    shape = (2, 32, 11, 9, 48, 3, 3, 1, 1)
    n, ic, ih, iw, oc = shape[:5]
    x = synth.relu_u8(1, (n, ic, ih, iw))
    w = synth.s8(2, (oc, ic, 3, 3))
    bias = synth.normal(3, (oc,), 0.1)
    xin = cases.to_blocked(x, 16)
    elt = synth.normal(4, (n * oc * ih * iw,))
    got, _, _ = conv_gpu(shape, xin, w, bias, 16, 0, True, cases.CONV_SCALES, eltwise=elt)      # fused residual add
    ref, _ = oracle_conv(shape, xin, w, bias, 16, 0, True, cases.CONV_SCALES, eltwise=elt)
    assert got.tobytes() == ref.tobytes()
    shape_d = (1, 16, 12, 12, 16, 3, 3, 1, 2)                                                      # dilation 2
    xd, wd, bd = cases.to_blocked(synth.relu_u8(5, (1, 16, 12, 12)), 16), synth.s8(6, (16, 16, 3, 3)), synth.normal(7, (16,), 0.1)
    got, _, _ = conv_gpu(shape_d, xd, wd, bd, 16, 0, False, cases.CONV_SCALES, dilation=2)
    ref, _ = oracle_conv(shape_d, xd, wd, bd, 16, 0, False, cases.CONV_SCALES, dilation=2)
    assert got.tobytes() == ref.tobytes()
    xp = np.ascontiguousarray(x).reshape(-1)                                                       # plain NCHW input
    got, _, _ = conv_gpu(shape, xp, w, bias, 0, 1, True, cases.CONV_SCALES)
    ref, _ = oracle_conv(shape, xp, w, bias, 0, 1, True, cases.CONV_SCALES)
    assert got.tobytes() == ref.tobytes()
    got, sc, _ = conv_gpu(shape, xin, w, bias, 16, 1, True, cases.CONV_SCALES, host=True)          # host buffers
    ref, sr = oracle_conv(shape, xin, w, bias, 16, 1, True, cases.CONV_SCALES)
    assert got.tobytes() == ref.tobytes() and np.array(sc, np.float32).tobytes() == sr.tobytes()


def test_conv_batch_independence():
    """Size-independent property used for the batch split across GPUs: conv(batch)[i] == conv(image i)."""
    shape = (4, 64, 14, 14, 64, 3, 3, 1, 1)
    x = synth.relu_u8(11, (4, 64, 14, 14))
    w, bias = synth.s8(12, (64, 64, 3, 3)), synth.normal(13, (64,), 0.1)
    full, _, (oh, ow) = conv_gpu(shape, cases.to_blocked(x, 16), w, bias, 16, 0, True, cases.CONV_SCALES)
    per = 64 * oh * ow
    for i in range(4):
        one, _, _ = conv_gpu((1,) + shape[1:], cases.to_blocked(x[i:i + 1], 16), w, bias, 16, 0, True, cases.CONV_SCALES)
        assert one.tobytes() == full[i * per:(i + 1) * per].tobytes()


def test_conv_batch_64_sampled_images():
    """The batch the benchmark times: one layer per kernel size at batch 64; eight sampled images of the
    device result against the oracle run on those images alone (images are independent)."""
    for shape in [(64, 256, 14, 14, 64, 1, 1, 1, 0), (64, 64, 14, 14, 64, 3, 3, 1, 1), (64, 128, 14, 14, 128, 3, 3, 2, 1)]:
        n, ic, ih, iw, oc, fh, fw, st, pad = shape
        x = synth.relu_u8(ic + oc + 64, (n, ic, ih, iw))
        w = (synth.normal(ic * 7 + oc, (oc, ic, fh, fw), 0.05) * 127 / 0.2).clip(-127, 127).round().astype(np.int8)
        bias = synth.normal(29, (oc,), 0.1)
        got, _, (oh, ow) = conv_gpu(shape, cases.to_blocked(x, 16), w, bias, 16, 0, True, [31.75, -1.0, 635.0])
        per = oc * oh * ow
        for i in (0, 7, 8, 21, 33, 47, 62, 63):
            ref, _ = oracle_conv((1,) + shape[1:], cases.to_blocked(x[i:i + 1], 16), w, bias, 16, 0, True, [31.75, -1.0, 635.0])
            assert got[i * per:(i + 1) * per].tobytes() == ref.tobytes(), (shape, i)


def test_conv_fp32_input_is_quantized_first():
    """convolution_direct.cpp:2679-2686: an fp32 input goes through quantize_x86 (dynamic scale written to
    scale[0]) and the u8 path."""
    shape = (2, 32, 9, 7, 48, 3, 3, 1, 1)
    n, ic, ih, iw, oc = shape[:5]
    xf = np.abs(synth.normal(41, (n, ic, ih, iw)))
    w, bias = synth.s8(42, (oc, ic, 3, 3)), synth.normal(43, (oc,), 0.1)
    xin_f = cases.to_blocked(xf, 16)
    s_in = np.array([-1], np.float32)
    q = np.zeros(xin_f.size, np.uint8)
    O.port.oracle_quantize_f32_u8(O.ptr(xin_f), xin_f.size, O.ptr(q), O.ptr(s_in), 0)
    ref, sr = oracle_conv(shape, q, w, bias, 16, 0, True, [float(s_in[0]), -1.0, 310.0])
    got, sc, _ = conv_gpu(shape, xin_f, w, bias, 16, 0, True, [-1.0, -1.0, 310.0], in_f32=True)
    assert got.tobytes() == ref.tobytes() and np.array(sc, np.float32).tobytes() == sr.tobytes()


def test_conv_per_channel_filter_scales():
    """Extension: one weight scale per output channel.  With all of them equal the result is the per-tensor
    one; with different ones it follows the definition channel by channel: the bias term uses
    scaleI * sF[oc] and the accumulator is divided by it."""
    shape = (2, 64, 12, 12, 48, 3, 3, 1, 1)
    n, ic, ih, iw, oc, fh, fw, st, pad = shape
    x = synth.relu_u8(51, (n, ic, ih, iw))
    w, bias = synth.s8(52, (oc, ic, 3, 3)), synth.normal(53, (oc,), 0.1)
    xin = cases.to_blocked(x, 16)
    s_in, s_f = 37.5, 310.0
    ref, _ = oracle_conv(shape, xin, w, bias, 16, 0, True, [s_in, -1.0, s_f])
    got, _, _ = conv_gpu(shape, xin, w, bias, 16, 0, True, [s_in, -1.0, s_f], filter_scales=np.full(oc, s_f, np.float32))
    assert got.tobytes() == ref.tobytes()
    fs = (s_f * (1.0 + 0.5 * np.abs(synth.normal(54, (oc,))))).astype(np.float32)
    got, _, (oh, ow) = conv_gpu(shape, xin, w, bias, 16, 0, True, [s_in, -1.0, s_f], filter_scales=fs)
    got = got.reshape(n, oc // 16, oh, ow, 16)
    for o in (0, 5, 17, 47):                                   # channel o alone with its own scale, through the oracle
        one, _ = oracle_conv(shape, xin, w, bias, 16, 0, True, [s_in, -1.0, float(fs[o])])
        assert got[:, o // 16, :, :, o % 16].tobytes() == one.reshape(n, oc // 16, oh, ow, 16)[:, o // 16, :, :, o % 16].tobytes()


def test_conv_fused_u8_with_given_output_scale():
    """Extension (bolt_b200_convolution_ex): a known output scale fuses ReLU + requantization into the epilogue.  Checked
    against the oracle's int32 accumulators pushed through the reference's I32 -> U8_Q arithmetic with
    both scales given (avx512/quantize.cpp:372-414), the path Bolt's fully-connected layer takes when
    the output scale is known (fully_connected.cpp:479-487)."""
    for shape in [(2, 64, 14, 14, 64, 3, 3, 1, 1), (1, 128, 28, 28, 72, 1, 1, 1, 0), (2, 32, 9, 9, 48, 3, 3, 2, 1)]:
        n, ic, ih, iw, oc, fh, fw, st, pad = shape
        x = synth.relu_u8(ic + oc, (n, ic, ih, iw))
        w = (synth.normal(ic * 5 + oc, (oc, ic, fh, fw), 0.05) * 127 / 0.2).clip(-127, 127).round().astype(np.int8)
        bias = synth.normal(19, (oc,), 0.1)
        xin = cases.to_blocked(x, 16)
        s_in, s_out, s_f = 31.75, 9.5, 635.0
        got, sc, _ = conv_gpu(shape, xin, w, bias, 16, 1, True, [s_in, -1.0, s_f], output_scale=s_out)
        assert sc[1] == s_out
        s = O.ConvShape(n, ic, ih, iw, oc, fh, fw, st, st, pad, pad, pad, pad, 1, 1, 16, 16, 1, 1)
        acc = np.zeros(got.size, np.int32)
        scr = np.array([s_in, -1.0, s_f], np.float32)
        O.port.oracle_conv_int8(C.byref(s), O.ptr(xin), O.ptr(w), O.ptr(bias), None, O.ptr(np.zeros(got.size, np.uint8)), O.ptr(scr), O.ptr(acc))
        ref = np.zeros(got.size, np.uint8)
        sq = np.array([s_out, np.float32(s_in) * np.float32(s_f)], np.float32)
        O.port.oracle_quantize_i32_u8(O.ptr(acc), acc.size, O.ptr(ref), O.ptr(sq))
        assert got.tobytes() == ref.tobytes(), shape
