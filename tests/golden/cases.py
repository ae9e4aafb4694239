"""Case lists and seeded inputs shared by make_golden.py (which stores the reference's outputs)
and by the tests (which regenerate the same inputs and compare against the stored outputs)."""
import numpy as np

from bolt_b200 import synth

GEMM_SHAPES = [(1, 1, 1), (3, 5, 7), (8, 8, 8), (9, 17, 33), (33, 33, 33), (24, 40, 48), (25, 64, 49),
               (40, 96, 72), (5, 4100, 16), (32, 256, 48)]
GEMM_F32_SCALE = [0.37]
GEMM_U8_SCALE = [-1, 0.004]


def gemm_variants(i):
    """(a_t, b_t) pairs pinned for shape i.  Transposed A with K > 4096 is left out: from the
    second K block on the reference transposes its own scratch instead of A
    (mmm_avx512_vnni.cpp:1849-1855, `packA = tmp`), so its result there is not the product."""
    k = GEMM_SHAPES[i][1]
    return [(a, b) for a in (0, 1) for b in (0, 1) if not (a == 1 and k > 4096)]


def gemm_inputs(i, a_t, b_t):
    m, k, n = GEMM_SHAPES[i]
    seed = 1000 + i * 4 + a_t * 2 + b_t
    A = synth.u8(seed, (k, m) if a_t else (m, k))
    B = synth.s8(seed + 500, (n, k) if b_t else (k, n))
    Cin = synth.integers(seed + 900, (m, n), -1000, 1000)
    return A, B, Cin


GEMV_SHAPES = [(1, 1), (7, 5), (8, 8), (15, 33), (64, 64), (65, 100), (100, 2100), (129, 31), (256, 512)]


def gemv_inputs(i, w_t):
    n, k = GEMV_SHAPES[i]
    seed = 3000 + i * 2 + w_t
    W = synth.s8(seed, (k, n) if w_t else (n, k))
    x = synth.u8(seed + 500, (k,))
    yin = synth.integers(seed + 900, (n,), -1000, 1000)
    return W, x, yin


QUANT_SIZES = [1, 15, 16, 17, 100, 4099]


def quant_inputs(i):
    n = QUANT_SIZES[i]
    seed = 5000 + i
    x = synth.normal(seed, (n,))
    a = synth.integers(seed + 100, (n,), -100000, 100000)
    u = synth.u8(seed + 200, (n,))
    b = synth.normal(seed + 300, (n,))
    b[0] = 0.5
    off = synth.integers(seed + 400, (n,), -1000, 1000)
    return x, a, u, b, off


# (n, ic, ih, iw, oc, fh, fw, stride, pad)
CONV_SHAPES = [(1, 16, 8, 8, 16, 1, 1, 1, 0), (2, 32, 9, 7, 48, 3, 3, 1, 1), (1, 64, 14, 14, 64, 3, 3, 2, 1),
               (2, 16, 6, 6, 24, 1, 1, 2, 0), (1, 8, 5, 5, 8, 3, 3, 1, 1), (1, 24, 7, 7, 40, 3, 3, 1, 1),
               (1, 64, 12, 12, 32, 1, 1, 1, 0), (1, 128, 9, 9, 32, 3, 3, 2, 1)]
CONV_SCALES = [37.5, -1.0, 310.0]   # input scale, output scale (dynamic), filter scale


def to_blocked(x, blk):
    """[N, C, H, W] -> flat channel-blocked layout: blocks of `blk` channels, narrower tail block."""
    n, c, h, w = x.shape
    out = []
    for i in range(n):
        cb = 0
        while cb < c:
            wd = min(blk, c - cb)
            out.append(x[i, cb:cb + wd].transpose(1, 2, 0).reshape(-1))
            cb += wd
    return np.concatenate(out)


def conv_inputs(i, in_block):
    n, ic, ih, iw, oc, fh, fw, st, pad = CONV_SHAPES[i]
    x = synth.relu_u8(7000 + i, (n, ic, ih, iw))
    w = synth.s8(7100 + i, (oc, ic, fh, fw))
    bias = synth.normal(7200 + i, (oc,), 0.1)
    return to_blocked(x, in_block), w, bias


def conv_variants(i):
    """(in_block, out_u8, relu) combinations pinned for shape i"""
    ic = CONV_SHAPES[i][1]
    blocks = (8, 16) if ic % 16 == 0 else (8,)
    return [(b, u, r) for b in blocks for u in (0, 1) for r in (0, 1)]


def conv_extra_variants(i):
    """(key, out_u8, activation mode, with eltwise) beyond conv_variants: the u8 output of a layer with a
    residual input, and activation modes that are not ReLU (2 and 3 act as ReLU, 4 as none: the kernels
    test mode & 3)."""
    if i not in (1, 2, 6):
        return []
    return [("eltu8", 1, 1, True), ("eltu8n", 1, 0, True), ("act2", 0, 2, False), ("act3u8", 1, 3, False), ("act4", 0, 4, False)]


def conv_eltwise(i, total):
    return synth.normal(7300 + i, (total,), 0.5)


GEMV_ROW_SHAPES = [(1, 1), (3, 5), (4, 16), (7, 33), (17, 64), (33, 130), (64, 256), (67, 1000)]


def gemv_row_inputs(i, m_t):
    n, k = GEMV_ROW_SHAPES[i]
    seed = 9000 + i * 2 + m_t
    Mx = synth.u8(seed, (k, n) if m_t else (n, k))
    v = synth.s8(seed + 500, (k,))
    return Mx, v


# 1-bit convolution: (n, ic, ih, iw, oc, fh, fw, stride, pad).  The reference's scalar branch
# accumulates in binary16, which is exact while every partial sum stays within +-2048; with random
# signs the partial sums of these shapes stay far below that (K = ic * fh * fw <= 2304).
BNN_SHAPES = [(1, 8, 5, 5, 8, 3, 3, 1, 1), (2, 32, 7, 6, 32, 3, 3, 1, 1), (1, 64, 9, 9, 72, 3, 3, 2, 1),
              (2, 40, 6, 6, 16, 1, 1, 1, 0), (1, 96, 8, 8, 48, 5, 5, 1, 2), (1, 256, 10, 10, 32, 3, 3, 1, 1)]


def pack_bits_msb(bits):
    """flat 0/1 array -> bytes, MSB first (the DT_BIN01 / DT_BIN11 storage, data_type.h:463-485)"""
    return np.packbits(bits.astype(np.uint8), bitorder="big")


def bnn_inputs(i, xnor, scaling):
    """scaling 0: scale 1, bias 0 (the raw tap sums); 1: scales that are powers of two and biases that
    are multiples of 1/4 (every step exact in binary16); 2: scale = mean |W| per channel and a normal
    bias (XNOR-Net's alpha / beta).  All as binary16 bit patterns; input in NCHWc8."""
    n, ic, ih, iw, oc, fh, fw, st, pad = BNN_SHAPES[i]
    seed = 11000 + 10 * i + (5 if xnor else 0)
    x = synth.normal(seed, (n, ic, ih, iw)).astype(np.float16)
    if not xnor:
        x = (x * np.float16(0.5) + np.float16(0.5)).astype(np.float16)   # DoReFa activations around 0.5
    x.reshape(-1)[::7] = np.float16(0.0 if xnor else 0.5)                # values exactly on the threshold
    wf = synth.normal(seed + 1, (oc, ic, fh, fw))
    wbits = pack_bits_msb((wf >= 0).reshape(-1))
    if scaling == 0:
        scale, bias = np.ones(oc, np.float16), np.zeros(oc, np.float16)
    elif scaling == 1:
        scale = (2.0 ** -(np.arange(oc) % 4)).astype(np.float16)
        bias = ((np.arange(oc) % 9 - 4) * 0.25).astype(np.float16)
    else:
        scale = np.abs(wf).reshape(oc, -1).mean(axis=1).astype(np.float16)
        bias = synth.normal(seed + 2, (oc,), 0.1).astype(np.float16)
    return to_blocked(x.view(np.uint16), 8), wbits, scale.view(np.uint16), bias.view(np.uint16)


# ---- matmul operator -------------------------------------------------------------------------------
# data types as Bolt numbers them
MM_F32, MM_U8, MM_I8 = 6, 10, 1
# name -> (A shape, A type, A scale, transposeA, B shape, B type, B scale, transposeB, bias length, C type, C scale).
# Shapes are the stored shapes, outermost first.  A scale <= 0 on an fp32 tensor asks for 127 / absmax.  Every case
# writes fp32 or dynamically quantized u8, or is a one-row product: the reference's GEMM with a u8 result of
# more than one row stores its rows 4N bytes apart (past the end of the tensor), so there is nothing to pin there.
MATMUL_CASES = {
    "f32": ((2, 3, 40, 64), MM_F32, -1, 0, (2, 3, 64, 24), MM_F32, -1, 0, 0, MM_F32, -1),
    "u8dyn": ((2, 3, 40, 64), MM_F32, -1, 0, (2, 3, 64, 24), MM_F32, -1, 0, 0, MM_U8, -1),
    "row": ((2, 3, 1, 64), MM_F32, -1, 0, (2, 3, 64, 24), MM_F32, -1, 0, 0, MM_F32, -1),
    "row_tb": ((2, 3, 1, 64), MM_F32, -1, 0, (2, 3, 24, 64), MM_F32, -1, 1, 0, MM_F32, -1),
    "row_u8": ((4, 1, 96), MM_F32, -1, 0, (4, 96, 50), MM_F32, -1, 0, 0, MM_U8, 0.7),
    "row_u8dyn": ((4, 1, 96), MM_F32, -1, 0, (4, 96, 50), MM_F32, -1, 0, 0, MM_U8, -1),
    "col": ((2, 3, 40, 64), MM_F32, -1, 0, (2, 3, 64, 1), MM_F32, -1, 0, 0, MM_F32, -1),
    "col_ta": ((2, 3, 64, 40), MM_F32, -1, 1, (2, 3, 64, 1), MM_F32, -1, 0, 0, MM_F32, -1),
    "tb": ((2, 3, 40, 64), MM_F32, -1, 0, (2, 3, 24, 64), MM_F32, -1, 1, 0, MM_F32, -1),
    "ta": ((2, 3, 64, 40), MM_F32, -1, 1, (2, 3, 64, 24), MM_F32, -1, 0, 0, MM_F32, -1),
    "ta_tb": ((2, 3, 64, 40), MM_F32, -1, 1, (2, 3, 24, 64), MM_F32, -1, 1, 0, MM_F32, -1),
    "bias": ((2, 3, 40, 64), MM_F32, -1, 0, (2, 3, 64, 24), MM_F32, -1, 0, 24, MM_F32, -1),
    "bcast": ((2, 3, 40, 64), MM_F32, -1, 0, (1, 1, 64, 24), MM_F32, -1, 0, 0, MM_F32, -1),
    "bcast_rank": ((2, 3, 40, 64), MM_F32, -1, 0, (64, 24), MM_F32, -1, 0, 0, MM_F32, -1),
    "bcast_a": ((1, 33, 50), MM_F32, -1, 0, (5, 50, 17), MM_F32, -1, 0, 0, MM_F32, -1),
    "quantized": ((3, 33, 50), MM_U8, 31.5, 0, (3, 50, 17), MM_I8, 200.0, 0, 0, MM_F32, 1.0),
    "quantized_u8": ((3, 33, 50), MM_U8, 31.5, 0, (3, 50, 17), MM_I8, 200.0, 0, 0, MM_U8, 0.0),
    "mixed": ((3, 33, 50), MM_U8, 31.5, 0, (3, 50, 17), MM_F32, -1, 0, 0, MM_F32, -1),
    "given_scales": ((2, 40, 64), MM_F32, 5.0, 0, (2, 64, 24), MM_F32, 3.0, 0, 0, MM_F32, -1),
    "attention_qk": ((1, 2, 128, 64), MM_F32, -1, 0, (1, 2, 128, 64), MM_F32, -1, 1, 0, MM_F32, -1),
    "attention_pv": ((1, 2, 128, 128), MM_F32, -1, 0, (1, 2, 128, 64), MM_F32, -1, 0, 0, MM_F32, -1),
    "ragged": ((3, 7, 13), MM_F32, -1, 0, (3, 13, 5), MM_F32, -1, 0, 0, MM_F32, -1),
}


def matmul_inputs(name):
    a_shape, a_dt, a_s, ta, b_shape, b_dt, b_s, tb, bias_n, c_dt, c_s = MATMUL_CASES[name]
    seed = 8800 + sorted(MATMUL_CASES).index(name) * 3

    def make(sd, shape, dt):
        if dt == MM_F32:
            return synth.normal(sd, shape)
        return synth.u8(sd, shape) if dt == MM_U8 else synth.s8(sd, shape)

    A, B = make(seed, a_shape, a_dt), make(seed + 1, b_shape, b_dt)
    bias = synth.normal(seed + 2, (bias_n,)) if bias_n else None
    return (A, a_dt, a_s, ta, B, b_dt, b_s, tb, bias, c_dt, c_s)


# ---- u8 pooling ------------------------------------------------------------------------------------
# (n, c, ih, iw, kernel, stride, pad, mean, count_include_pad, ceil)
POOL_CASES = [(2, 32, 9, 9, 3, 2, 1, 0, 0, 0), (2, 32, 9, 9, 3, 2, 1, 1, 0, 0), (2, 32, 9, 9, 3, 2, 1, 1, 1, 0),
              (1, 16, 7, 7, 7, 1, 0, 1, 0, 0), (1, 16, 7, 7, 7, 1, 0, 0, 0, 0), (2, 64, 14, 14, 2, 2, 0, 0, 0, 0),
              (2, 64, 14, 14, 2, 2, 0, 1, 0, 0), (1, 16, 10, 13, 3, 1, 1, 1, 0, 0), (1, 48, 8, 8, 3, 2, 0, 0, 0, 1),
              (1, 48, 8, 8, 3, 2, 0, 1, 1, 1), (1, 16, 5, 5, 5, 1, 2, 1, 0, 0), (1, 64, 56, 56, 3, 2, 1, 0, 0, 0)]


def pool_out_hw(case):
    n, c, ih, iw, k, s, p, mean, cip, ceil = case
    if ceil:
        return (ih + 2 * p - k + s - 1) // s + 1, (iw + 2 * p - k + s - 1) // s + 1
    return (ih + 2 * p - k) // s + 1, (iw + 2 * p - k) // s + 1


def pool_input(i):
    n, c, ih, iw = POOL_CASES[i][:4]
    # mean windows below the zero point store 255 in the reference: keep both kinds of windows in the data
    return synth.u8(9100 + i, (n * c * ih * iw,))
