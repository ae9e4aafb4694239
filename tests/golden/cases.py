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


GEMV_ROW_SHAPES = [(1, 1), (3, 5), (4, 16), (7, 33), (17, 64), (33, 130), (64, 256), (67, 1000)]


def gemv_row_inputs(i, m_t):
    n, k = GEMV_ROW_SHAPES[i]
    seed = 9000 + i * 2 + m_t
    Mx = synth.u8(seed, (k, n) if m_t else (n, k))
    v = synth.s8(seed + 500, (k,))
    return Mx, v
