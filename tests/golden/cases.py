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
