"""Counter-based synthetic data: the same bytes on every machine and numpy version.

splitmix64 of (seed, element index) drives everything; normal deviates are an Irwin-Hall sum of
eight 16-bit uniforms (integer arithmetic plus one exact scaling), so that no libm call can make
two hosts disagree by an ulp.  Used by the parity tests, the golden-fixture generator and the
benchmark, which all have to feed identical inputs to the CUDA library and to the CPU oracle.
"""
import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x):
    x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
    z = x
    z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
    z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
    return z ^ (z >> np.uint64(31))


def bits64(seed, n, stream=0):
    """n 64-bit words for (seed, stream)."""
    with np.errstate(over="ignore"):
        base = _splitmix64(np.uint64(seed) * np.uint64(0x100000001B3) + np.uint64(stream))
        idx = np.arange(n, dtype=np.uint64)
        return _splitmix64(idx * np.uint64(0xD6E8FEB86659FD93) + base)


def u8(seed, shape):
    n = int(np.prod(shape))
    w = bits64(seed, (n + 7) // 8)
    return w.view(np.uint8)[:n].reshape(shape).copy()


def s8(seed, shape):
    return u8(seed, shape).view(np.int8)


def integers(seed, shape, lo, hi, dtype=np.int32):
    """uniform integers in [lo, hi)"""
    n = int(np.prod(shape))
    w = bits64(seed, n)
    return (lo + (w % np.uint64(hi - lo)).astype(np.int64)).astype(dtype).reshape(shape)


def normal(seed, shape, std=1.0):
    """approximately N(0, std^2), float32, bit-reproducible"""
    n = int(np.prod(shape))
    acc = np.zeros(n, np.int64)
    for s in range(2):
        w = bits64(seed, n, stream=s + 1)
        for sh in (0, 16, 32, 48):
            acc += ((w >> np.uint64(sh)) & np.uint64(0xFFFF)).astype(np.int64)
    # 8 uniforms on [0, 65535]: mean 8 * 32767.5, variance 8 * (65536^2 - 1) / 12
    centred = (acc * 2 - 8 * 65535).astype(np.float64) / 2.0
    sigma = np.sqrt(8 * (65536.0 ** 2 - 1) / 12.0)
    return (centred * (std / sigma)).astype(np.float32).reshape(shape)


def relu_u8(seed, shape):
    """ReLU-distributed u8 activations with zero point 128: clamp(rne(relu(N(0,1)) * s) + 128),
    s chosen so that 4 sigma lands on 255."""
    x = np.maximum(normal(seed, shape), 0)
    q = np.rint(x * np.float32(127.0 / 4.0)).astype(np.int32) + 128
    return np.clip(q, 1, 255).astype(np.uint8)
