"""The benchmarked workload itself against the CPU oracle: LinearStack.step() (dynamic u8 quantization of
the fp32 input, u8 x s8 GEMMs with per-output-channel weight scales, fused requantization to u8 between
layers, fp32 output) compared bit for bit with a CPU chain built from the oracle.

CPU chain per layer: int32 accumulators = offsetC[n] + sum_k A_u8 * W_s8 -- an exact float64 matrix
product (every sum is far below 2^53), tied to the oracle by comparing sampled rows with O.port_gemm --
then the documented epilogue, factor[n] = num / (sA * sB[n]) in binary32 (multiply, divide), and
u8 = usat8(rne((float)acc * factor[n]) + 128) / f32 = (float)acc * factor[n], the arithmetic of
mmm_avx512_vnni.cpp:1796-1808.  With one weight scale for all channels the chain must also equal
O.port_gemm with Bolt's scale argument, which test_oracle_pins.py pins to the compiled reference."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(__file__))
import oracle as O  # noqa: E402
import bolt_b200 as B  # noqa: E402
from bolt_b200 import synth  # noqa: E402
from bolt_b200.linear_stack import Linear, LinearStack, quantize_weight_host  # noqa: E402

pytestmark = pytest.mark.gpu


def make_stack(M, dims, per_channel, seed):
    layers, host = [], []
    for i in range(len(dims) - 1):
        W = synth.normal(seed + i, (dims[i], dims[i + 1]), 0.05)
        q, sc = quantize_weight_host(W, per_channel)
        layers.append(Linear(q, sc))
        host.append((q, sc))
    return LinearStack(layers, M, per_channel), host


def usat8_quirk(v):
    """vpmovusdb on rne + 128: the sum is read as unsigned, so negatives store 255"""
    return np.where((v >= 0) & (v <= 255), v, 255).astype(np.uint8)


def cpu_chain(x, host_layers, out_scales, rows_checked=48):
    """x fp32 [M, K0] -> (list of u8 activations per layer input, fp32 output)."""
    M = x.shape[0]
    s = np.array([-1], np.float32)
    q = np.zeros(x.size, np.uint8)
    O.port.oracle_quantize_f32_u8(O.ptr(np.ascontiguousarray(x)), x.size, O.ptr(q), O.ptr(s), 0)
    act = q.reshape(M, -1)
    sA = np.float32(s[0])
    acts = [act]
    rows = np.unique(np.linspace(0, M - 1, rows_checked).astype(np.int64))
    last = len(host_layers) - 1
    for i, (Wq, sB) in enumerate(host_layers):
        off = O.port_offsetc(Wq)
        acc = (act.astype(np.float64) @ Wq.astype(np.float64)).astype(np.int64) + off[None, :].astype(np.int64)
        assert np.abs(acc).max() < 2 ** 31
        acc = acc.astype(np.int32)
        assert np.array_equal(acc[rows], O.port_gemm(np.ascontiguousarray(act[rows]), Wq, off, None)), "layer %d accumulators" % i
        num = np.float32(1.0) if i == last else np.float32(out_scales[i])
        fac = (num / (sA * sB.astype(np.float32))).astype(np.float32)
        f = acc.astype(np.float32) * fac[None, :]
        if i == last:
            return acts, f.astype(np.float32)
        act = usat8_quirk(np.rint(f).astype(np.int64) + 128)
        if np.all(sB == sB[0]):  # one weight scale: Bolt's own scale protocol gives the same bytes
            ref = O.port_gemm(np.ascontiguousarray(acts[-1][rows]), Wq, off, [-1, float(fac[0])])
            assert np.array_equal(act[rows], ref), "layer %d vs scale protocol" % i
        acts.append(act)
        sA = np.float32(out_scales[i])


@pytest.mark.parametrize("M,dims,per_channel", [
    (4096, [768, 3072, 768, 3072, 768], True),     # two layer pairs of the benchmarked stack, full token count
    (4096, [768, 3072, 768], False),               # per-tensor weight scale: also equals Bolt's scale protocol
    (1000, [256, 1024, 2048, 512, 64], True),      # widths without a period, ragged M, several row blocks
    (77, [32, 32], True),
])
def test_stack_step_matches_cpu_chain(M, dims, per_channel):
    import torch

    st, host = make_stack(M, dims, per_channel, 900 + M)
    x = synth.normal(5 + M, (M, dims[0]))
    st.x_dev.copy_(torch.from_numpy(x.reshape(-1)).cuda())
    st.calibrate()
    st.step()
    B.CHECK_STATUS(B.lib().bolt_b200_synchronize(), "synchronize")
    acts, out = cpu_chain(x, host, st.out_scales)
    got = st.out_dev.cpu().numpy().reshape(M, dims[-1])
    assert got.tobytes() == out.tobytes()
    # the first layer's input (the dynamically quantized activations) is still in its buffer when the
    # number of layers is odd; otherwise compare what is left: the last u8 activation
    n = len(dims) - 1
    if n >= 2:
        last_act = acts[-1]
        buf = st.act[(n - 1) % 2].cpu().numpy()[: last_act.size].reshape(last_act.shape)
        assert np.array_equal(buf, last_act)


def test_full_depth_on_sampled_rows():
    """All 12 layer pairs of the benchmarked stack on 64 tokens (rows are independent once the input
    scale is fixed; the stack is built for M = 64 here)."""
    import torch

    M, dims = 64, [768, 3072] * 12 + [768]
    st, host = make_stack(M, dims, True, 100)
    x = synth.normal(1000, (M, 768))
    st.x_dev.copy_(torch.from_numpy(x.reshape(-1)).cuda())
    st.calibrate()
    st.step()
    B.CHECK_STATUS(B.lib().bolt_b200_synchronize(), "synchronize")
    _, out = cpu_chain(x, host, st.out_scales, rows_checked=8)
    assert st.out_dev.cpu().numpy().tobytes() == out.tobytes()
