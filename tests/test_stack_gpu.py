"""The persistent linear-stack kernel (bolt_b200_linear_stack_*) against the layer-by-layer path: same
bits in every layer's output, for stacks with ragged M, different widths and tile shapes.  The
layer-by-layer path itself is pinned against the oracle in test_blas_gpu.py."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(__file__))
import bolt_b200 as B  # noqa: E402
from bolt_b200 import synth  # noqa: E402
from bolt_b200.linear_stack import Linear, LinearStack, quantize_weight_host  # noqa: E402

pytestmark = pytest.mark.gpu


def make_stack(M, dims, per_channel, seed):
    layers = []
    for i in range(len(dims) - 1):
        W = synth.normal(seed + i, (dims[i], dims[i + 1]), 0.05)
        q, sc = quantize_weight_host(W, per_channel)
        layers.append(Linear(q, sc))
    return LinearStack(layers, M, per_channel)


@pytest.mark.parametrize("M,dims,per_channel", [
    (300, [64, 96, 64], True),
    (128, [128, 256, 128, 32], False),
    (1000, [256, 1024, 256, 1024, 256], True),
    (4096, [768, 3072, 768, 3072, 768], True),
    (77, [32, 32], True),
])
def test_fused_stack_matches_layer_by_layer(M, dims, per_channel):
    import torch

    st = make_stack(M, dims, per_channel, 900 + M)
    x = torch.from_numpy(synth.normal(5 + M, (M * dims[0],))).cuda()
    st.x_dev.copy_(x)
    st.calibrate()
    st.step()
    torch.cuda.synchronize()
    ref_out = st.out_dev.clone()
    ref_acts = [a.clone() for a in st.act]
    st.out_dev.zero_()
    for a in st.act:
        a.zero_()
    st.build_fused()
    for _ in range(2):  # twice: the progress counters are reset by every run
        st.step_fused()
        B.CHECK_STATUS(B.lib().bolt_b200_synchronize(), "synchronize")
        assert torch.equal(st.out_dev, ref_out)
        for a, r in zip(st.act, ref_acts):
            assert torch.equal(a, r)
    st.free_fused()
