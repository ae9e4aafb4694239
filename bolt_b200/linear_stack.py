"""A stack of quantized fully-connected layers kept 8-bit between layers -- the serving-side use
of the GEMM path (what Bolt's FullyConnected operator does per layer on x86,
compute/tensor/src/fully_connected.cpp:373-411,457-495: u8 activations, s8 pre-packed weights,
bias folded into offsetC, `scale = {-1, outScale/(scaleI*scaleW)}` for a fused u8 output).

torch is used for device memory and streams only; every kernel is launched by libbolt_b200.so.
"""
import ctypes as C

import numpy as np

from . import (CHECK_STATUS, DF_NORMAL, DF_TRANSPOSE, DT_F32, DT_I8, DT_I32, DT_U8_Q, GemmEpilogue, lib,
               matrix_matrix_multiply_transform_rhs, matrix_matrix_multiply_transform_rhs_bytes, tensor2df)


def _torch():
    import torch

    return torch


def quantize_weight_host(W, per_channel):
    """fp32 [K, N] -> s8 [K, N] and scale(s): 127/absmax per tensor or per output channel, the
    arithmetic of quantizeF32ToI8 (avx512/quantize.cpp:181-234): rne(x * s) clamped to +-127."""
    W = np.asarray(W, np.float32)
    if per_channel:
        mx = np.abs(W).max(axis=0)
    else:
        mx = np.full(W.shape[1], np.abs(W).max(), np.float32)
    s = np.where(mx == 0, np.float32(1), np.float32(127) / mx).astype(np.float32)
    q = np.clip(np.rint((W * s[None, :]).astype(np.float32)), -127, 127).astype(np.int8)
    return q, s


class Linear:
    """One pre-packed layer on the device."""

    def __init__(self, Wq, w_scale, bias=None):
        torch = _torch()
        K, N = Wq.shape
        self.K, self.N = K, N
        desc = tensor2df(DT_I8, DF_NORMAL, K, N)
        nbytes, self.rhs_bytes = matrix_matrix_multiply_transform_rhs_bytes(desc)
        src = torch.from_numpy(np.ascontiguousarray(Wq).view(np.uint8).reshape(-1)).cuda()
        self.packed = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        matrix_matrix_multiply_transform_rhs(desc, C.c_void_p(src.data_ptr()), C.c_void_p(self.packed.data_ptr()))
        torch.cuda.current_stream().synchronize()
        self.Wq_host = Wq  # kept for checks against a CPU computation
        self.w_scale_host = np.asarray(w_scale, np.float32)
        self.uniform = bool(np.all(self.w_scale_host == self.w_scale_host[0]))
        self.w_scale = torch.from_numpy(self.w_scale_host.copy()).cuda()
        self.bias = bias
        self.offsetC_ptr = self.packed.data_ptr() + self.rhs_bytes


class LinearStack:
    """x fp32 [M, K0] -> dynamic per-tensor u8 -> L x (u8 x s8 GEMM with fused requantization)
    -> fp32 [M, N_last].  `out_scales[l]` is the calibrated scale of layer l's u8 output."""

    def __init__(self, layers, M, per_channel=True):
        torch = _torch()
        self.layers = layers
        self.M = M
        self.per_channel = per_channel
        self.out_scales = [None] * len(layers)
        widest = max(max(l.K, l.N) for l in layers)
        self.act = [torch.zeros(M * widest, dtype=torch.uint8, device="cuda") for _ in range(2)]
        self.x_dev = torch.zeros(M * layers[0].K, dtype=torch.float32, device="cuda")
        self.out_dev = torch.zeros(M * layers[-1].N, dtype=torch.float32, device="cuda")
        self.acc_dev = None
        self.d_scale = torch.zeros(4, dtype=torch.float32, device="cuda")
        self.ops_per_step = sum(2 * M * l.K * l.N for l in layers)
        self.launches_per_step = 3 + len(layers)

    # ---- pieces -------------------------------------------------------------------------
    def _gemm(self, l, a_ptr, c_ptr, out_dt, out_scale, sA, d_sA=None, factor=None, warm=None):
        ep = GemmEpilogue()
        # the next layer's packed weight is asked into L2 while this layer computes
        ep.prefetch, ep.prefetch_bytes = (None, 0) if warm is None else (C.c_void_p(warm.packed.data_ptr()), warm.rhs_bytes)
        ep.col_factor = None if factor is None else C.c_void_p(factor.data_ptr())
        ep.out_dt, ep.accumulate, ep.out_scale = out_dt, 0, float(out_scale)
        ep.sA, ep.sB = float(sA), float(l.w_scale_host[0])
        ep.d_sA = d_sA
        ep.row_scale = None
        ep.col_scale = None if l.uniform else C.c_void_p(l.w_scale.data_ptr())
        CHECK_STATUS(lib().bolt_b200_gemm_u8s8_ex(l.N, self.M, l.K, C.c_void_p(a_ptr), C.c_void_p(l.packed.data_ptr()),
                                                  C.c_void_p(l.offsetC_ptr), C.c_void_p(c_ptr), C.byref(ep)), "gemm")

    def quantize_input(self):
        n = self.M * self.layers[0].K
        L = lib()
        CHECK_STATUS(L.bolt_b200_absmax_scale_f32(C.c_void_p(self.x_dev.data_ptr()), n, C.c_void_p(self.d_scale.data_ptr())))
        CHECK_STATUS(L.bolt_b200_quantize_f32_u8_dev(C.c_void_p(self.x_dev.data_ptr()), n,
                                                     C.c_void_p(self.act[0].data_ptr()), C.c_void_p(self.d_scale.data_ptr())))

    def gemms(self):
        """All layers, activations ping-ponging between two device buffers; needs calibrate() first."""
        cur = 0
        sA, d_sA = 1.0, C.c_void_p(self.d_scale.data_ptr())
        last = len(self.layers) - 1
        fac = getattr(self, "layer_factors", None)
        for i, l in enumerate(self.layers):
            f = fac[i] if (fac is not None and i > 0) else None  # layer 0 divides by the dynamic input scale
            if i == last:
                self._gemm(l, self.act[cur].data_ptr(), self.out_dev.data_ptr(), DT_F32, 1.0, sA, d_sA, f)
            else:
                self._gemm(l, self.act[cur].data_ptr(), self.act[1 - cur].data_ptr(), DT_U8_Q, self.out_scales[i], sA, d_sA, f,
                           warm=self.layers[i + 1])
                sA, d_sA = self.out_scales[i], None
                cur = 1 - cur

    def step(self):
        """One pass, device resident: input already in x_dev, result left in out_dev."""
        self.quantize_input()
        self.gemms()

    def calibrate(self):
        """Sets out_scales from one pass over the current x_dev: each layer's int32 accumulators are
        dequantized per channel and 127/absmax of the real-valued output becomes its u8 scale."""
        torch = _torch()
        self.quantize_input()
        torch.cuda.synchronize()
        sA = float(self.d_scale[0].item())
        cur = 0
        for i, l in enumerate(self.layers[:-1]):
            acc = torch.zeros(self.M * l.N, dtype=torch.int32, device="cuda")
            self._gemm(l, self.act[cur].data_ptr(), acc.data_ptr(), DT_I32, 1.0, 1.0)
            torch.cuda.synchronize()
            real = acc.view(self.M, l.N).float() / (np.float32(sA) * l.w_scale[None, :])
            mx = float(real.abs().max().item())
            so = float(np.float32(127.0) / np.float32(mx)) if mx > 0 else 1.0
            self.out_scales[i] = so
            self._gemm(l, self.act[cur].data_ptr(), self.act[1 - cur].data_ptr(), DT_U8_Q, so, sA)
            sA, cur = so, 1 - cur
        torch.cuda.synchronize()
        self._build_factors()

    def _build_factors(self):
        """Per-channel conversion factors of layers 1.. (their input scales are calibrated constants):
        num / (sA * sB[n]) once, instead of a division per column per tile inside the kernels."""
        torch = _torch()
        L = lib()
        n = len(self.layers)
        self.layer_factors = [torch.zeros(l.N, dtype=torch.float32, device="cuda") for l in self.layers]
        sA = None
        for i, l in enumerate(self.layers):
            last = i == n - 1
            num = 1.0 if last else self.out_scales[i]
            if i > 0:
                cs = None if l.uniform else C.c_void_p(l.w_scale.data_ptr())
                CHECK_STATUS(L.bolt_b200_col_factor(num, sA, None, float(l.w_scale_host[0]), cs, l.N,
                                                    C.c_void_p(self.layer_factors[i].data_ptr())), "col_factor")
            if not last:
                sA = self.out_scales[i]
        torch.cuda.synchronize()

    def run_host(self, x_host, out_host):
        """End to end from pinned host memory: H2D of the fp32 input, one pass, D2H of the fp32 output."""
        torch = _torch()
        self.x_dev.copy_(x_host, non_blocking=True)
        self.step()
        out_host.copy_(self.out_dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()


class HostPipeline:
    """Steps fed from, and returned to, pinned host memory with the copies of neighbouring steps overlapping
    the computation: the H2D copy of step i+1 and the D2H copy of step i-1 run on their own streams while
    step i computes (two staging slots on the device, events between the three streams).  Every step still
    moves its whole input and its whole output across PCIe."""

    def __init__(self, stack):
        torch = _torch()
        self.stack = stack
        self.h2d, self.d2h = torch.cuda.Stream(), torch.cuda.Stream()
        self.x_stage = [torch.empty_like(stack.x_dev) for _ in range(2)]
        self.o_stage = [torch.empty_like(stack.out_dev) for _ in range(2)]
        self.ev_in = [torch.cuda.Event() for _ in range(2)]       # input of slot s has arrived
        self.consumed = [torch.cuda.Event() for _ in range(2)]    # slot s's input has been taken over by the step
        self.ev_out = [torch.cuda.Event() for _ in range(2)]      # slot s's output is staged
        self.drained = [torch.cuda.Event() for _ in range(2)]     # slot s's output has left for the host
        cur = torch.cuda.current_stream()
        for e in self.consumed + self.drained:
            e.record(cur)

    def run(self, x_hosts, out_hosts, step_fn=None, before_step=None):
        """x_hosts[i] -> step -> out_hosts[i] for every i; returns when the last output is on the host.
        step_fn: what computes one step from stack.x_dev into stack.out_dev (default stack.step; a CUDA-graph
        replay of it works too); before_step: optional hook enqueued on the compute stream before each step."""
        torch = _torch()
        st = self.stack
        main = torch.cuda.current_stream()
        step_fn = step_fn or st.step
        for i, (xh, oh) in enumerate(zip(x_hosts, out_hosts)):
            s = i & 1
            self.h2d.wait_event(self.consumed[s])
            with torch.cuda.stream(self.h2d):
                self.x_stage[s].copy_(xh, non_blocking=True)
                self.ev_in[s].record(self.h2d)
            main.wait_event(self.ev_in[s])
            main.wait_event(self.drained[s])
            st.x_dev.copy_(self.x_stage[s], non_blocking=True)
            self.consumed[s].record(main)
            if before_step is not None:
                before_step()
            step_fn()
            self.o_stage[s].copy_(st.out_dev, non_blocking=True)
            self.ev_out[s].record(main)
            self.d2h.wait_event(self.ev_out[s])
            with torch.cuda.stream(self.d2h):
                oh.copy_(self.o_stage[s], non_blocking=True)
                self.drained[s].record(self.d2h)
        self.d2h.synchronize()


def bert_base_stack(M=4096, layers=12, hidden=768, inter=3072, per_channel=True, seed=100):
    """BERT-base-shaped linear stack: `layers` x (hidden -> inter -> hidden), weights ~N(0, 0.02)."""
    from . import synth

    ls = []
    for i in range(layers):
        for (k, n, s) in ((hidden, inter, 0), (inter, hidden, 1)):
            W = synth.normal(seed + 2 * i + s, (k, n), 0.02)
            q, sc = quantize_weight_host(W, per_channel)
            ls.append(Linear(q, sc))
    return LinearStack(ls, M, per_channel)
