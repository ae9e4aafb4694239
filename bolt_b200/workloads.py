"""Synthetic workloads for the kernels next to the headline GEMM stack: the FFN-shaped GEMM sweep
and GEMV, the ResNet-50-shaped int8 convolutions, the 1-bit convolution, stand-alone quantize /
dequantize and the tensor-core issue-rate probe.  Each returns a dict of measured
figures; `bench.py --workload NAME` prints it as one JSON line.

Timing: CUDA events on the launching stream, one pair per iteration, a 256 MiB read between
iterations (a read, so that L2 holds neither the workload's lines nor dirty lines whose write-back
would compete with the timed kernel), 3 warm-up iterations.
"""
import ctypes as C

import numpy as np

from . import (CHECK_STATUS, CONVOLUTION_ALGORITHM_NULL, DF_NCHW, DF_NCHWC8, DF_NCHWC16, DF_NORMAL, DT_BIN11, DT_F16,
               DT_F32, DT_I8, DT_I32, DT_U8_Q, GemmEpilogue, conv_param, convolution, convolution_infer_forward_algorithm,
               convolution_infer_forward_tmp_bytes, convolution_infer_output_size, convolution_transform_filter,
               convolution_transform_filter_bytes, lib, matrix_matrix_multiply_transform_rhs,
               matrix_matrix_multiply_transform_rhs_bytes, synth, tensor1d, tensor2df, tensor4df)


def _torch():
    import torch

    return torch


def _p(t, off=0):
    return C.c_void_p(t.data_ptr() + off)


class Timer:
    def __init__(self):
        torch = _torch()
        self.torch = torch
        self.flush = torch.zeros(64 << 20, dtype=torch.float32, device="cuda")  # 256 MiB; fp32 so that sum() only reads

    def evict(self):
        self.sink = self.flush.sum()

    def graph(self, fn):
        """capture fn() (stream-only work) into a CUDA graph on a side stream; returns the replay callable"""
        torch = self.torch
        fn()
        torch.cuda.synchronize()
        st = torch.cuda.Stream()
        lib().bolt_b200_set_stream(C.c_void_p(st.cuda_stream))
        g = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(g, stream=st):
                fn()
        finally:
            lib().bolt_b200_set_stream(None)
        return g.replay

    def run(self, fn, iters=10, warmup=3):
        """mean milliseconds per call of fn()"""
        torch = self.torch
        for _ in range(warmup):
            self.evict()
            fn()
        evs = []
        for _ in range(iters):
            self.evict()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            evs.append((a, b))
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in evs) / iters


def _dev(a):
    torch = _torch()
    return torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(-1).copy()).cuda()


def _packed_weight(K, N, seed):
    """random s8 [K, N] generated on the device (the values do not matter for speed), packed"""
    torch = _torch()
    w = torch.randint(-127, 128, (K, N), dtype=torch.int8, device="cuda", generator=torch.Generator("cuda").manual_seed(seed))
    desc = tensor2df(DT_I8, DF_NORMAL, K, N)
    nbytes, rhs = matrix_matrix_multiply_transform_rhs_bytes(desc)
    packed = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    matrix_matrix_multiply_transform_rhs(desc, _p(w), _p(packed))
    torch.cuda.synchronize()
    return packed, rhs


def _ffn_parity(M, K, N, a, w_host, offs_host, sB, rs, num, c, out_u8, rows):
    """sampled rows of the device result against exact integer accumulators and the defined epilogue
    factor = num / (sA[m] * sB[n]) (binary32 multiply, divide), computed with numpy"""
    A = a[rows].cpu().numpy().astype(np.float64)
    acc = (A @ w_host).astype(np.int64) + offs_host[None, :]   # w_host: float64 copy of the s8 weight, sums exact
    fac = (np.float32(num) / (rs[rows].cpu().numpy().astype(np.float32)[:, None] * sB[None, :])).astype(np.float32)
    f = (acc.astype(np.int32).astype(np.float32) * fac).astype(np.float32)
    if out_u8:
        v = np.rint(f).astype(np.int64) + 128
        want = np.where((v >= 0) & (v <= 255), v, 255).astype(np.uint8)
        got = c.view(M, N)[rows].cpu().numpy()
    else:
        want = f
        got = c.view(_torch().float32).view(M, N)[rows].cpu().numpy()
    return bool(got.tobytes() == want.tobytes())


def ffn_sweep(peaks, iters=5):
    """u8 x s8 GEMM, K 8192, N 28672, M in {16, 128, 2048, 16384}: weights s8 with one scale per output
    channel, activations u8 with one scale per token, u8 (requantized) and fp32 outputs; a sample of rows of
    every result is compared bit for bit with a numpy computation."""
    torch = _torch()
    L, tm = lib(), Timer()
    K, N = 8192, 28672
    gen = torch.Generator("cuda").manual_seed(1)
    w = torch.randint(-127, 128, (K, N), dtype=torch.int8, device="cuda", generator=gen)
    desc = tensor2df(DT_I8, DF_NORMAL, K, N)
    nbytes, rhs = matrix_matrix_multiply_transform_rhs_bytes(desc)
    packed = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    matrix_matrix_multiply_transform_rhs(desc, _p(w), _p(packed))
    torch.cuda.synchronize()
    w_host = w.cpu().numpy().astype(np.float64)
    del w
    offs_host = packed[rhs: rhs + 4 * N].cpu().numpy().view(np.int32).astype(np.int64)
    sB_host = (np.float32(127.0) / (np.float32(0.05) + np.float32(0.02) * np.abs(synth.normal(7, (N,))))).astype(np.float32)
    sB = torch.from_numpy(sB_host).cuda()
    L.bolt_b200_set_pointer_mode(1)
    rows = []
    for M in (16, 128, 2048, 16384):
        a = torch.randint(0, 256, (M, K), dtype=torch.uint8, device="cuda", generator=gen)
        rs = (torch.rand(M, device="cuda", generator=gen) * 20 + 30).float()       # per-token activation scales
        for out_u8 in (True, False):
            c = torch.empty(M * N * (1 if out_u8 else 4), dtype=torch.uint8, device="cuda")
            ep = GemmEpilogue()
            ep.out_dt, ep.accumulate, ep.out_scale = (DT_U8_Q if out_u8 else DT_F32), 0, 40.0
            ep.sA, ep.sB = 1.0, 1.0
            ep.row_scale, ep.col_scale = _p(rs), _p(sB)
            call = lambda: L.bolt_b200_gemm_u8s8_ex(N, M, K, _p(a), _p(packed), _p(packed, rhs), _p(c), C.byref(ep))
            ms = tm.run(call, iters)
            sample = np.unique(np.linspace(0, M - 1, 6).astype(np.int64))
            ok = _ffn_parity(M, K, N, a, w_host, offs_host, sB_host, rs, 40.0 if out_u8 else 1.0, c, out_u8, sample)
            ops = 2.0 * M * N * K
            rows.append({"M": M, "out": "u8" if out_u8 else "f32", "ms": ms, "tops": ops / ms / 1e9,
                         "weight_GBps": K * N / ms / 1e6, "parity_rows": int(len(sample)), "parity": ok,
                         "tensor_cores": int(L.bolt_b200_last_gemm_used_tensor_cores())})
            del c
    L.bolt_b200_set_pointer_mode(0)
    best = max(rows, key=lambda r: r["tops"])
    return {"workload": "ffn_gemm_sweep K=8192 N=28672, per-channel weight scales, per-token activation scales",
            "rows": rows, "best_tops": best["tops"],
            "frac_of_2x_bf16_burst": best["tops"] / (2.0 * peaks["bf16_tflops"]),
            "frac_of_2x_bf16_sustained": best["tops"] / (2.0 * peaks["bf16_tflops_sustained"]),
            "frac_of_nominal_4500": best["tops"] / 4500.0,
            "roofs": "M 16, 128: the 235 MB weight stream (HBM); M >= 2048: tensor pipe under the board power limit"}


def i8_peak(peaks):
    """tcgen05.mma.kind::i8 issue rate with nothing else in the way: a burst (about a millisecond) and
    a run of seconds (under the power limit)."""
    L = lib()
    ms, tops = C.c_float(), C.c_float()
    out = {}
    for name, n in (("burst", 8192), ("sustained", 24000000)):
        CHECK_STATUS(L.bolt_b200_i8_mma_rate(n, C.byref(ms), C.byref(tops)), "i8_mma_rate")
        out[name] = {"mma_per_sm": n, "ms": ms.value, "tops": tops.value}
    return {"workload": "i8_peak: back-to-back tcgen05.mma.kind::i8 128x256x32, one CTA per SM, no loads", **out,
            "nominal_dense_int8_tops": 4500.0, "two_x_bf16_burst": 2.0 * peaks["bf16_tflops"],
            "two_x_bf16_sustained": 2.0 * peaks["bf16_tflops_sustained"]}


def gemv(peaks, iters=20):
    """M = 1: y = W x, W s8 [28672, 8192] pre-packed, x u8, int32 / fp32 / u8 outputs."""
    torch = _torch()
    from . import (DF_NKN32K4, matrix_vector_multiply_transform_weight, matrix_vector_multiply_transform_weight_bytes)

    L, tm = lib(), Timer()
    N, K = 28672, 8192
    w = torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda")
    desc = tensor2df(DT_I8, DF_NORMAL, N, K)
    nb = matrix_vector_multiply_transform_weight_bytes(desc)
    packed = torch.zeros(nb, dtype=torch.uint8, device="cuda")
    matrix_vector_multiply_transform_weight(desc, _p(w), _p(packed))
    torch.cuda.synchronize()
    del w
    x = torch.randint(0, 256, (K,), dtype=torch.uint8, device="cuda")
    y = torch.zeros(N, dtype=torch.int32, device="cuda")
    off = ((N + 15) // 16 * 16) * ((K + 7) // 8 * 8)
    L.bolt_b200_set_pointer_mode(1)
    scale = (C.c_float * 2)(-1.0, 0.001)
    out = {}
    for name, sp in (("s32", None), ("u8", C.cast(scale, C.POINTER(C.c_float)))):
        ms = tm.run(lambda: CHECK_STATUS(L.mvm_cuda_b200(N, K, DT_I8, DF_NKN32K4, _p(packed), _p(x), _p(y), _p(packed, off), sp)), iters)
        bytes_ = N * K + K + 4 * N + (4 * N * 2 if sp is None else N)
        out[name] = {"us": ms * 1e3, "GBps": bytes_ / ms / 1e6, "frac_of_hbm": bytes_ / ms / 1e6 / peaks["hbm_gbs"]}
    L.bolt_b200_set_pointer_mode(0)
    return {"workload": "gemv N=28672 K=8192", **out}


def quantize(peaks, iters=20):
    """stand-alone quantize / requantize / dequantize on a 16384 x 3072 tensor (four batches of
    4096 x 3072 activations: 201 MB of fp32, larger than L2)."""
    torch = _torch()
    L, tm = lib(), Timer()
    n = 16384 * 3072
    x = torch.randn(n, device="cuda")
    acc = torch.randint(-100000, 100000, (n,), dtype=torch.int32, device="cuda")
    q = torch.empty(n, dtype=torch.uint8, device="cuda")
    f = torch.empty(n, dtype=torch.float32, device="cuda")
    ds = torch.zeros(4, dtype=torch.float32, device="cuda")
    hbm = peaks["hbm_gbs"]
    res = {}

    def dyn():
        L.bolt_b200_absmax_scale_f32(_p(x), n, _p(ds))
        L.bolt_b200_quantize_f32_u8_dev(_p(x), n, _p(q), _p(ds))

    ms = tm.run(dyn, iters)
    res["f32_to_u8_dynamic"] = {"us": ms * 1e3, "GBps_5B_per_elem": 5.0 * n / ms / 1e6, "GBps_9B_per_elem": 9.0 * n / ms / 1e6,
                                "frac_of_hbm_9B": 9.0 * n / ms / 1e6 / hbm}
    ms = tm.run(lambda: L.bolt_b200_quantize_f32_u8_dev(_p(x), n, _p(q), _p(ds)), iters)
    res["f32_to_u8_given_scale"] = {"us": ms * 1e3, "GBps": 5.0 * n / ms / 1e6, "frac_of_hbm": 5.0 * n / ms / 1e6 / hbm}
    L.bolt_b200_set_pointer_mode(1)
    qd, dd = tensor1d(DT_I32, n), tensor1d(DT_F32, n)
    bd = tensor1d(DT_F32, 0)
    sc = (C.c_float * 1)(0.37)
    ms = tm.run(lambda: L.dequantize_cuda_b200(C.byref(qd), _p(acc), C.cast(sc, C.POINTER(C.c_float)), C.byref(bd), None,
                                               C.byref(dd), _p(f)), iters)
    res["i32_to_f32"] = {"us": ms * 1e3, "GBps": 8.0 * n / ms / 1e6, "frac_of_hbm": 8.0 * n / ms / 1e6 / hbm}
    L.bolt_b200_set_pointer_mode(0)
    return {"workload": "quantize 16384x3072", **res}


# (ic, hw, oc, k, stride, pad): the 22 distinct ResNet-50 layer shapes after the stem
RESNET50_LAYERS = [
    (64, 56, 64, 1, 1, 0), (64, 56, 64, 3, 1, 1), (64, 56, 256, 1, 1, 0), (256, 56, 64, 1, 1, 0), (256, 56, 128, 1, 1, 0),
    (128, 56, 128, 3, 2, 1), (256, 56, 512, 1, 2, 0),
    (128, 28, 128, 3, 1, 1), (128, 28, 512, 1, 1, 0), (512, 28, 128, 1, 1, 0), (512, 28, 256, 1, 1, 0),
    (256, 28, 256, 3, 2, 1), (512, 28, 1024, 1, 2, 0),
    (256, 14, 256, 3, 1, 1), (256, 14, 1024, 1, 1, 0), (1024, 14, 256, 1, 1, 0), (1024, 14, 512, 1, 1, 0),
    (512, 14, 512, 3, 2, 1), (1024, 14, 2048, 1, 2, 0),
    (512, 7, 512, 3, 1, 1), (512, 7, 2048, 1, 1, 0), (2048, 7, 512, 1, 1, 0)]


def resnet_conv(peaks, batch=64, iters=5, out_u8=False, once=False):
    """int8 convolution, NCHWc16 u8 input, fused bias + ReLU; fp32 output, or u8 output requantized in
    the epilogue with a known output scale.  once: every layer is launched a single time and nothing is timed
    (one launch per layer for a profiler to capture)."""
    torch = _torch()
    L, tm = lib(), Timer()
    rows, tot_ops, tot_ms, tot_roof = [], 0.0, 0.0, 0.0
    calls, keep = [], []
    peak_tensor = 2.0 * peaks["bf16_tflops"]   # TOP/s: no int8 entry in the measured peaks, 2 x the bf16 burst figure
    target = DT_U8_Q if out_u8 else DT_F32
    for (ic, hw, oc, k, st, pad) in RESNET50_LAYERS:
        p = conv_param(oc, k, k, st, pad, 1, True)
        in_desc = tensor4df(DT_U8_Q, DF_NCHWC16, batch, ic, hw, hw)
        f_desc = tensor4df(DT_I8, DF_NCHW, oc, ic, k, k)
        out_desc = convolution_infer_output_size(in_desc, f_desc, p, target)
        oh = out_desc.dims[1]
        alg = convolution_infer_forward_algorithm(in_desc, f_desc, out_desc, p, target)
        w = torch.randint(-127, 128, (oc * ic * k * k,), dtype=torch.int8, device="cuda")
        ftm = torch.zeros(convolution_transform_filter_bytes(f_desc, p, alg), dtype=torch.uint8, device="cuda")
        ftm_desc = convolution_transform_filter(f_desc, _p(w), p, alg, _p(ftm))
        tb = convolution_infer_forward_tmp_bytes(in_desc, ftm_desc, out_desc, p, alg)
        x = torch.randint(128, 256, (batch * ic * hw * hw,), dtype=torch.uint8, device="cuda")
        bias = torch.randn(oc, device="cuda") * 0.1
        tmp = torch.empty(tb, dtype=torch.uint8, device="cuda")
        out = torch.empty(batch * oc * oh * oh * (1 if out_u8 else 4), dtype=torch.uint8, device="cuda")
        sc = [31.75, -1.0, 635.0]
        known_out_scale = 9.5 if out_u8 else None      # u8 output: known output scale, fused requantization
        L.bolt_b200_set_pointer_mode(1)

        def call(in_desc=in_desc, x=x, ftm_desc=ftm_desc, ftm=ftm, p=p, alg=alg, sc=sc, bias=bias, tb=tb, tmp=tmp,
                 out_desc=out_desc, out=out):
            convolution(in_desc, _p(x), ftm_desc, _p(ftm), p, alg, list(sc), _p(bias), tb, _p(tmp), out_desc, _p(out), True,
                        None, known_out_scale)

        if once:
            tm.evict()
            call()
            torch.cuda.synchronize()
            L.bolt_b200_set_pointer_mode(0)
            rows.append({"layer": "%dx%d %d->%d @%d s%d" % (k, k, ic, oc, hw, st)})
            continue
        fn = tm.graph(call)  # neither path leaves the stream: replay as a CUDA graph (no host time inside)
        ms = tm.run(fn, iters)
        L.bolt_b200_set_pointer_mode(0)
        calls.append(call)
        keep.append((w, ftm, x, tmp, out, bias))
        ops = 2.0 * batch * oc * oh * oh * ic * k * k
        # algorithmic bytes: input + filter + output once
        nbytes = batch * ic * hw * hw + oc * ic * k * k + batch * oc * oh * oh * (1 if out_u8 else 4)
        t_tensor = ops / (peak_tensor * 1e12) * 1e3
        t_hbm = nbytes / (peaks["hbm_gbs"] * 1e9) * 1e3
        roof_ms = max(t_tensor, t_hbm)
        rows.append({"layer": "%dx%d %d->%d @%d s%d" % (k, k, ic, oc, hw, st), "ms": ms, "tops": ops / ms / 1e9,
                     "GBps": nbytes / ms / 1e6, "bound": "tensor" if t_tensor >= t_hbm else "hbm",
                     "roof_ms": roof_ms, "frac_of_roof": roof_ms / ms})
        tot_ops += ops
        tot_ms += ms
        tot_roof += roof_ms
    if once:
        return {"workload": "resnet50_int8_conv batch %d (%s out), one launch per layer" % (batch, "u8" if out_u8 else "fp32"),
                "rows": rows}
    # all 22 layers one after the other as one graph (each on its own buffers, 256 MiB evicted before every pass):
    # what a network pass costs, without the front-end latency that a graph of a single short kernel shows
    L.bolt_b200_set_pointer_mode(1)

    def one_pass():
        for c in calls:
            c()

    pass_ms = tm.run(tm.graph(one_pass), iters)
    L.bolt_b200_set_pointer_mode(0)
    del keep[:]
    torch.cuda.empty_cache()
    return {"workload": "resnet50_int8_conv batch %d (%s out)" % (batch, "u8" if out_u8 else "fp32"), "rows": rows,
            "total_ms": tot_ms, "tops": tot_ops / tot_ms / 1e9, "roof_total_ms": tot_roof, "frac_of_roof": tot_roof / tot_ms,
            "pass_ms": pass_ms, "pass_tops": tot_ops / pass_ms / 1e9, "pass_frac_of_roof": tot_roof / pass_ms,
            "pass": "the 22 layers back to back in one CUDA graph; rows[] are single-layer graphs timed one at a time",
            "roof": "per layer max(ops / (2 x bf16_tflops), algorithmic bytes / hbm_gbs); `bound` names the binding one"}


def pooling(peaks, iters=10):
    """u8 pooling, NCHWc16: the 3x3 stride-2 maximum after a ResNet stem (64 x 112 x 112, batch 256: 206 MB in, 51 MB
    out -- larger than L2) and a 2x2 stride-2 mean on 256 x 56 x 56."""
    from . import pooling as pool_call, pooling_param
    torch = _torch()
    L, tm = lib(), Timer()
    rows = []
    for name, (n, c, hw, k, s, pad, mean) in (("max 3x3 s2 p1 64x112x112 b256", (256, 64, 112, 3, 2, 1, False)),
                                              ("mean 2x2 s2 256x56x56 b256", (256, 256, 56, 2, 2, 0, True))):
        oh = (hw + 2 * pad - k) // s + 1
        x = torch.randint(128, 256, (n * c * hw * hw,), dtype=torch.uint8, device="cuda")
        y = torch.empty(n * c * oh * oh, dtype=torch.uint8, device="cuda")
        in_desc = tensor4df(DT_U8_Q, DF_NCHWC16, n, c, hw, hw)
        out_desc = tensor4df(DT_U8_Q, DF_NCHWC16, n, c, oh, oh)
        pp = pooling_param(k, s, pad, mean)
        L.bolt_b200_set_pointer_mode(1)

        def call(in_desc=in_desc, x=x, pp=pp, out_desc=out_desc, y=y):
            pool_call(in_desc, _p(x), pp, [1.0, 0.0], out_desc, _p(y))

        ms = tm.run(tm.graph(call), iters)
        L.bolt_b200_set_pointer_mode(0)
        nbytes = x.numel() + y.numel()
        rows.append({"case": name, "ms": ms, "GBps": nbytes / ms / 1e6, "frac_of_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"]})
        del x, y
    return {"workload": "u8 pooling NCHWc16 (algorithmic bytes: input + output once)", "rows": rows}


def bnn(peaks, batch=128, iters=5):
    """1-bit 3x3 convolution, C 256 -> 256, 28 x 28, pad 1, XNOR mode, fp16 NCHWc8 in and out."""
    torch = _torch()
    L, tm = lib(), Timer()
    ic = oc = 256
    hw, k = 28, 3
    p = conv_param(oc, k, k, 1, 1)
    in_desc = tensor4df(DT_F16, DF_NCHWC8, batch, ic, hw, hw)
    f_desc = tensor4df(DT_BIN11, DF_NCHW, oc, ic, k, k)
    out_desc = tensor4df(DT_F16, DF_NCHWC8, batch, oc, hw, hw)
    alg = convolution_infer_forward_algorithm(in_desc, f_desc, out_desc, p, DT_F16)
    wbits = torch.randint(0, 256, (oc * ic * k * k // 8,), dtype=torch.uint8, device="cuda")
    ftm = torch.zeros(convolution_transform_filter_bytes(f_desc, p, alg), dtype=torch.uint8, device="cuda")
    ftm_desc = convolution_transform_filter(f_desc, _p(wbits), p, alg, _p(ftm))
    tb = convolution_infer_forward_tmp_bytes(in_desc, ftm_desc, out_desc, p, alg)
    x = torch.randn(batch * ic * hw * hw, device="cuda").half()
    alpha = (torch.rand(oc, device="cuda") * 0.1 + 0.01).half()
    beta = torch.zeros(oc, device="cuda").half()
    tmp = torch.empty(tb, dtype=torch.uint8, device="cuda")
    out = torch.empty(batch * oc * hw * hw, dtype=torch.float16, device="cuda")
    L.bolt_b200_set_pointer_mode(1)
    ms = tm.run(lambda: convolution(in_desc, _p(x), ftm_desc, _p(ftm), p, alg, _p(alpha), _p(beta), tb, _p(tmp), out_desc, _p(out)),
                iters)
    L.bolt_b200_set_pointer_mode(0)
    words = batch * hw * hw * oc * (k * k * ic // 32)
    bytes_ = x.numel() * 2 + out.numel() * 2 + oc * ic * k * k // 8
    return {"workload": "bnn_xnor 3x3 C256 28x28 batch %d" % batch, "ms": ms, "Gword_ops_per_s": words / ms / 1e6,
            "frac_of_popc_issue_nominal": words / ms / 1e6 / (16 * 148 * 1.965), "GBps": bytes_ / ms / 1e6,
            "frac_of_hbm": bytes_ / ms / 1e6 / peaks["hbm_gbs"],
            "note": "bound by the popcount issue rate (nominal: 16 per clock per SM x 148 SMs x 1.965 GHz = 4.65 T/s), not by HBM"}


def resnet_conv_u8_once(peaks):
    return resnet_conv(peaks, out_u8=True, once=True)


def resnet_conv_u8(peaks):
    return resnet_conv(peaks, out_u8=True)


WORKLOADS = {"ffn": ffn_sweep, "gemv": gemv, "quantize": quantize, "resnet_conv": resnet_conv, "resnet_conv_u8_once": resnet_conv_u8_once,
             "resnet_conv_u8": resnet_conv_u8, "bnn": bnn, "i8_peak": i8_peak, "pooling": pooling}
