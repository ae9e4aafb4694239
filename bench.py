#!/usr/bin/env python
"""Benchmark of the quantized GEMM path on the BERT-base-shaped int8 linear stack.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

A step is one pass of 4096 tokens through 12 x (768 -> 3072 -> 768) quantized linear layers:
dynamic per-tensor u8 quantization of the fp32 input, 24 u8 x s8 GEMMs with per-output-channel
weight scales and fused requantization to u8 between layers, fp32 output.  Synthetic seeded data.

`value`  : int8 GEMM TOP/s (2*M*N*K ops of the 24 GEMMs) with the input resident in HBM,
           the whole step replayed as one CUDA graph, L2 flushed between timed steps.  One GEMM launch
           per layer.
`e2e`    : the same metric through LinearStack.run_host: pinned host input -> H2D -> step -> D2H.
`roofline`: the tcgen05 GEMM kernel alone (24 launches per pass) against the int8 issue rate measured on the same GPU
(and, beside it, 2 x the measured bf16 peak).
`cpu_baseline` / --impl reference: the reference's own x86 AVX512-VNNI code (or the scalar oracle
           port when that cannot run) on the host cores, same shapes, bounded sample.
With N > 1 every rank runs its own 4096-token batch (weak scaling, no collective on the data path).
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M_TOKENS, LAYERS, HIDDEN, INTER = 4096, 12, 768, 3072
OPS_PER_STEP = 2 * M_TOKENS * HIDDEN * INTER * 2 * LAYERS  # 463.86 GOP
WORKLOAD = "bert_base_int8_linear_stack: 12 x (768->3072->768), M=4096 tokens, s8 per-channel weights, u8 per-tensor activations, fused requant, fp32 out"
# dram__bytes_read.sum + dram__bytes_write.sum per launch of gemm_u8s8_tcgen05_kernel, averaged over
# the 24 launches of one pass (profiles/gemm_u8s8_tcgen05_bert_stack.md).
GEMM_DRAM_TRAFFIC_PER_LAUNCH = 12536085


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except (OSError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 50 ms while the measured passes run."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, pw, reasons = [], [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                pw.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_min_mhz": min(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "power_w": float(np.median(pw)) if pw else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------ CPU arm
def cpu_stack_baseline(seconds=12.0, threads=None):
    """The reference's CPU path for the same stack: per layer an int8 GEMM through Bolt's
    matrix_matrix_multiply (pre-packed weight, int32 out, OpenMP over all host threads -- the only
    part of the path the reference threads, mmm_avx512_vnni.cpp:1858-1860) followed by its
    I32 -> U8_Q requantization (quantize_x86, single thread as shipped)."""
    import oracle as O
    from bolt_b200 import synth
    from bolt_b200.linear_stack import quantize_weight_host

    cores = threads or os.cpu_count() or 1
    if O.ref is not None:
        kind, m = "reference", M_TOKENS
        O.ref.ref_set_threads(cores)
    else:
        kind, m, cores = "port", 64, 1
    shapes = [(HIDDEN, INTER), (INTER, HIDDEN)]
    ws = [quantize_weight_host(synth.normal(100 + i, s, 0.02), False)[0] for i, s in enumerate(shapes)]
    acts = [synth.u8(7, (m, HIDDEN)), synth.u8(8, (m, INTER))]
    if kind == "reference":
        plans = [O.ref.ref_gemm_plan(m, n, k, 0, 0, O.ptr(w), 0) for (k, n), w in zip(shapes, ws)]
        accs = [np.zeros((m, n), np.int32) for (_, n) in shapes]
        qs = [np.zeros(m * n, np.uint8) for (_, n) in shapes]

        def layer_pair():
            for j in range(2):
                accs[j][...] = 0
                O.ref.ref_gemm_run(plans[j], O.ptr(acts[j]), O.ptr(accs[j]), None, None)
                sc = np.array([0.5, 300.0], np.float32)
                O.ref.ref_quantize(accs[j].size, O.DT_I32, O.ptr(accs[j]), O.DT_U8_Q, O.ptr(qs[j]), O.ptr(sc), 0)
    else:
        offs = [O.port_offsetc(w) for w in ws]

        def layer_pair():
            for j in range(2):
                O.port_gemm(acts[j], ws[j], offs[j], [-1, 0.002])

    layer_pair()  # warm-up
    t0 = time.perf_counter()
    pairs = 0
    while True:
        layer_pair()
        pairs += 1
        el = time.perf_counter() - t0
        if el > seconds or (kind == "reference" and pairs >= 10 * LAYERS):
            break
    if kind == "reference":
        for p in plans:
            O.ref.ref_gemm_free(p)
    ops = pairs * 2 * m * HIDDEN * INTER * 2
    tops = ops / el / 1e12
    sample = "%d layer pairs (768->3072->768) at M=%d, %s, %.1f s" % (
        pairs, m, "Bolt x86 AVX512-VNNI GEMM (OpenMP) + single-thread requantize" if kind == "reference"
        else "scalar oracle port (host CPU lacks avx512_vnni or the reference build is absent)", el)
    return {"value": tops, "unit": "TOP/s", "cores": cores, "kind": kind, "sample": sample}, el / pairs * LAYERS


def run_reference_arm(args, rank):
    if rank != 0:
        return
    base, step_s = cpu_stack_baseline(seconds=max(5.0, min(60.0, 4.0 * (args.steps + args.warmup))))
    line = {
        "impl": "reference", "metric": "int8_gemm_tops", "value": base["value"], "unit": "TOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8*s8->s32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": "host CPU run"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------ GPU arm
def check_rows_against_numpy(stack, x, rows):
    """The step's arithmetic restated with numpy on a few token rows (rows are independent once the
    dynamic input scale is fixed): F32 -> U8_Q as quantizeF32ToU8 does it, exact integer accumulators,
    factor[n] = num / (sA * sB[n]) in binary32, u8 = usat8(rne(acc * factor) + 128) between layers, fp32
    at the end.  Returns True when the device output rows carry the same bits."""
    sA = np.float32(stack.d_scale[0].item())
    xr = x.reshape(stack.M, -1)[rows].astype(np.float32)
    act = np.clip(np.rint((xr * sA).astype(np.float32) + np.float32(128)), 1, 255).astype(np.uint8)
    last = len(stack.layers) - 1
    for i, l in enumerate(stack.layers):
        W = l.Wq_host.astype(np.float64)
        acc = (act.astype(np.float64) @ W - 128.0 * W.sum(axis=0)[None, :]).astype(np.int64).astype(np.int32)
        num = np.float32(1.0) if i == last else np.float32(stack.out_scales[i])
        fac = (num / (sA * l.w_scale_host)).astype(np.float32)
        f = (acc.astype(np.float32) * fac[None, :]).astype(np.float32)
        if i == last:
            got = stack.out_dev.cpu().numpy().reshape(stack.M, -1)[rows]
            return got.tobytes() == f.tobytes()
        v = np.rint(f).astype(np.int64) + 128
        act = np.where((v >= 0) & (v <= 255), v, 255).astype(np.uint8)
        sA = np.float32(stack.out_scales[i])
    return False


def run_sharded_record(rank, world, lib, dist, stream, evict):
    """The N-split of the FFN-shaped GEMM (K 8192, N 28672, per-channel weight scales, per-token activation
    scales, u8 output) on `world` GPUs: every rank owns N / world output columns; the blocks are assembled on
    every rank with an NCCL all-gather over NVLink.  Per M: this rank's GEMM alone, the all-gather alone, and
    both with the gather of one row chunk overlapping the GEMM of the next; device times, maximum over ranks.
    Rank 0 also runs the whole product on its own GPU: the strong-scaling reference and, for M <= 128, the
    bytes the gathered result has to equal."""
    import torch

    from bolt_b200.sharded import ShardedFFN

    K, N = 8192, 28672
    ffn = ShardedFFN(rank, world, K, N)
    # the fused variant needs buffers shared between the processes; every rank tries the set-up and one call, and
    # the ranks agree on the outcome, so that a rank on which it is unavailable cannot leave the others waiting
    fused_note = None
    try:
        ffn.setup_fused()
        ffn.fused_compute(128)
        torch.cuda.synchronize()
        mine = 1
    except Exception as exc:   # noqa: BLE001 -- reported in the record
        mine, fused_note = 0, "%s: %s" % (type(exc).__name__, exc)
    agreed = torch.tensor([mine], device="cuda")
    dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
    fused_on = bool(agreed.item() == 1)
    one = None
    if rank == 0:
        # the unsplit problem on one GPU: all shards side by side
        w = torch.cat([ffn.shard_weight(r) for r in range(world)], dim=1).contiguous()
        one = ShardedFFN(0, 1, K, N, weight=w, like=ffn)
        del w

    def timed(fn, iters=7):
        """median of `iters` device times (each after an L2 eviction), maximum over ranks"""
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            evict()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            fn()
            b.record(stream)
            b.synchronize()
            ts.append(a.elapsed_time(b))
        t = torch.tensor([sorted(ts)[len(ts) // 2]], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    rows = []
    for M in (1, 128, 2048, 16384):
        ms_c = timed(lambda: ffn.compute(M))
        ms_g = timed(lambda: ffn.gather(M))
        ms_o = timed(lambda: ffn.overlapped(M)) if M >= 2048 else None
        # the gather fused into the GEMM's epilogue (peer stores) + a one-element all-reduce as the barrier
        ms_f = timed(lambda: ffn.fused(M)) if (M >= 128 and fused_on) else None
        ops = 2.0 * M * N * K
        gathered = (world - 1) / world * M * N            # bytes every rank receives
        row = {"M": M, "compute_ms": ms_c, "gather_ms": ms_g, "overlapped_ms": ms_o,
               "compute_tops_all_gpus": ops / ms_c / 1e9,
               "gather_GBps_in_per_gpu": gathered / ms_g / 1e6,
               "fused_ms": ms_f}
        cands = [(ms_c + ms_g, "compute then gather")]
        if ms_o is not None:
            cands.append((ms_o, "overlapped"))
        if ms_f is not None:
            cands.append((ms_f, "fused peer stores"))
        row["end_to_end_ms"], row["end_to_end_mode"] = min(cands)
        if ms_f is not None:
            sent = (world - 1) * M * (N // world)          # bytes this rank stores into its peers
            row["fused_GBps_out_per_gpu"] = sent / ms_f / 1e6
            row["fused_roof_ms"] = max(sent / 770e9 * 1e3, 2.0 * M * (N // world) * K / (2 * 1637.4e12) * 1e3)
        row["end_to_end_tops"] = ops / row["end_to_end_ms"] / 1e9
        nvlink_ms = gathered / 770e9 * 1e3                 # measured peer-copy rate per direction on this pool
        row["nvlink_roof_ms"] = nvlink_ms
        row["limiter"] = ("collective latency" if M <= 128 else
                          ("NVLink (gather longer than the GEMM)" if ms_g > ms_c else "tensor pipe (GEMM longer than the gather)"))
        parity = None
        if rank == 0:
            t1 = []
            for i in range(8):
                evict()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                one.compute(M)
                b.record(stream)
                b.synchronize()
                if i > 0:
                    t1.append(a.elapsed_time(b))
            row["one_gpu_ms"] = sorted(t1)[len(t1) // 2]
            row["compute_speedup"] = row["one_gpu_ms"] / ms_c
            row["compute_efficiency"] = row["compute_speedup"] / world
            row["end_to_end_speedup"] = row["one_gpu_ms"] / row["end_to_end_ms"]
        if M <= 128:
            # gathered [M, N] on every rank against rank 0's single-GPU bytes
            ffn.compute(M)
            ffn.gather(M)
            torch.cuda.synchronize()
            ref = torch.empty(M * N, dtype=torch.uint8, device="cuda")
            if rank == 0:
                ref.copy_(one.block[: M * N])
            dist.broadcast(ref, 0)
            same = torch.equal(ffn.assembled(M).reshape(-1), ref)
            if M >= 128 and fused_on:
                ffn.fused(M)
                torch.cuda.synchronize()
                same = same and torch.equal(ffn.fused_result(M).reshape(-1), ref)
            ok = torch.tensor([1 if same else 0], device="cuda")
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            parity = bool(ok.item() == 1)
        row["parity"] = parity
        rows.append(row)
    torch.cuda.synchronize()
    dist.barrier()
    ffn.close_fused()
    if not fused_on and fused_note is None:
        fused_note = "unavailable on another rank"
    return {"fused_available": fused_on, "fused_note": fused_note,
            "workload": "ffn N-split: K=8192 N=28672 u8 out, per-channel / per-token scales, M=1 through the GEMV kernel",
            "world": world, "columns_per_gpu": N // world, "rows": rows,
            "mode": "gather = one all_gather_into_tensor of [M, N/world] u8 blocks into a shard-major buffer; "
                    "overlapped = 4 row chunks, gather of chunk i on a side stream while chunk i+1 computes; "
                    "fused = bolt_b200_gemm_u8s8_scatter: the epilogue stores every tile into all ranks' [M, N] results "
                    "(TMA stores to peer memory over NVLink), then a one-element all-reduce as the barrier"}


def run_b200_arm(args, rank, world, local_rank):
    import torch

    import bolt_b200 as B
    from bolt_b200 import synth
    from bolt_b200.linear_stack import bert_base_stack

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the B200 arm has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    lib = B.load(build_if_missing=False)
    B.CHECK_STATUS(lib.bolt_b200_set_device(local_rank))
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    B.CHECK_STATUS(lib.bolt_b200_set_stream(C.c_void_p(stream.cuda_stream)))

    stack = bert_base_stack(M_TOKENS, LAYERS, HIDDEN, INTER, per_channel=True)
    x_host = torch.from_numpy(synth.normal(1000 + rank, (M_TOKENS, HIDDEN))).reshape(-1).pin_memory()
    out_host = torch.zeros(M_TOKENS * HIDDEN, dtype=torch.float32).pin_memory()
    stack.x_dev.copy_(x_host)
    stack.calibrate()
    # the timed computation against a CPU computation of the same step, on a sample of token rows
    stack.step()
    torch.cuda.synchronize()
    parity_rows = np.unique(np.linspace(0, M_TOKENS - 1, 24).astype(np.int64))
    parity_ok = bool(check_rows_against_numpy(stack, x_host.numpy(), parity_rows))
    if not parity_ok:
        raise SystemExit("bench.py: the device output differs from the CPU computation on the sampled rows")
    B.CHECK_STATUS(lib.bolt_b200_set_pointer_mode(1))
    flush = torch.zeros(64 << 20, dtype=torch.float32, device="cuda")  # 256 MiB = 2 x L2; fp32 so that sum() only reads
    sink = []

    def evict():
        sink[:] = [flush.sum()]

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # eager warm-up (also sets kernel attributes before any capture)
    step_eager = stack.step
    gemm_eager = stack.gemms  # the dominant kernel alone: the 24 GEMM launches
    for _ in range(max(args.warmup, 3)):
        step_eager()
    torch.cuda.synchronize()
    launch_mode = "cuda_graph"
    g_step = g_gemm = None
    try:
        g_step = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_step, stream=stream):
            step_eager()
        g_gemm = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_gemm, stream=stream):
            gemm_eager()
        g_step.replay()
        g_gemm.replay()
        torch.cuda.synchronize()
    except Exception as e:  # capture refused: time plain stream launches instead
        launch_mode = "stream (graph capture failed: %s)" % type(e).__name__
        g_step = g_gemm = None
    B.CHECK_STATUS(lib.bolt_b200_set_stream(C.c_void_p(stream.cuda_stream)))

    def timed(fn, steps):
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for a, b in evs:
            evict()                 # read 256 MiB: L2 keeps neither this workload's lines nor dirty ones
            a.record(stream)
            fn()
            b.record(stream)
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in evs) / 1e3

    step_fn = g_step.replay if g_step is not None else step_eager
    gemm_fn = g_gemm.replay if g_gemm is not None else gemm_eager
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # sampled from the warm-up to the end of the e2e pass: the timed region alone is ~10 ms
    for _ in range(args.warmup):
        evict()
        step_fn()
    barrier()
    launches0 = lib.bolt_b200_launch_count()
    wall0 = time.perf_counter()
    dev_s = timed(step_fn, args.steps)
    barrier()
    wall_s = time.perf_counter() - wall0
    launches = lib.bolt_b200_launch_count() - launches0
    if g_step is not None:
        launches = stack.launches_per_step * args.steps  # replays re-launch the captured kernels
    # roofline pass: the GEMM launches alone
    gemm_s = timed(gemm_fn, args.steps)
    # end to end through the public host API
    for _ in range(2):
        stack.run_host(x_host, out_host)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        evict()
        torch.cuda.synchronize()
    flush_s = time.perf_counter() - t0
    t0 = time.perf_counter()
    for _ in range(args.steps):
        evict()
        stack.run_host(x_host, out_host)
    torch.cuda.synchronize()
    e2e_serial_s = max(time.perf_counter() - t0 - flush_s, 1e-9)
    # the same steps with the copies of neighbouring steps overlapping the computation; every step still moves
    # its input and its output across PCIe, and the 256 MiB eviction read stays inside (it is not subtracted)
    from bolt_b200.linear_stack import HostPipeline
    pipe = HostPipeline(stack)
    n_e2e = max(args.steps, 20)
    pipe.run([x_host] * 4, [out_host] * 4, step_fn=step_fn, before_step=evict)
    barrier()
    t0 = time.perf_counter()
    pipe.run([x_host] * n_e2e, [out_host] * n_e2e, step_fn=step_fn, before_step=evict)
    e2e_s = max((time.perf_counter() - t0) * args.steps / n_e2e, 1e-9)
    e2e_ok = bool(check_rows_against_numpy(stack, x_host.numpy(), parity_rows)) and bool(
        np.array_equal(out_host.numpy().reshape(M_TOKENS, -1)[parity_rows], stack.out_dev.cpu().numpy().reshape(M_TOKENS, -1)[parity_rows]))
    clocks = sampler.stop() if rank == 0 else None
    # the same step replayed back to back for about two seconds: what the stack sustains under the power limit
    sustained = None
    if rank == 0 and world == 1 and g_step is not None and not args.no_sustained:
        s2 = ClockSampler(local_rank)
        s2.start()
        reps, t_s = 0, 0.0
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        wall = time.perf_counter()
        while time.perf_counter() - wall < 2.0:
            a.record(stream)
            for _ in range(200):
                g_step.replay()
            b.record(stream)
            b.synchronize()
            t_s += a.elapsed_time(b) / 1e3
            reps += 200
        c2 = s2.stop()
        peaks_s, _ = measured_peaks()
        tops_s = OPS_PER_STEP * reps / t_s / 1e12
        sustained = {"seconds": t_s, "steps": reps, "tops": tops_s, "ms_per_step": t_s / reps * 1e3,
                     "frac_of_2x_bf16_sustained": tops_s / (2.0 * peaks_s.get("bf16_tflops_sustained", peaks_s["bf16_tflops"])),
                     "clocks": c2, "note": "no L2 eviction between steps (weights stay in L2), graph replays back to back"}
    # the int8 ceiling of this GPU, measured now: tcgen05.mma.kind::i8 issued back to back from resident operands
    probe_tops = None
    if rank == 0:
        ms_p, tops_p = C.c_float(), C.c_float()
        if lib.bolt_b200_i8_mma_rate(20000, C.byref(ms_p), C.byref(tops_p)) == 0 and tops_p.value > 0:
            probe_tops = float(tops_p.value)
    status = lib.bolt_b200_device_status()

    vals = torch.tensor([dev_s, gemm_s, e2e_s, e2e_serial_s], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    dev_s, gemm_s, e2e_s, e2e_serial_s = [float(v) for v in vals.cpu()]
    if dist is not None:
        dist.barrier()
    sharded = None
    if dist is not None and not args.no_sharded:
        sharded = run_sharded_record(rank, world, lib, dist, stream, evict)
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    peaks, peak_src = measured_peaks()
    total_ops = OPS_PER_STEP * args.steps * world
    value = total_ops / dev_s / 1e12
    n_gemm = 2 * LAYERS
    gemm_tops = OPS_PER_STEP / (gemm_s / args.steps) / 1e12
    proxy_i8 = 2.0 * peaks["bf16_tflops"]
    peak_i8 = probe_tops if probe_tops else proxy_i8
    base, _ = cpu_stack_baseline(seconds=12.0) if (world == 1 and not args.no_cpu_baseline) else (None, None)
    line = {
        "metric": "int8_gemm_tops", "value": value, "unit": "TOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_s / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8*s8->s32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_tokens": M_TOKENS * world, "parallelism": "dp%d" % world,
                   "l2": "flushed between timed steps (256 MiB read)", "launch": launch_mode,
                   "device_status": status, "wall_s_timed_region": wall_s},
        "e2e": {"value": total_ops / e2e_s / 1e12, "unit": "TOP/s",
                "h2d_bytes_per_step": M_TOKENS * HIDDEN * 4, "d2h_bytes_per_step": M_TOKENS * HIDDEN * 4,
                "ms_per_step": e2e_s / args.steps * 1e3,
                "mode": "HostPipeline: H2D of step i+1 and D2H of step i-1 overlap step i; the eviction read is inside",
                "output_checked": e2e_ok,
                "serial_ms_per_step": e2e_serial_s / args.steps * 1e3,
                "serial_value": total_ops / e2e_serial_s / 1e12},
        "gpu_launches": int(launches),
        "parity_checked": parity_ok,
        "parity_note": "%d of %d token rows of the step's fp32 output compared bit for bit with a numpy "
                       "restatement of the whole 24-layer chain before timing" % (len(parity_rows), M_TOKENS),
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": gemm_tops, "peak": peak_i8, "unit": "TFLOP/s",
                     "frac": gemm_tops / peak_i8,
                     "traffic": GEMM_DRAM_TRAFFIC_PER_LAUNCH,
                     "kernel": "gemm_u8s8_tcgen05_kernel",
                     "launches_per_step": n_gemm,
                     "us_per_launch": gemm_s / args.steps / n_gemm * 1e6,
                     "ops_per_launch": OPS_PER_STEP / n_gemm,
                     "peak_source": ("tcgen05 kind::i8 issue-rate probe run in this process (1.4 ms burst, no loads, no epilogue)"
                                     if probe_tops else "2 x bf16_tflops of " + peak_src),
                     "peak_2x_bf16": proxy_i8, "frac_of_2x_bf16": gemm_tops / proxy_i8,
                     "note": "int8 multiply-add ops (2*M*N*K) in the TFLOP/s slot; MEASURED_PEAKS.json has no int8 entry: "
                             "peak is the issue rate measured on this GPU, beside it 2 x bf16_tflops of " + peak_src
                             + "; nominal dense int8 is 4500"},
    }
    if sustained is not None:
        line["sustained"] = sustained
    if sharded is not None:
        line["sharded"] = sharded
    if base is not None:
        line["cpu_baseline"] = base
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def run_side_workload(args):
    """The kernels next to the headline (bolt_b200/workloads.py), one JSON line."""
    import torch

    import bolt_b200 as B
    from bolt_b200 import workloads

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; there is no CPU fallback")
    B.load(build_if_missing=False)
    peaks, src = measured_peaks()
    sampler = ClockSampler(0)
    sampler.start()
    res = workloads.WORKLOADS[args.workload](peaks)
    res["clocks"] = sampler.stop()   # sampled every 50 ms over the whole workload, warm-up included
    mhz = res["clocks"].get("sm_mhz")
    if mhz:
        # time x clock, so that runs taken at different clocks can be compared: millions of SM cycles
        for row in res.get("rows", []):
            if "ms" in row:
                row["mcycles_at_median_clock"] = row["ms"] * mhz * 1e-3
    res["peaks"] = {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"],
                    "bf16_tflops_sustained": peaks.get("bf16_tflops_sustained"), "source": src}
    res["device_status"] = B.lib().bolt_b200_device_status()
    print(json.dumps(res))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the timed CPU leg (profiling runs)")
    ap.add_argument("--no-sustained", action="store_true", help="skip the two-second back-to-back replay")
    ap.add_argument("--no-sharded", action="store_true", help="with --gpus > 1: skip the N-split FFN record")
    ap.add_argument("--workload", default="bert_stack",
                    help="bert_stack (the headline, default) or one of the side workloads: ffn, gemv, quantize, "
                         "resnet_conv, resnet_conv_u8, bnn, pooling, i8_peak (1 GPU, prints that workload's figures as one "
                         "JSON line with the clocks sampled while it ran)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload != "bert_stack":
        if rank == 0:
            run_side_workload(args)
        return
    if args.impl == "reference":
        run_reference_arm(args, rank)
    else:
        run_b200_arm(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
