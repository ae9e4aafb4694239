"""N-split GEMM / GEMV across the GPUs of one box: each rank owns a slice of the weight's output
columns, computes its `[M, N_local]` block with libbolt_b200.so, and an all-gather over NVLink
(NCCL through torch.distributed) assembles `[M, N]` on every rank.

The output columns of a GEMM are independent, so the only exchange on the path is the gather of the
results; activations (and their scale) are replicated.  The partition arithmetic and the gather
layout are plain host logic and run unchanged on CPU tensors with the gloo backend (that is how
they are tested without GPUs).
"""
import ctypes as C

import numpy as np


def shard_range(N, world, rank, align=32):
    """Columns [n0, n1) owned by `rank`: equal slices rounded up to `align` columns (whole 32-column
    chunks keep the tensor-core epilogue on its fast path); trailing ranks may get less, or nothing."""
    per = -(-N // world)
    per = -(-per // align) * align
    n0 = min(N, rank * per)
    n1 = min(N, n0 + per)
    return n0, n1


def shard_width(N, world, align=32):
    """Width of the widest shard = row pitch of one rank's slot in the gather buffer."""
    n0, n1 = shard_range(N, world, 0, align)
    return n1 - n0


def gather_columns(local, M, N, group=None, align=32):
    """local: this rank's `[M, width]` block (torch tensor, padded to the common shard width).
    Returns `[M, N]` assembled from all ranks' blocks.  One all_gather_into_tensor on a shard-major
    `[world][M][width]` buffer, then a strided copy into column order."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    width = shard_width(N, world, align)
    assert tuple(local.shape) == (M, width), (tuple(local.shape), (M, width))
    flat = torch.empty((world * M, width), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, local.contiguous(), group=group)  # rank r's block = rows [r*M, (r+1)*M)
    buf = flat.view(world, M, width)
    out = torch.empty((M, N), dtype=local.dtype, device=local.device)
    for r in range(world):
        n0, n1 = shard_range(N, world, r, align)
        if n1 > n0:
            out[:, n0:n1] = buf[r, :, : n1 - n0]
    return out


class ShardedLinear:
    """One quantized linear layer, N-split.  `Wq` s8 `[K, N]` and `w_scale` `[N]` are the full
    tensors; every rank keeps only its columns on the device."""

    def __init__(self, Wq, w_scale, rank, world, align=32):
        from .linear_stack import Linear

        self.K, self.N = Wq.shape
        self.rank, self.world, self.align = rank, world, align
        self.n0, self.n1 = shard_range(self.N, world, rank, align)
        self.width = shard_width(self.N, world, align)
        self.local = None
        if self.n1 > self.n0:
            self.local = Linear(np.ascontiguousarray(Wq[:, self.n0:self.n1]), np.asarray(w_scale)[self.n0:self.n1])

    def forward_local(self, a_dev, M, sA, out_dt, out_scale=1.0):
        """u8 activations `[M, K]` on the device -> this rank's `[M, width]` block (zero beyond its
        own columns).  Output type: DT_U8_Q (needs out_scale) or DT_F32."""
        import torch

        from . import CHECK_STATUS, DT_F32, GemmEpilogue, lib

        dt = torch.float32 if out_dt == DT_F32 else torch.uint8
        nloc = self.n1 - self.n0
        block = torch.zeros((M, self.width), dtype=dt, device="cuda")
        if self.local is None:
            return block
        tight = block if nloc == self.width else torch.empty((M, nloc), dtype=dt, device="cuda")
        ep = GemmEpilogue()
        ep.out_dt, ep.accumulate, ep.out_scale = out_dt, 0, float(out_scale)
        ep.sA, ep.sB = float(sA), float(self.local.w_scale_host[0])
        ep.d_sA, ep.row_scale = None, None
        ep.col_scale = None if self.local.uniform else C.c_void_p(self.local.w_scale.data_ptr())
        CHECK_STATUS(lib().bolt_b200_gemm_u8s8_ex(nloc, M, self.K, C.c_void_p(a_dev.data_ptr()),
                                                  C.c_void_p(self.local.packed.data_ptr()),
                                                  C.c_void_p(self.local.offsetC_ptr), C.c_void_p(tight.data_ptr()),
                                                  C.byref(ep)), "gemm")
        if tight is not block:
            block[:, :nloc] = tight
        return block

    def forward(self, a_dev, M, sA, out_dt, out_scale=1.0, group=None):
        return gather_columns(self.forward_local(a_dev, M, sA, out_dt, out_scale), M, self.N, group, self.align)


# ---------------------------------------------------------------------------------------------------
# Measurement of the N-split on the GPUs of one box (used by bench.py when it runs under torchrun).

class ShardedFFN:
    """The FFN-shaped product `[M, K] x [K, N]` (K 8192, N 28672 by default) with the weight's output
    columns split over the ranks: s8 weights with one scale per output channel, u8 activations with one
    scale per token, u8 (requantized) output.  Every rank generates the same activations and its own weight
    columns from seeds, so no data has to be distributed before the timed region.

    compute(M)            this rank's `[M, N / world]` block (GEMM on the tensor cores, GEMV kernel for M = 1)
    gather(M)             all_gather_into_tensor of the blocks into a shard-major `[world][M][N / world]` buffer
    overlapped(M, chunks) the rows are cut into chunks; chunk i is gathered on a side stream while chunk
                          i + 1 is computed
    """

    def __init__(self, rank, world, K=8192, N=28672, max_m=16384, seed=7, weight=None, like=None):
        """weight: s8 `[K, N / world]` on the device instead of the generated shard; like: another
        ShardedFFN whose activations and token scales are shared."""
        import torch

        from . import (DF_NORMAL, DT_I8, lib, matrix_matrix_multiply_transform_rhs, matrix_matrix_multiply_transform_rhs_bytes,
                       tensor2df)

        assert N % (32 * world) == 0
        self.rank, self.world, self.K, self.N = rank, world, K, N
        self.nloc = N // world
        self.max_m = max_m
        self.torch = torch
        self.lib = lib()
        self.w_gen_seed = seed
        w = self.shard_weight(rank) if weight is None else weight
        desc = tensor2df(DT_I8, DF_NORMAL, K, self.nloc)
        nbytes, self.rhs = matrix_matrix_multiply_transform_rhs_bytes(desc)
        self.packed = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        matrix_matrix_multiply_transform_rhs(desc, C.c_void_p(w.data_ptr()), C.c_void_p(self.packed.data_ptr()))
        torch.cuda.synchronize()
        del w
        if like is None:
            g = torch.Generator("cuda").manual_seed(seed + 1000)
            self.a = torch.randint(0, 256, (max_m, K), dtype=torch.uint8, device="cuda", generator=g)
            self.rs = (torch.rand(max_m, device="cuda", generator=g) * 20 + 30).float()
        else:
            self.a, self.rs = like.a, like.rs
        self.sB = self.channel_scales()[rank * self.nloc:(rank + 1) * self.nloc].contiguous()
        self.block = torch.empty(max_m * self.nloc, dtype=torch.uint8, device="cuda")
        self.full = torch.empty(world * max_m * self.nloc, dtype=torch.uint8, device="cuda")
        self.y32 = torch.zeros(self.nloc, dtype=torch.int32, device="cuda")
        self.side = torch.cuda.Stream()

    def shard_weight(self, r):
        """s8 `[K, N / world]`: the columns of rank r (every rank can regenerate any shard)"""
        torch = self.torch
        g = torch.Generator("cuda").manual_seed(self.w_gen_seed * 100 + r)
        return torch.randint(-127, 128, (self.K, self.nloc), dtype=torch.int8, device="cuda", generator=g)

    def channel_scales(self):
        torch = self.torch
        g = torch.Generator("cuda").manual_seed(self.w_gen_seed + 2000)
        return (torch.rand(self.N, device="cuda", generator=g) * 500 + 1500).float()

    def compute(self, M, row0=0, rows=None):
        """rows [row0, row0 + rows) of this rank's block"""
        from . import CHECK_STATUS, DF_NKN32K4, DT_I8, DT_U8_Q, GemmEpilogue

        rows = M if rows is None else rows
        L = self.lib
        out = C.c_void_p(self.block.data_ptr() + row0 * self.nloc)
        if M == 1:
            # M = 1 goes through the GEMV kernel (per-tensor scales: the reference's protocol), packed layout shared
            scale = (C.c_float * 2)(-1.0, 0.0005)
            CHECK_STATUS(L.mvm_cuda_b200(self.nloc, self.K, DT_I8, DF_NKN32K4, C.c_void_p(self.packed.data_ptr()),
                                         C.c_void_p(self.a.data_ptr()), out, C.c_void_p(self.packed.data_ptr() + self.rhs),
                                         C.cast(scale, C.POINTER(C.c_float))), "mvm")
            return
        ep = GemmEpilogue()
        ep.out_dt, ep.accumulate, ep.out_scale, ep.sA, ep.sB = DT_U8_Q, 0, 40.0, 1.0, 1.0
        ep.row_scale = C.c_void_p(self.rs.data_ptr() + 4 * row0)
        ep.col_scale = C.c_void_p(self.sB.data_ptr())
        CHECK_STATUS(L.bolt_b200_gemm_u8s8_ex(self.nloc, rows, self.K, C.c_void_p(self.a.data_ptr() + row0 * self.K),
                                              C.c_void_p(self.packed.data_ptr()), C.c_void_p(self.packed.data_ptr() + self.rhs),
                                              out, C.byref(ep)), "gemm")

    def gather(self, M, row0=0, rows=None):
        import torch.distributed as dist

        rows = M if rows is None else rows
        src = self.block[row0 * self.nloc:(row0 + rows) * self.nloc]
        if row0 == 0 and rows == M:
            dst = self.full[: self.world * M * self.nloc]
        else:
            # chunked: every chunk gets its own shard-major slot [world][rows][nloc]
            dst = self.full[self.world * row0 * self.nloc: self.world * (row0 + rows) * self.nloc]
        dist.all_gather_into_tensor(dst, src)

    def overlapped(self, M, chunks=4):
        torch = self.torch
        main = torch.cuda.current_stream()
        per = -(-M // chunks)
        per = max(128, -(-per // 128) * 128)
        evs = []
        r0 = 0
        while r0 < M:
            rows = min(per, M - r0)
            self.compute(M, r0, rows)
            ev = torch.cuda.Event()
            ev.record(main)
            self.side.wait_event(ev)
            with torch.cuda.stream(self.side):
                self.gather(M, r0, rows)
            r0 += rows
        done = torch.cuda.Event()
        done.record(self.side)
        main.wait_event(done)

    def assembled(self, M):
        """`[M, N]` from the shard-major gather buffer (after gather(M))"""
        return self.full[: self.world * M * self.nloc].view(self.world, M, self.nloc).permute(1, 0, 2).reshape(M, self.N)

    # ---- the all-gather fused into the GEMM: every rank stores its tiles into all ranks' [M, N] results -------
    def setup_fused(self):
        """Allocates this rank's `[max_m, N]` result with the library's allocator, exchanges its handle with the other
        ranks (one process per GPU) and maps theirs.  Needs an initialised process group."""
        import torch.distributed as dist

        from . import CHECK_STATUS

        L = self.lib
        L.bolt_b200_malloc.restype = C.c_void_p
        # local, fallible part first; the exchange below is reached by every rank whatever happened here
        mine = None
        self.result_ptr = L.bolt_b200_malloc(C.c_size_t(self.max_m * self.N))
        if self.result_ptr:
            handle = (C.c_char * 64)()
            if L.bolt_b200_ipc_export(C.c_void_p(self.result_ptr), handle) == 0:
                mine = bytes(handle.raw)
        handles = [None] * self.world
        dist.all_gather_object(handles, mine)
        if any(h is None for h in handles):
            raise RuntimeError("a rank could not allocate or export its result buffer")
        self.dest = []
        self.imported = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.dest.append(self.result_ptr)
                continue
            p = C.c_void_p()
            CHECK_STATUS(L.bolt_b200_ipc_import(C.c_char_p(h), C.byref(p)), "ipc_import")
            self.dest.append(p.value)
            self.imported.append(p.value)
        self.flag = self.torch.zeros(1, dtype=self.torch.int32, device="cuda")

    def fused(self, M):
        """this rank's columns of `[M, N]` into every rank's result, then a one-element all-reduce as the barrier
        after which all columns of the local result are complete"""
        import torch.distributed as dist

        self.fused_compute(M)
        dist.all_reduce(self.flag)

    def fused_compute(self, M):
        """the scatter GEMM alone (no collective)"""
        from . import CHECK_STATUS, DT_U8_Q, GemmEpilogue, Scatter

        ep = GemmEpilogue()
        ep.out_dt, ep.accumulate, ep.out_scale, ep.sA, ep.sB = DT_U8_Q, 0, 40.0, 1.0, 1.0
        ep.row_scale = C.c_void_p(self.rs.data_ptr())
        ep.col_scale = C.c_void_p(self.sB.data_ptr())
        sc = Scatter()
        sc.n_dest, sc.ld, sc.col0 = self.world, self.N, self.rank * self.nloc
        for r in range(self.world):
            sc.dest[r] = self.dest[r]
        CHECK_STATUS(self.lib.bolt_b200_gemm_u8s8_scatter(self.nloc, M, self.K, C.c_void_p(self.a.data_ptr()),
                                                          C.c_void_p(self.packed.data_ptr()),
                                                          C.c_void_p(self.packed.data_ptr() + self.rhs), C.byref(ep), C.byref(sc)),
                     "gemm scatter")

    def fused_result(self, M):
        """torch view of the first M rows of this rank's fused result"""
        class _Raw:
            pass

        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (M, self.N), "typestr": "|u1", "data": (int(self.result_ptr), False), "version": 2}
        return self.torch.as_tensor(raw, device="cuda")

    def close_fused(self):
        for p in getattr(self, "imported", []):
            self.lib.bolt_b200_ipc_close(C.c_void_p(p))
        self.imported = []
        if getattr(self, "result_ptr", None):
            self.lib.bolt_b200_free(C.c_void_p(self.result_ptr))
            self.result_ptr = None
