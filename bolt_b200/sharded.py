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
