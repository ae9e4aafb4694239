"""Host logic of the N-split GEMM (bolt_b200/sharded.py) on CPU: the partition arithmetic, and the
all-gather + column assembly with two gloo ranks, each holding the exact integer product of its own
weight columns (the part the GPUs would compute)."""
import os
import socket
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from bolt_b200.sharded import shard_range, shard_width  # noqa: E402

WORKER = r"""
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from bolt_b200 import synth
from bolt_b200.sharded import gather_columns, shard_range, shard_width
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
ok = True
for (M, K, N) in [(5, 16, 70), (16, 64, 28672 // 64), (3, 8, 31), (4, 8, 64)]:
    A = synth.u8(1, (M, K)).astype(np.int64)
    W = synth.s8(2, (K, N)).astype(np.int64)
    full = (A @ W).astype(np.int32)
    n0, n1 = shard_range(N, world, rank)
    width = shard_width(N, world)
    local = np.zeros((M, width), np.int32)
    local[:, : n1 - n0] = (A @ W[:, n0:n1]).astype(np.int32)
    out = gather_columns(torch.from_numpy(local), M, N)
    ok = ok and np.array_equal(out.numpy(), full)
flag = torch.tensor([1 if ok else 0])
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
dist.destroy_process_group()
sys.exit(0 if flag.item() == 1 else 1)
"""


def test_shard_ranges_cover_and_align():
    for N in (1, 31, 32, 33, 768, 3072, 28672, 1000):
        for world in (1, 2, 3, 4, 8):
            cols, prev = 0, 0
            for r in range(world):
                n0, n1 = shard_range(N, world, r)
                assert n0 == prev and n0 <= n1 <= N
                assert n0 % 32 == 0 or n0 == N
                assert n1 - n0 <= shard_width(N, world)
                cols += n1 - n0
                prev = n1
            assert cols == N and prev == N
    assert shard_range(28672, 8, 3) == (3 * 3584, 4 * 3584)


def test_gather_columns_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script), ROOT], env=env))
    codes = [p.wait(timeout=180) for p in procs]
    assert codes == [0, 0]


def test_scatter_offsets_agree_with_the_shard_ranges():
    """The fused N-split stores rank r's columns at r * (N / world) of every rank's [M, N] result; that has to be the
    same partition the gather-based path uses (shard_range), for the widths both paths accept."""
    from bolt_b200.sharded import shard_range, shard_width

    for N in (28672, 3072, 8192):
        for world in (1, 2, 4, 8):
            if N % (32 * world):
                continue
            nloc = N // world
            assert shard_width(N, world) == nloc
            covered = 0
            for r in range(world):
                n0, n1 = shard_range(N, world, r)
                assert (n0, n1) == (r * nloc, (r + 1) * nloc)
                assert n0 % 32 == 0            # the scatter epilogue's column offset rule
                covered += n1 - n0
            assert covered == N
