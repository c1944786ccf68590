"""World-size-2 gloo tests of the sharding helpers (CPU ranks; the oracle stands in for the
device BLAS so that the row partition + all-gather can be checked end to end)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, m, n, k, trans_a, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from dlf_b200 import shard
    from dlf_b200.gblas import Transpose
    from support import OracleBlas
    g = torch.Generator().manual_seed(0)  # replicated inputs: same seed on every rank
    A = torch.rand((k, m) if trans_a else (m, k), generator=g) * 2 - 1
    B = torch.rand(k, n, generator=g) * 2 - 1
    C0 = torch.randn(m, n, generator=g)
    C = C0.clone()
    ta = Transpose.Trans if trans_a else Transpose.NoTrans
    shard.gemm_row_sharded(ta, Transpose.NoTrans, 0.5, A, B, 0.5, C, world, rank,
                           backend=OracleBlas())
    ref = 0.5 * ((A.t() if trans_a else A).double() @ B.double()) + 0.5 * C0.double()
    err = float((C.double() - ref).norm() / ref.norm())
    if m % (world * 4) == 0:
        # the panel-wise form (all-gather of a finished panel while the next is computed; on the
        # CPU the two simply alternate) must give the same C on every rank
        C2 = C0.clone()
        shard.gemm_row_sharded_overlapped(ta, Transpose.NoTrans, 0.5, A, B, 0.5, C2, world, rank, 4,
                                          backend=OracleBlas())
        err = max(err, float((C2.double() - ref).norm() / ref.norm()))
    # conv-style batch split: slabs are disjoint and cover the batch
    start, cnt = shard.split(11, world, rank)
    gathered = [None] * world
    dist.all_gather_object(gathered, (start, cnt))
    if rank == 0:
        out.put((err, gathered))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("m,trans_a", [(64, False), (64, True), (37, True)])
def test_row_sharded_gemm_all_gather_world2(m, trans_a):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, m, 24, 40, trans_a, q)) for r in range(2)]
    [p.start() for p in procs]
    err, gathered = q.get(timeout=120)
    [p.join(timeout=60) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    assert err < 1e-6
    assert gathered == [(0, 6), (6, 5)]


def test_split_covers_range():
    from dlf_b200 import shard
    for total in (0, 1, 7, 64, 1000):
        for world in (1, 2, 3, 8):
            slabs = [shard.split(total, world, r) for r in range(world)]
            assert slabs[0][0] == 0
            for (s0, c0), (s1, _) in zip(slabs, slabs[1:]):
                assert s0 + c0 == s1
            assert sum(c for _, c in slabs) == total
            assert max(c for _, c in slabs) - min(c for _, c in slabs) <= 1
