"""CPU tests of the M-sharding logic: slab arithmetic, and the local / gathered
product with two gloo ranks, where the per-slab product is supplied by the test
(the oracle) because no GPU kernel can run here."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.conftest import PACKAGE_NAME


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_slab_arithmetic(pkg):
    ms = pkg.mshard
    assert ms.slab_rows(65536, 8) == 8192 and ms.slab_bounds(65536, 8, 7) == (57344, 65536)
    assert ms.slab_rows(1000, 4) == 256            # ceil(1000/4) = 250 -> next multiple of 128
    bounds = [ms.slab_bounds(1000, 4, r) for r in range(4)]
    assert bounds == [(0, 256), (256, 512), (512, 768), (768, 1000)]
    assert [ms.slab_bounds(130, 4, r) for r in range(4)] == [(0, 128), (128, 130), (130, 130), (130, 130)]
    assert ms.slab_rows(0, 4) == 0 and ms.slab_bounds(0, 4, 2) == (0, 0)
    # slabs tile [0, M) exactly, for a sweep of sizes
    for M in (1, 127, 128, 129, 4096, 65536, 100003):
        for G in (1, 2, 4, 8):
            cover = [ms.slab_bounds(M, G, r) for r in range(G)]
            assert cover[0][0] == 0 and cover[-1][1] == M
            assert all(cover[i][1] == cover[i + 1][0] for i in range(G - 1))
    assert ms.chunk_bounds(8192, 4) == [(0, 2048), (2048, 4096), (4096, 6144), (6144, 8192)]
    assert ms.chunk_bounds(300, 2) == [(0, 256), (256, 300)]
    assert ms.chunk_bounds(0, 3) == []
    with pytest.raises(ValueError):
        ms.slab_bounds(10, 2, 2)


def _cpu_matmul(a, b, out=None, **kwargs):
    """Stand-in for the GPU op inside the gloo test: float64 product, fp32 result."""
    r = (a.double() @ b.double()).float()
    if kwargs.get("bias") is not None:
        r = r + kwargs["bias"]
    if out is not None:
        out.copy_(r)
        return out
    return r


def _worker(rank, world, port, M, N, K, chunks, ret):
    import importlib
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ms = importlib.import_module(PACKAGE_NAME).mshard
        g = torch.Generator().manual_seed(0)
        a = torch.randn(M, K, generator=g)
        b_src = torch.randn(K, N, generator=g)
        sh = ms.MShardedMatmul(M, N, matmul_fn=_cpu_matmul)
        b = b_src.clone() if rank == 0 else torch.zeros(K, N)
        sh.replicate_b(b)
        a_slab = a[sh.start:sh.stop]
        local = sh.local(a_slab, b)
        full = sh.gathered(a_slab, b, out_dtype=torch.float32, chunks=chunks)
        want = (a.double() @ b_src.double()).float()
        ok = (torch.equal(b, b_src) and torch.equal(local, want[sh.start:sh.stop]) and tuple(full.shape) == (M, N)
              and torch.equal(full, want))
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("M,N,K,chunks", [(512, 96, 64, 1), (512, 96, 64, 2), (300, 40, 32, 1), (300, 40, 32, 3), (100, 16, 8, 1)])
def test_two_gloo_ranks_local_and_gathered(M, N, K, chunks):
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, M, N, K, chunks, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert dict(ret) == {0: True, 1: True}


# ----- failure handling, on the host only: a rank that leaves, and a rank that silently stops -----
def _leaving_worker(rank, world, port, announce, ret):
    import importlib
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ms = importlib.import_module(PACKAGE_NAME).mshard
    M, N, K = 256, 32, 16
    g = torch.Generator().manual_seed(0)
    a, b = torch.randn(M, K, generator=g), torch.randn(K, N, generator=g)
    sh = ms.MShardedMatmul(M, N, matmul_fn=_cpu_matmul, deadline_s=2.0)
    slab = a[sh.start:sh.stop]
    full = sh.gathered(slab, b, out_dtype=torch.float32)                 # step 1: everybody takes part
    ok1 = torch.equal(full, (a.double() @ b.double()).float())
    if rank == 1:
        # step 2 never happens on this rank: with an announcement, or silently
        if announce:
            sh.leave()
        time.sleep(6.0)                                                   # stay alive past rank 0's deadline, then go
        ret[rank] = ("left", ok1)
        os._exit(0)
    t0 = time.perf_counter()
    outcome = "finished"
    try:
        if announce:
            while not sh.departed() and time.perf_counter() - t0 < 5.0:  # the announcement is a store write away
                time.sleep(0.01)
        sh.gathered(slab, b, out_dtype=torch.float32)                    # step 2
    except ms.PeerLeft:
        outcome = "peer_left"
    except ms.CollectiveTimeout:
        outcome = "timeout"
    ret[rank] = (outcome, ok1, time.perf_counter() - t0)
    os._exit(0)                                                           # the group is broken on purpose: skip its teardown


@pytest.mark.parametrize("announce", [True, False])
def test_a_rank_that_leaves_between_steps_is_reported_within_the_deadline(announce):
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_leaving_worker, args=(r, world, port, announce, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    outcome, ok1, elapsed = ret[0]
    assert ok1 and ret[1] == ("left", True)
    if announce:
        assert outcome == "peer_left" and elapsed < 2.0          # seen in the store before anything was launched
    else:
        assert outcome == "timeout" and 1.5 < elapsed < 5.5       # the 2 s deadline, not a hang
