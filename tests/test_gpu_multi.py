"""Multi-GPU tests of the M-sharded product (needs >= 2 GPUs; skipped otherwise).
One process per GPU over NCCL.  Each rank multiplies its slab with the CUDA op;
the gathered result must equal, bit for bit, the single-GPU product of the whole
matrix (rows are independent and tiles are computed the same way on every GPU)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.conftest import PACKAGE_NAME

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import importlib
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        pkg = importlib.import_module(PACKAGE_NAME)
        ops, ms = pkg.sm120_ops, pkg.mshard
        results = {}
        for name, M, N, K, chunks in (("bf16", 2048, 1024, 512, 1), ("bf16_chunked", 2048, 1024, 512, 4),
                                      ("ragged", 1000, 264, 136, 2), ("fp8", 4096, 2048, 1024, 2)):
            g = torch.Generator(device="cuda").manual_seed(7)
            a32 = torch.randn(M, K, generator=g, device="cuda")
            b32 = torch.randn(N, K, generator=g, device="cuda")          # stored [N, K]
            kw = dict(transpose_b=True)
            if name == "fp8":
                a, sa = ops.quantize_fp8(a32)
                b, sb = ops.quantize_fp8(b32)
                kw.update(scale_a=sa, scale_b=sb)
            else:
                a, b = a32.bfloat16(), b32.bfloat16()
            sh = ms.MShardedMatmul(M, N)
            b_local = b.clone() if rank == 0 else torch.zeros_like(b)
            sh.replicate_b(b_local)                                      # B travels once, from rank 0
            whole = ops.fused_matmul(a, b, **kw)                         # single-GPU product of everything
            slab = a[sh.start:sh.stop]
            local = sh.local(slab, b_local, **kw)
            full = sh.gathered(slab, b_local, out_dtype=torch.bfloat16, chunks=chunks, **kw)
            bufs = ms.PeerBuffers(sh, torch.bfloat16, torch.device("cuda", rank))
            # three steps in a row with different A, none separated by a host synchronisation: each
            # result is copied out (stream-ordered) before the next call, which is the rule for the
            # two alternating peer buffers
            fused = []
            for step in range(3):
                a_step = a if step == 0 else (a.float() * 0.5 ** step).to(a.dtype)
                fused.append(sh.gathered_fused(a_step[sh.start:sh.stop], b_local, bufs, **kw).clone())
            torch.cuda.synchronize()
            ok = tuple(fused[0].shape) == (M, N) and torch.equal(fused[0], whole)
            for step in (1, 2):
                a_step = (a.float() * 0.5 ** step).to(a.dtype)
                ok = ok and torch.equal(fused[step], ops.fused_matmul(a_step, b, **kw))
            results[name + "_fused"] = bool(ok)
            bufs.close()
            del bufs
            results[name] = bool(torch.equal(b_local, b) and torch.equal(local, whole[sh.start:sh.stop])
                                 and tuple(full.shape) == (M, N) and torch.equal(full, whole))
        ret[rank] = results
    finally:
        dist.destroy_process_group()


def test_m_sharded_product_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    for r in range(world):
        assert all(ret[r].values()), (r, dict(ret[r]))
