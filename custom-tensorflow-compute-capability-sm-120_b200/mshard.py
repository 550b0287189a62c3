"""M-sharding of one GEMM across the GPUs of a box: one process per GPU.

C = A @ B is split by rows: rank r of G owns the contiguous slab
A[r*Ms:(r+1)*Ms, :] (Ms = ceil(M / G), rounded up to the 128-row tile) and
computes the same rows of C with B replicated on every GPU.  The slabs are
independent, so the product itself needs no communication.  Only when the
caller asks for the gathered C is anything exchanged, in one of two ways:

* ``gathered``: an all-gather of the [Ms, N] slabs over NCCL (NVLink /
  NVSwitch), issued per row-chunk on a side stream so that the all-gather of
  chunk c overlaps the GEMM of chunk c+1;
* ``gathered_fused``: the GEMM kernel's own epilogue stores every output block
  into every rank's copy of C (peer memory mapped through CUDA IPC, TMA stores
  over NVLink), so the all-gather happens while the tiles are computed and the
  only collective left is a one-element barrier.

The reference has no multi-GPU code (its only trace is
tf.distribute.MirroredStrategy in docs/api-reference.md:510-511); this module
is the part of the B200 build that BASELINE config 5 (FP8, M = 65536) runs on.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

TILE_M = 128


def slab_rows(M: int, world_size: int, align: int = TILE_M) -> int:
    """Rows per rank: ceil(M / world_size) rounded up to `align`."""
    if M < 0 or world_size < 1:
        raise ValueError("M must be >= 0 and world_size >= 1")
    per = -(-M // world_size)
    return -(-per // align) * align if per > 0 else 0


def slab_bounds(M: int, world_size: int, rank: int, align: int = TILE_M) -> Tuple[int, int]:
    """[start, stop) of the rows of A and C that `rank` owns; empty for ranks
    past the end of a short matrix."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside [0, {world_size})")
    ms = slab_rows(M, world_size, align)
    start = min(M, rank * ms)
    return start, min(M, start + ms)


def chunk_bounds(rows: int, chunks: int, align: int = TILE_M) -> List[Tuple[int, int]]:
    """Split [0, rows) into at most `chunks` contiguous pieces whose sizes are
    multiples of `align` (except the last)."""
    if rows <= 0:
        return []
    chunks = max(1, int(chunks))
    per = -(-rows // chunks)
    per = -(-per // align) * align
    out = []
    s = 0
    while s < rows:
        out.append((s, min(rows, s + per)))
        s += per
    return out


class MShardedMatmul:
    """Runs the M-sharded product on this rank.

    matmul_fn(a_rows, b, out=..., **kwargs) computes one slab (or one chunk of
    it) into `out`; by default it is ``sm120_ops.fused_matmul``.  It is a
    parameter so that the partition and gather logic can be exercised with CPU
    ranks (gloo), where no GPU kernel can run.
    """

    def __init__(self, M: int, N: int, group: Optional[dist.ProcessGroup] = None,
                 matmul_fn: Optional[Callable] = None, align: int = TILE_M):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group
        self.world_size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.M, self.N = int(M), int(N)
        self.align = align
        self.rows_per_rank = slab_rows(self.M, self.world_size, align)
        self.start, self.stop = slab_bounds(self.M, self.world_size, self.rank, align)
        if matmul_fn is None:
            from . import sm120_ops
            matmul_fn = sm120_ops.fused_matmul
        self.matmul_fn = matmul_fn
        self._comm_stream = None

    @property
    def local_rows(self) -> int:
        return self.stop - self.start

    def replicate_b(self, b: torch.Tensor, src: int = 0) -> torch.Tensor:
        """Broadcast B (and anything else every rank needs, e.g. scales) from
        `src`; done once at set-up, outside any timed region."""
        dist.broadcast(b, src=src, group=self.group)
        return b

    def local(self, a_slab: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, **kwargs) -> torch.Tensor:
        """This rank's rows of C; no communication."""
        if a_slab.shape[0] != self.local_rows:
            raise ValueError(f"rank {self.rank} owns {self.local_rows} rows of A, got {a_slab.shape[0]}")
        return self.matmul_fn(a_slab, b, out=out, **kwargs)

    def gathered(self, a_slab: torch.Tensor, b: torch.Tensor, out_dtype: torch.dtype, chunks: int = 1,
                 **kwargs) -> torch.Tensor:
        """The whole C [M, N] on every rank.  Row-chunk c of every slab is
        all-gathered while chunk c+1 is being multiplied."""
        if a_slab.shape[0] != self.local_rows:
            raise ValueError(f"rank {self.rank} owns {self.local_rows} rows of A, got {a_slab.shape[0]}")
        G, ms = self.world_size, self.rows_per_rank
        dev = a_slab.device
        # padded result: slab r at rows [r*ms, (r+1)*ms); trimmed to M at the end
        full = torch.empty((G * ms, self.N), dtype=out_dtype, device=dev)
        mine = full[self.rank * ms:(self.rank + 1) * ms]
        if self.local_rows < ms:
            mine[self.local_rows:].zero_()
        on_gpu = dev.type == "cuda"
        if on_gpu and self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=dev)
        pieces = chunk_bounds(ms, chunks, self.align)
        for (s, e) in pieces:
            rows_here = max(0, min(e, self.local_rows) - s)
            if rows_here > 0:
                self.matmul_fn(a_slab[s:s + rows_here], b, out=mine[s:s + rows_here], **kwargs)
            views = [full[r * ms + s: r * ms + e] for r in range(G)]
            if on_gpu:
                ready = torch.cuda.Event()
                ready.record(torch.cuda.current_stream(dev))
                with torch.cuda.stream(self._comm_stream):
                    self._comm_stream.wait_event(ready)
                    self._all_gather(views, mine[s:e], single=(len(pieces) == 1), full=full)
            else:
                self._all_gather(views, mine[s:e], single=(len(pieces) == 1), full=full)
        if on_gpu:
            torch.cuda.current_stream(dev).wait_stream(self._comm_stream)
        return full[: self.M]

    def _all_gather(self, views, chunk, single: bool, full: torch.Tensor) -> None:
        if single:
            # slabs are contiguous in rank order: one all-gather straight into place
            dist.all_gather_into_tensor(full, chunk.contiguous() if not chunk.is_contiguous() else chunk, group=self.group)
        else:
            dist.all_gather(views, chunk, group=self.group)


class PeerBuffers:
    """Every rank's gathered-C buffer [G*Ms, N], reachable from this process.

    Each rank allocates its buffer with torch and publishes the CUDA IPC handle of
    the allocation that holds it (plus the buffer's offset inside it); every other
    rank opens that handle with ITS OWN device current, which maps the memory for
    kernels of that device and sets up peer access.  `addr[r]` is then the address
    of rank r's buffer in this process.  Set up once, outside timed regions; the
    buffer must stay alive as long as any rank uses it."""

    def __init__(self, sharded: "MShardedMatmul", out_dtype: torch.dtype, device: torch.device):
        import ctypes
        from . import _binding
        G, ms = sharded.world_size, sharded.rows_per_rank
        self.rank = sharded.rank
        self.device = device
        self.full = torch.zeros((G * ms, sharded.N), dtype=out_dtype, device=device)
        self.row_bytes = sharded.N * self.full.element_size()
        lib = _binding.load_library()
        handle = ctypes.create_string_buffer(64)
        offset = ctypes.c_uint64(0)
        with torch.cuda.device(device):
            rc = lib.sm120_ipc_export(self.full.data_ptr(), handle, ctypes.byref(offset))
        if rc != 0:
            raise RuntimeError(f"cannot export the C buffer through CUDA IPC: {_binding.error_string(rc)}")
        published: List[object] = [None] * G
        dist.all_gather_object(published, (bytes(handle.raw), int(offset.value)), group=sharded.group)
        self.addr: List[int] = []
        self._opened: List[int] = []
        with torch.cuda.device(device):
            for r in range(G):
                if r == self.rank:
                    self.addr.append(self.full.data_ptr())
                    continue
                raw, off = published[r]
                base = ctypes.c_void_p(0)
                rc = lib.sm120_ipc_import(ctypes.create_string_buffer(raw, 64), ctypes.byref(base))
                if rc != 0 or not base.value:
                    raise RuntimeError(f"cannot open rank {r}'s C buffer: {_binding.error_string(rc)}")
                self._opened.append(base.value)
                self.addr.append(base.value + off)
        dist.barrier(group=sharded.group)                             # nobody proceeds before every handle is open

    def close(self) -> None:
        """Unmap the peers' buffers (collective: every rank calls it, with no kernel in flight)."""
        from . import _binding
        torch.cuda.synchronize(self.device)
        dist.barrier()
        lib = _binding.load_library()
        with torch.cuda.device(self.device):
            for base in self._opened:
                lib.sm120_ipc_close(base)
        self._opened = []
        dist.barrier()


def _gathered_fused(self, a_slab: torch.Tensor, b: torch.Tensor, buffers: PeerBuffers, **kwargs) -> torch.Tensor:
    """The whole C [M, N] on every rank from ONE kernel per rank: the epilogue
    writes this rank's rows into every rank's buffer.  A one-element all-reduce
    afterwards orders the ranks (it moves no matrix data)."""
    if a_slab.shape[0] != self.local_rows:
        raise ValueError(f"rank {self.rank} owns {self.local_rows} rows of A, got {a_slab.shape[0]}")
    ms = self.rows_per_rank
    lo, hi = self.rank * ms, self.rank * ms + self.local_rows
    if self.local_rows > 0:
        peers = [buffers.addr[r] + lo * buffers.row_bytes for r in range(self.world_size) if r != self.rank]
        self.matmul_fn(a_slab, b, out=buffers.full[lo:hi], peer_outs=peers, **kwargs)
    token = torch.zeros(1, device=a_slab.device)
    dist.all_reduce(token, group=self.group)        # enqueued behind the GEMM: completes when every rank's GEMM has
    return buffers.full[: self.M]


MShardedMatmul.gathered_fused = _gathered_fused
