"""M-sharding of one GEMM across the GPUs of a box: one process per GPU.

C = A @ B is split by rows: rank r of G owns the contiguous slab
A[r*Ms:(r+1)*Ms, :] (Ms = ceil(M / G), rounded up to the 128-row tile) and
computes the same rows of C with B replicated on every GPU.  The slabs are
independent, so the product itself needs no communication.  Only when the
caller asks for the gathered C does a collective run: an all-gather of the
[Ms, N] slabs over NCCL (NVLink / NVSwitch), issued per row-chunk on a side
stream so that the all-gather of chunk c overlaps the GEMM of chunk c+1.

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
