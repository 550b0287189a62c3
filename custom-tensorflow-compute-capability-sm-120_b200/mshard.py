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

Failure handling is host-side only.  A rank that stops taking part announces it
in the process group's store (``leave``); the others look there before they
launch anything that waits for it (``departed``) and raise ``PeerLeft``.  With a
deadline (``deadline_s``) every collective of ``gathered`` / ``gathered_fused`` is
waited for on the host with that limit; when it runs out the process group is
aborted (NCCL) and ``CollectiveTimeout`` is raised, so a rank that silently
stopped costs its peers one deadline instead of a hang.

The reference has no multi-GPU code (its only trace is
tf.distribute.MirroredStrategy in docs/api-reference.md:510-511); this module
is what the M-sharded FP8 workload (M = 65536, N = K = 8192) runs on.
"""
from __future__ import annotations

import datetime
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

TILE_M = 128


class PeerLeft(RuntimeError):
    """Another rank announced that it has stopped taking part; nothing was launched."""


class CollectiveTimeout(RuntimeError):
    """A collective did not finish within the deadline; the process group was aborted."""


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
                 matmul_fn: Optional[Callable] = None, align: int = TILE_M, deadline_s: Optional[float] = None):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group
        self.deadline_s = deadline_s
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

    # -- failure handling (host side) -------------------------------------------
    _LEFT_KEY = "sm120_mshard/left/{}"

    @staticmethod
    def _store():
        return dist.distributed_c10d._get_default_store()

    def leave(self) -> None:
        """Announce that this rank stops taking part.  Call it between two steps, with none
        of this rank's kernels or collectives in flight; the rank may then exit."""
        self._store().set(self._LEFT_KEY.format(self.rank), "1")

    def departed(self) -> List[int]:
        """Ranks that have announced their departure (a non-blocking look into the store)."""
        store = self._store()
        return [r for r in range(self.world_size) if r != self.rank and store.check([self._LEFT_KEY.format(r)])]

    def _require_peers(self) -> None:
        gone = self.departed()
        if gone:
            raise PeerLeft(f"rank(s) {gone} left the M-sharded product; rank {self.rank} launched nothing")

    def _await(self, work, what: str) -> None:
        """Wait for an asynchronous collective: stream-ordered without a deadline, on the host with one."""
        if work is None:
            return
        if self.deadline_s is None:
            work.wait()
            return
        try:
            done = work.wait(datetime.timedelta(seconds=self.deadline_s))
        except Exception as e:                      # both backends raise when the time is up
            self._abort()
            raise CollectiveTimeout(f"{what} did not finish within {self.deadline_s} s on rank {self.rank}: {e}") from e
        if done is False:
            self._abort()
            raise CollectiveTimeout(f"{what} did not finish within {self.deadline_s} s on rank {self.rank}")

    def _abort(self) -> None:
        """Tear the communicator down without waiting for the peers (NCCL); a no-op where the backend has no abort."""
        try:
            if dist.get_backend(self.group) == "nccl" and hasattr(dist.distributed_c10d, "_abort_process_group"):
                dist.distributed_c10d._abort_process_group(self.group)
        except Exception:
            pass

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
        self._require_peers()
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
            work = dist.all_gather_into_tensor(full, chunk.contiguous() if not chunk.is_contiguous() else chunk,
                                               group=self.group, async_op=True)
        else:
            work = dist.all_gather(views, chunk, group=self.group, async_op=True)
        self._await(work, "all-gather of the C slabs")


class PeerBuffers:
    """Every rank's gathered-C buffers [G*Ms, N], reachable from this process.

    Each rank allocates TWO buffers with torch and publishes the CUDA IPC handle of
    the allocation that holds each (plus the buffer's offset inside it); every other
    rank opens the handles with ITS OWN device current, which maps the memory for
    kernels of that device and sets up peer access.  `addr[k][r]` is then the address
    of rank r's buffer k in this process.  Set up once, outside timed regions; the
    buffers must stay alive as long as any rank uses them.

    Why two: call i of ``gathered_fused`` writes buffer i % 2.  A rank's call i + 1 may
    start while a peer is still reading the result of call i (the ranks are ordered
    only AFTER each product), so it must not write the same memory; buffer i % 2 is
    written again by call i + 2, which no rank starts before every rank has passed
    the closing all-reduce of call i + 1 in stream order.  The view that call i returns
    is therefore valid for work that this rank enqueues before its call i + 1."""

    def __init__(self, sharded: "MShardedMatmul", out_dtype: torch.dtype, device: torch.device):
        import ctypes
        from . import _binding
        G, ms = sharded.world_size, sharded.rows_per_rank
        self.rank = sharded.rank
        self.device = device
        self.group = sharded.group
        self.fulls = [torch.zeros((G * ms, sharded.N), dtype=out_dtype, device=device) for _ in range(2)]
        self.row_bytes = sharded.N * self.fulls[0].element_size()
        self.calls = 0
        lib = _binding.load_library()
        mine = []
        for full in self.fulls:
            handle = ctypes.create_string_buffer(64)
            offset = ctypes.c_uint64(0)
            with torch.cuda.device(device):
                rc = lib.sm120_ipc_export(full.data_ptr(), handle, ctypes.byref(offset))
            if rc != 0:
                raise RuntimeError(f"cannot export the C buffer through CUDA IPC: {_binding.error_string(rc)}")
            mine.append((bytes(handle.raw), int(offset.value)))
        published: List[object] = [None] * G
        dist.all_gather_object(published, mine, group=sharded.group)
        self.addr: List[List[int]] = [[], []]
        self._opened: List[int] = []
        opened_by_handle = {}
        with torch.cuda.device(device):
            for r in range(G):
                for k in range(2):
                    if r == self.rank:
                        self.addr[k].append(self.fulls[k].data_ptr())
                        continue
                    raw, off = published[r][k]
                    base = opened_by_handle.get((r, raw))           # both buffers may sit in one allocation
                    if base is None:
                        ptr = ctypes.c_void_p(0)
                        rc = lib.sm120_ipc_import(ctypes.create_string_buffer(raw, 64), ctypes.byref(ptr))
                        if rc != 0 or not ptr.value:
                            raise RuntimeError(f"cannot open rank {r}'s C buffer: {_binding.error_string(rc)}")
                        base = ptr.value
                        opened_by_handle[(r, raw)] = base
                        self._opened.append(base)
                    self.addr[k].append(base + off)
        dist.barrier(group=sharded.group)                             # nobody proceeds before every handle is open

    @property
    def full(self) -> torch.Tensor:
        """The buffer that the most recent call wrote (the first one before any call)."""
        return self.fulls[(self.calls - 1) % 2 if self.calls else 0]

    def close(self, collective: bool = True) -> None:
        """Unmap the peers' buffers.  Normally collective: every rank calls it with no kernel in
        flight, and the barriers keep any rank from freeing memory a peer may still write.  On an
        error path (a peer left or timed out) pass collective=False: only this rank's device is
        synchronised, so its own kernels no longer touch the peers' memory, and nothing waits for
        a rank that may be gone; keep this object (and its buffers) alive until the process ends."""
        from . import _binding
        torch.cuda.synchronize(self.device)
        if collective:
            dist.barrier(group=self.group)
        lib = _binding.load_library()
        with torch.cuda.device(self.device):
            for base in self._opened:
                lib.sm120_ipc_close(base)
        self._opened = []
        if collective:
            dist.barrier(group=self.group)

    def __enter__(self) -> "PeerBuffers":
        return self

    def __exit__(self, exc_type, exc, tb) -> None:
        self.close(collective=exc_type is None)


def _gathered_fused(self, a_slab: torch.Tensor, b: torch.Tensor, buffers: PeerBuffers, **kwargs) -> torch.Tensor:
    """The whole C [M, N] on every rank from ONE kernel per rank: the epilogue
    writes this rank's rows into every rank's buffer.  A one-element all-reduce
    afterwards orders the ranks (it moves no matrix data).  The result is a view of
    one of the two peer buffers: use it (enqueue the work that reads it) before this
    rank's next call, see PeerBuffers."""
    if a_slab.shape[0] != self.local_rows:
        raise ValueError(f"rank {self.rank} owns {self.local_rows} rows of A, got {a_slab.shape[0]}")
    self._require_peers()
    ms = self.rows_per_rank
    lo, hi = self.rank * ms, self.rank * ms + self.local_rows
    k = buffers.calls % 2
    buffers.calls += 1
    full = buffers.fulls[k]
    if self.local_rows > 0:
        peers = [buffers.addr[k][r] + lo * buffers.row_bytes for r in range(self.world_size) if r != self.rank]
        self.matmul_fn(a_slab, b, out=full[lo:hi], peer_outs=peers, **kwargs)
    token = torch.zeros(1, device=a_slab.device)
    # enqueued behind the GEMM: completes when every rank's GEMM (and its peer stores) has
    work = dist.all_reduce(token, group=self.group, async_op=True)
    self._await(work, "the closing all-reduce of the fused gather")
    return full[: self.M]


MShardedMatmul.gathered_fused = _gathered_fused
