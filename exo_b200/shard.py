"""Row-sharded GEMM over the GPUs of one node: one process per GPU.

``C[rows r] = A[rows r] @ B`` needs all of B but only its own rows of A and C
(apps/x86/sgemm/sgemm.py:20-23 has no dependence between rows), so a large GEMM
is split into contiguous row blocks of A and C, one per rank; B is broadcast
once from rank 0 (NCCL over NVLink when the tensors are CUDA tensors) and then
every rank runs the same single-GPU kernel on its block.  There is no
collective inside a step when the operands are resident in device memory.

When a step is given HOST buffers (the reference's calling convention) on more
than one rank, B would otherwise cross PCIe once per rank.  Instead every rank
uploads only its 1/world slice of B, the slices are all-gathered over NVLink
into each rank's own copy (NCCL on local buffers: no peer loads), and the rank's
rows of A and C stream through the library's host-pointer row pipeline while
that happens.  Host-to-device bytes per step then stay at |A| + |B| for the
whole job however many ranks take part.

Failure handling stays on the host: before the one collective, every rank
checks in through the process group's key-value store with a deadline.  A rank
that never arrives makes the others raise ``ShardError`` *before* any GPU work
or collective has been enqueued, so no rank is left waiting inside NCCL.
"""
from __future__ import annotations

import time
from dataclasses import dataclass


class ShardError(RuntimeError):
    pass


@dataclass(frozen=True)
class RowBlock:
    start: int
    stop: int

    @property
    def rows(self) -> int:
        return self.stop - self.start


def row_blocks(M: int, world: int, tile: int = 128) -> list[RowBlock]:
    """Contiguous row blocks, one per rank, boundaries on multiples of ``tile``
    (the CTA tile height) so no tile straddles two GPUs; the remainder tiles go
    to the first ranks, the ragged tail (M % tile) to the last non-empty block.
    Ranks beyond the number of tiles get empty blocks."""
    if M < 1 or world < 1 or tile < 1:
        raise ValueError("M, world and tile must be >= 1")
    tiles = -(-M // tile)
    base, extra = divmod(tiles, world)
    blocks, t = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        start = min(t * tile, M)
        stop = min((t + n) * tile, M)
        blocks.append(RowBlock(start, stop))
        t += n
    assert blocks[0].start == 0 and blocks[-1].stop == M or any(b.stop == M for b in blocks)
    return blocks


def check_in(store, rank: int, world: int, tag: str, timeout_s: float) -> None:
    """Host-side readiness barrier with a deadline, on a torch.distributed store."""
    store.set(f"exo_b200/{tag}/{rank}", b"1")
    deadline = time.monotonic() + timeout_s
    missing = list(range(world))
    while missing:
        missing = [r for r in missing if not _has(store, f"exo_b200/{tag}/{r}")]
        if not missing:
            return
        if time.monotonic() > deadline:
            raise ShardError(f"rank(s) {missing} did not check in within {timeout_s:.1f} s ({tag}); "
                             "no GPU work was enqueued")
        time.sleep(0.01)


def _has(store, key: str) -> bool:
    try:
        return bool(store.check([key]))
    except Exception:
        return False


class ShardedGemm:
    """The multi-GPU driver of the large GEMM.

    ``gemm(a_rows, b, c_rows)`` is the single-GPU kernel call (by default the bf16
    tensor-core entry point); it is a parameter so that the partitioning and
    exchange logic can be exercised on CPU ranks with the gloo backend."""

    def __init__(self, dist, M: int, N: int, K: int, gemm=None, tile: int = 128, timeout_s: float = 30.0,
                 store=None):
        self.dist = dist
        self.rank = dist.get_rank() if dist is not None else 0
        self.world = dist.get_world_size() if dist is not None else 1
        self.M, self.N, self.K = M, N, K
        self.blocks = row_blocks(M, self.world, tile)
        self.block = self.blocks[self.rank]
        self.timeout_s = timeout_s
        self.store = store
        self._gemm = gemm or _default_bf16_gemm
        self._round = 0
        self._dev_b = None  # this rank's device copy of B for host-operand steps

    def broadcast_b(self, b):
        """The only exchange: B from rank 0 into every rank's own memory."""
        if self.world == 1:
            return b
        if self.store is not None:
            self._round += 1
            check_in(self.store, self.rank, self.world, f"bcast{self._round}", self.timeout_s)
        # bytes are bytes: a uint8 view keeps every backend happy with any element type
        import torch

        self.dist.broadcast(b.view(torch.uint8) if b.is_contiguous() else b, src=0)
        return b

    def local_rows(self, full):
        """This rank's row block of a full M-row tensor."""
        return full[self.block.start:self.block.stop]

    def b_slices(self, n_cols: int) -> list[tuple[int, int]]:
        """Column ranges of B (rows of its [N, K] array), one per rank, for the
        upload-a-slice-then-all-gather exchange; equal sizes when world divides N."""
        base, extra = divmod(n_cols, self.world)
        out, start = [], 0
        for r in range(self.world):
            n = base + (1 if r < extra else 0)
            out.append((start, start + n))
            start += n
        return out

    def gather_b_from_host(self, b_host, device=None):
        """Every rank uploads its slice of the host copy of B and receives the other
        slices from its peers.  Returns this rank's full device copy (kept and reused
        across steps).  ``device`` None: CPU tensors stay on the CPU (gloo ranks)."""
        import torch

        if self._dev_b is None or self._dev_b.shape != b_host.shape or self._dev_b.dtype != b_host.dtype:
            self._dev_b = torch.empty(b_host.shape, dtype=b_host.dtype, device=device or b_host.device)
        full = self._dev_b
        slices = self.b_slices(b_host.shape[0])
        lo, hi = slices[self.rank]
        if hi > lo:
            full[lo:hi].copy_(b_host[lo:hi], non_blocking=True)
        if self.world == 1:
            return full
        if self.store is not None:
            self._round += 1
            check_in(self.store, self.rank, self.world, f"gather{self._round}", self.timeout_s)
        flat = full.view(torch.uint8) if full.dtype != torch.uint8 else full
        if len({h - l for (l, h) in slices}) == 1 and hasattr(self.dist, "all_gather_into_tensor") \
                and flat.is_cuda:
            self.dist.all_gather_into_tensor(flat, flat[lo:hi])
        else:  # ragged split (or a backend without the fused form): one broadcast per slice
            for r, (l, h) in enumerate(slices):
                if h > l:
                    self.dist.broadcast(flat[l:h], src=r)
        return full

    def step(self, a_rows, b, c_rows):
        if self.block.rows == 0 and self.world == 1:
            return c_rows
        if a_rows.shape[0] != self.block.rows or c_rows.shape[0] != self.block.rows:
            raise ShardError(f"rank {self.rank}: expected {self.block.rows} rows, got "
                             f"A {a_rows.shape[0]} / C {c_rows.shape[0]}")
        if self.world > 1 and not getattr(b, "is_cuda", False) and self._wants_device():
            # host operands on several ranks: B crosses PCIe once per job, not once per rank
            import torch

            b = self.gather_b_from_host(b, device=torch.device("cuda", torch.cuda.current_device()))
        if self.block.rows == 0:
            return c_rows
        self._gemm(a_rows, b, c_rows)
        return c_rows

    def _wants_device(self) -> bool:
        """True when the GEMM runs on a GPU (the default kernel call); a test-supplied
        ``gemm`` on CPU ranks keeps every tensor where it is."""
        return self._gemm is _default_bf16_gemm


def _default_bf16_gemm(a_rows, b, c_rows):
    from . import api

    rows, K = a_rows.shape
    N = b.shape[0]  # b is column-major K x N, i.e. an [N, K] array
    api.library().gemm_bf16_exo(None, rows, N, K, a_rows, b, c_rows)
