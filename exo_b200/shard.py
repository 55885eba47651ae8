"""Row-sharded GEMM over the GPUs of one node: one process per GPU.

``C[rows r] = A[rows r] @ B`` needs all of B but only its own rows of A and C
(apps/x86/sgemm/sgemm.py:20-23 has no dependence between rows), so a large GEMM
is split into contiguous row blocks of A and C, one per rank; B is broadcast
once from rank 0 (NCCL over NVLink when the tensors are CUDA tensors) and then
every rank runs the same single-GPU kernel on its block.  There is no
collective inside a step.

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

    def step(self, a_rows, b, c_rows):
        if self.block.rows == 0:
            return c_rows
        if a_rows.shape[0] != self.block.rows or c_rows.shape[0] != self.block.rows:
            raise ShardError(f"rank {self.rank}: expected {self.block.rows} rows, got "
                             f"A {a_rows.shape[0]} / C {c_rows.shape[0]}")
        self._gemm(a_rows, b, c_rows)
        return c_rows


def _default_bf16_gemm(a_rows, b, c_rows):
    from . import api

    rows, K = a_rows.shape
    N = b.shape[0]  # b is column-major K x N, i.e. an [N, K] array
    api.library().gemm_bf16_exo(None, rows, N, K, a_rows, b, c_rows)
