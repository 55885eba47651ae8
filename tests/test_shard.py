"""The multi-GPU path on CPU: row partitioning, the one broadcast, and
host-side failure detection, as world_size-2 (and 3) gloo ranks."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_row_blocks_cover_and_align():
    from exo_b200.shard import row_blocks

    for M, world, tile in [(32768, 8, 128), (1000, 3, 128), (100, 4, 128), (129, 2, 128), (4096, 1, 128), (5, 8, 1)]:
        blocks = row_blocks(M, world, tile)
        assert len(blocks) == world
        assert blocks[0].start == 0
        assert max(b.stop for b in blocks) == M
        for a, b in zip(blocks, blocks[1:]):
            assert a.stop == b.start or b.rows == 0
        for b in blocks:
            assert b.start % tile == 0 or b.rows == 0
        assert sum(b.rows for b in blocks) == M
    b8 = row_blocks(32768, 8)
    assert all(b.rows == 4096 for b in b8)


def _cpu_gemm(a_rows, b, c_rows):
    # stand-in for the GPU kernel on CPU ranks: the oracle's bf16 GEMM (checker code,
    # injected by the test; the product default is the CUDA entry point)
    sys.path.insert(0, ROOT)
    import oracle

    c_rows.copy_(torch.from_numpy(
        oracle.port().gemm_bf16(a_rows.numpy().view(np.uint16), b.numpy().view(np.uint16)).view(np.int16)))


def _worker(rank, world, port, M, N, K, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from exo_b200.shard import ShardedGemm
    from tests import inputs

    A = torch.from_numpy(inputs.normal_bf16(1, (M, K)).view(np.int16))
    B = torch.from_numpy(inputs.normal_bf16(2, (N, K)).view(np.int16)) if rank == 0 else torch.zeros((N, K), dtype=torch.int16)
    sg = ShardedGemm(dist, M, N, K, gemm=_cpu_gemm)
    sg.broadcast_b(B)
    a = sg.local_rows(A).contiguous()
    c = torch.empty((sg.block.rows, N), dtype=torch.int16)
    sg.step(a, B, c)
    q.put((rank, sg.block.start, sg.block.stop, c.numpy().copy()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,M", [(2, 300), (3, 517)])
def test_sharded_gemm_equals_single_rank(world, M):
    import oracle
    from tests import inputs

    N, K = 40, 64
    port = free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, M, N, K, q)) for r in range(world)]
    for p in procs:
        p.start()
    parts = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    full = oracle.port().gemm_bf16(inputs.normal_bf16(1, (M, K)), inputs.normal_bf16(2, (N, K)))
    got = np.zeros((M, N), np.uint16)
    for _, start, stop, c in parts:
        got[start:stop] = c.view(np.uint16)
    # sharding must not change a single bit: same kernel, same rows
    assert np.array_equal(got, full)


def _gather_worker(rank, world, port, N, K, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from exo_b200.shard import ShardedGemm
    from tests import inputs

    true_b = torch.from_numpy(inputs.normal_bf16(9, (N, K)).view(np.int16))
    sg = ShardedGemm(dist, 256, N, K, gemm=_cpu_gemm)
    lo, hi = sg.b_slices(N)[rank]
    mine = torch.full((N, K), 0x7FC0, dtype=torch.int16)  # only this rank's slice is valid on this rank
    mine[lo:hi] = true_b[lo:hi]
    for _ in range(2):  # second round reuses the rank's buffer
        full = sg.gather_b_from_host(mine)
        q.put((rank, bool(torch.equal(full, true_b)), (lo, hi)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,N", [(2, 40), (3, 40)])
def test_b_is_uploaded_in_slices_and_gathered(world, N):
    """The host-operand exchange of the sharded GEMM: every rank contributes only its own
    slice of B (equal slices at world 2, ragged 14/13/13 at world 3) and ends with all of it."""
    port = free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gather_worker, args=(r, world, port, N, 16, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = [q.get(timeout=120) for _ in range(2 * world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for (_, ok, _) in out), out
    slices = sorted({s for (_, _, s) in out})
    assert slices[0][0] == 0 and slices[-1][1] == N and all(a[1] == b[0] for a, b in zip(slices, slices[1:]))


def _late_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from exo_b200.shard import ShardError, ShardedGemm

    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), wait_for_workers=False)
    if rank == 1:
        q.put((rank, "absent"))
        return  # this rank never checks in: a failure made on the host

    class FakeDist:  # no collective may be reached
        def get_rank(self):
            return rank

        def get_world_size(self):
            return world

        def broadcast(self, *a, **k):
            raise AssertionError("collective enqueued although a rank is missing")

    sg = ShardedGemm(FakeDist(), 256, 8, 8, timeout_s=1.0, store=store)
    try:
        sg.broadcast_b(torch.zeros(8, 8))
        q.put((rank, "no error"))
    except ShardError as e:
        q.put((rank, "ShardError: " + str(e)))


def test_missing_rank_is_detected_on_the_host_before_any_collective():
    port = free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_late_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = dict(q.get(timeout=60) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    assert out[1] == "absent"
    assert out[0].startswith("ShardError") and "rank(s) [1]" in out[0]


def test_shape_mismatch_is_rejected():
    from exo_b200.shard import ShardError, ShardedGemm

    sg = ShardedGemm(None, 256, 8, 8, gemm=lambda *a: None)
    with pytest.raises(ShardError):
        sg.step(torch.zeros(100, 8), torch.zeros(8, 8), torch.zeros(256, 8))
