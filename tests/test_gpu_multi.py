"""Row-sharded bf16 GEMM over NCCL on real GPUs: the concatenated shards must be
bit-identical to the single-GPU result (same kernel, same tiles, rows are
independent).  Needs at least two GPUs; skipped otherwise."""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, M, N, K, q):
    try:
        _rank_body(rank, world, port, M, N, K, q)
    except Exception as e:  # report instead of leaving the parent to time out
        q.put(f"rank {rank}: {type(e).__name__}: {e}")


def _rank_body(rank, world, port, M, N, K, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from exo_b200.shard import ShardedGemm
    from tests import inputs

    A = torch.from_numpy(inputs.normal_bf16(71, (M, K)).view(np.int16)).cuda()
    B = torch.from_numpy(inputs.normal_bf16(72, (N, K)).view(np.int16)).cuda() if rank == 0 else \
        torch.zeros((N, K), dtype=torch.int16, device="cuda")
    sg = ShardedGemm(dist, M, N, K)
    sg.broadcast_b(B)
    c = torch.empty((sg.block.rows, N), dtype=torch.int16, device="cuda")
    sg.step(sg.local_rows(A).contiguous(), B, c)
    torch.cuda.synchronize()
    # NCCL has no int16: gather the raw bytes
    parts = [torch.empty((b.rows, N * 2), dtype=torch.uint8, device="cuda") for b in sg.blocks]
    dist.all_gather(parts, c.view(torch.uint8))
    if rank == 0:
        import exo_b200

        full = torch.empty((M, N), dtype=torch.int16, device="cuda")
        exo_b200.library().gemm_bf16_exo(None, M, N, K, A, B, full)
        torch.cuda.synchronize()
        q.put(bool(torch.equal(torch.cat(parts, 0), full.view(torch.uint8))))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_bf16_gemm_is_bitwise_equal_to_one_gpu():
    import torch
    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    M, N, K = 1024 * world, 1024, 512
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, world, port, M, N, K, q)) for r in range(world)]
    for p in procs:
        p.start()
    ok = q.get(timeout=150)
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()
    assert ok is True, ok
