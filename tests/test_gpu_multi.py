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
        import oracle

        full = torch.empty((M, N), dtype=torch.int16, device="cuda")
        exo_b200.library().gemm_bf16_exo(None, M, N, K, A, B, full)
        torch.cuda.synchronize()
        same = bool(torch.equal(torch.cat(parts, 0), full.view(torch.uint8)))
        # and the gathered result against the oracle on a row sample that touches every rank's block
        rows = sorted({b.start for b in sg.blocks} | {b.stop - 1 for b in sg.blocks} | {M // 2 + 77})
        idx = torch.tensor(rows, device="cuda")
        got = inputs.bf16_bits_to_f32(torch.cat(parts, 0).view(torch.int16)[idx].cpu().numpy().view(np.uint16))
        port = oracle.port()
        port.set_threads(os.cpu_count() or 1)
        ref = inputs.bf16_bits_to_f32(port.gemm_bf16(A[idx].cpu().numpy().view(np.uint16),
                                                     B.cpu().numpy().view(np.uint16)))
        close = bool((np.abs(got - ref) <= 2.0 ** -7 * np.abs(ref) + 1e-3 * np.sqrt(K) * 4e-4).all())
        q.put(True if same and close else f"bitwise equal to one GPU: {same}; within tolerance of the oracle: {close}")
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_bf16_gemm_is_bitwise_equal_to_one_gpu():
    import torch
    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    # 5120 x 8192 per rank = 10 x 32 tiles of 512 x 256: every rank (and the one-GPU run) takes the
    # CTA-pair kernel that the scaling benchmark times, not the single-CTA kernel of small problems
    M, N, K = 5120 * world, 8192, 512
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
