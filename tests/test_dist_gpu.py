"""Two-GPU check of the fused GEMM + all-gather (the GEMM epilogue stores its column block into every rank's result
buffer over NVLink): every rank must end up with the whole row-major product, bit-identical to the NCCL route and to
the single-GPU kernel on the full matrix.  Runs as two child processes, one per GPU; skipped on a one-GPU machine."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, N, K, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    import torch.distributed as dist
    from tmq_b200 import dist as tdist
    from tmq_b200 import ops
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        gen = torch.Generator(device=dev).manual_seed(7)                  # same seed: the same matrix on every rank
        u = torch.rand(N, K, generator=gen, device=dev)
        W = torch.where(u < 0.3, -1.0, torch.where(u < 0.7, 0.0, 1.0))
        P = ops.compactify_ternary(W)
        scale = torch.rand(N, generator=gen, device=dev) * 0.09 + 0.01
        bias = torch.randn(N, generator=gen, device=dev)
        X = torch.randn(M, K, generator=gen, device=dev).to(torch.bfloat16)
        lin = tdist.ColumnShardedLinear(P, N, scale, bias, rank=rank, world_size=world)
        whole = ops.ternary_gemm(X, ops.prepack(P, N, ops.FMT_BF16), N, scale, bias, path="tiles")
        via_nccl = lin(X)
        results = []
        for rep in range(3):                                              # the buffer is reused: three rounds
            Xr = (X * (rep + 1)).to(torch.bfloat16)
            got = lin.fused(Xr).clone()
            want = ops.ternary_gemm(Xr, ops.prepack(P, N, ops.FMT_BF16), N, scale, bias, path="tiles")
            results.append(bool(torch.equal(got, want)))
        ops.check_gemm_status(dev)
        ok = bool(torch.equal(via_nccl, whole)) and all(results)
        out.put((rank, ok, lin._peer[M][0].kind))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (300, 1152, 520), (1024, 4096, 1024)])
def test_fused_gemm_allgather_two_gpus(M, N, K):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, M, N, K, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()                                                           # the exact children started above
    assert not alive, "a rank did not finish"
    assert all(p.exitcode == 0 for p in procs)
    got = sorted(out.get(timeout=10) for _ in range(2))
    assert [g[1] for g in got] == [True, True], got
