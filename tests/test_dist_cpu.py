"""Multi-rank host logic on CPU: two gloo ranks.  Covers the flat gradient bucket (data-parallel QAT), the
column-sharded linear with its all-gather (local product injected, the CUDA GEMM is covered by the GPU tests) and
the shard arithmetic."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

from oracle import ternary as T
from tmq_b200 import dist as tdist


def test_shard_range_covers_everything_once():
    for n, w, a in [(100, 3, 1), (11008, 8, 128), (28672, 8, 128), (130, 4, 128), (1, 2, 1), (1 << 26, 8, 4)]:
        pieces = [tdist.shard_range(n, r, w, a) for r in range(w)]
        assert pieces[0][0] == 0 and pieces[-1][1] == n
        for (b0, e0), (b1, e1) in zip(pieces, pieces[1:]):
            assert e0 == b1 and b0 <= e0
        for b, e in pieces[:-1]:
            assert (b % a == 0 or b == n) and (e % a == 0 or e == n)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cpu_matmul(x, packed_shard, n, scale, bias):
    W = torch.from_numpy(T.unpack(packed_shard.numpy(), (n, packed_shard.shape[0])))
    y = x @ W.T
    if scale is not None:
        y = y * scale
    if bias is not None:
        y = y + bias
    return y


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # ---- data-parallel gradient bucket
        torch.manual_seed(0)
        model = nn.Sequential(nn.Linear(12, 7), nn.ReLU(), nn.Linear(7, 3))
        bucket = tdist.FlatGradBucket(model.parameters())
        gen = torch.Generator().manual_seed(100)
        x_all, y_all = torch.randn(8, 12, generator=gen), torch.randn(8, 3, generator=gen)
        b, e = tdist.shard_range(8, rank, world)
        bucket.zero()
        nn.functional.mse_loss(model(x_all[b:e]), y_all[b:e]).backward()
        bucket.allreduce_mean()
        got = [p.grad.clone() for p in model.parameters()]
        # the same thing on one process: mean of the per-shard gradients
        want = [torch.zeros_like(p) for p in model.parameters()]
        for r in range(world):
            rb, re = tdist.shard_range(8, r, world)
            model.zero_grad(set_to_none=True)
            nn.functional.mse_loss(model(x_all[rb:re]), y_all[rb:re]).backward()
            for w_, p in zip(want, model.parameters()):
                w_ += p.grad / world
        ok_grad = all(torch.allclose(g, w_, rtol=1e-6, atol=1e-7) for g, w_ in zip(got, want))
        # the overlapped form: small buckets, all-reduces launched from gradient hooks during backward; two steps in a
        # row, so the hook counters must re-arm
        torch.manual_seed(0)
        model_b = nn.Sequential(nn.Linear(12, 7), nn.ReLU(), nn.Linear(7, 3))
        bucket_b = tdist.FlatGradBucket(model_b.parameters(), bucket_bytes=64)
        ok_grad = ok_grad and len(bucket_b.buckets) >= 2 and bucket_b.buckets[0][1] == bucket_b.flat.numel()
        for _ in range(2):
            bucket_b.zero()
            nn.functional.mse_loss(model_b(x_all[b:e]), y_all[b:e]).backward()
            bucket_b.allreduce_mean()
            ok_grad = ok_grad and all(torch.allclose(p.grad, w_, rtol=1e-6, atol=1e-7)
                                      for p, w_ in zip(model_b.parameters(), want))
        # ---- column-sharded ternary linear (uneven shards: 300 channels over 2 ranks, 128-aligned)
        rng = np.random.default_rng(1)
        N, K, M = 300, 40, 5
        W = rng.integers(-1, 2, (N, K)).astype(np.float32)
        P = torch.from_numpy(T.pack(W))
        scale, bias = torch.rand(N, generator=gen) + 0.5, torch.randn(N, generator=gen)
        xs = torch.randn(M, K, generator=gen)
        lin = tdist.ColumnShardedLinear(P, N, scale, bias, matmul=_cpu_matmul)
        y = lin(xs)
        full = (xs @ torch.from_numpy(W).T) * scale + bias
        ok_cols = torch.allclose(y, full, rtol=1e-6, atol=1e-6) and lin.bounds == [(0, 256), (256, 300)]
        # equal shards take the single all_gather_into_tensor route
        N2 = 512
        W2 = rng.integers(-1, 2, (N2, K)).astype(np.float32)
        lin2 = tdist.ColumnShardedLinear(torch.from_numpy(T.pack(W2)), N2, matmul=_cpu_matmul)
        full2 = xs @ torch.from_numpy(W2).T
        ok_cols = ok_cols and torch.allclose(lin2(xs), full2, rtol=1e-6, atol=1e-6)
        xs6 = torch.randn(6, K, generator=gen)
        full6 = xs6 @ torch.from_numpy(W2).T
        ok_cols = ok_cols and torch.allclose(lin2(xs6, chunks=2), full6, rtol=1e-6, atol=1e-6)      # overlapped variant
        ok_cols = ok_cols and torch.allclose(lin2(xs, chunks=2), full2, rtol=1e-6, atol=1e-6)       # 5 rows: one chunk
        blocks = lin2(xs, blocked=True)
        ok_cols = ok_cols and blocks.shape == (world, M, N2 // world) and torch.allclose(
            blocks.permute(1, 0, 2).reshape(M, N2), full2, rtol=1e-6, atol=1e-6)
        blocks2 = lin2(xs6, blocked=True, chunks=3)
        ok_cols = ok_cols and blocks2.shape == (3, world, 2, N2 // world) and torch.allclose(
            blocks2.permute(0, 2, 1, 3).reshape(6, N2), full6, rtol=1e-6, atol=1e-6)
        # ---- scalar all-reduce
        s = tdist.allreduce_scalar(torch.tensor(float(rank + 1), dtype=torch.float64))
        ok_scalar = s.item() == sum(range(1, world + 1))
        with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
            f.write(f"{int(ok_grad)} {int(ok_cols)} {int(ok_scalar)}")
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert open(tmp_path / f"rank{r}.txt").read() == "1 1 1", r
