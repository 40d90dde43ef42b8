"""Bit-exact parity of GPU packing / unpacking with the reference-generated fixtures and the oracle."""
import numpy as np
import pytest
import torch

from oracle import ternary as T

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from tmq_b200 import ops
    return ops


@pytest.mark.parametrize("name", ["lin", "conv", "soft", "wide", "conv1x1", "ints", "bytes"])
def test_pack_golden(ops, gold_pack, name):
    W = torch.from_numpy(gold_pack[f"{name}_in"])
    ref = gold_pack[f"{name}_packed"]
    got_cuda = ops.compactify_ternary(W.cuda())
    assert got_cuda.is_cuda and got_cuda.dtype == torch.int32 and tuple(got_cuda.shape) == ref.shape
    assert np.array_equal(got_cuda.cpu().numpy(), ref)
    got_host = ops.compactify_ternary(W)              # host tensors make the round trip, like the reference API
    assert not got_host.is_cuda and np.array_equal(got_host.numpy(), ref)


@pytest.mark.parametrize("name", ["conv", "conv1x1"])
def test_unpack_golden_4d(ops, gold_pack, name):
    P = torch.from_numpy(gold_pack[f"{name}_packed"]).cuda()
    ref = gold_pack[f"{name}_expanded"]
    out = ops.expand_ternary(P, list(ref.shape), False)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("shape", [(1, 1), (16, 1), (17, 3), (15, 33), (64, 64), (100, 257), (11008 // 8, 4096 // 8)])
def test_pack_unpack_shapes(ops, shape):
    rng = np.random.default_rng(shape[0] * 1000 + shape[1])
    W = (rng.random(shape, dtype=np.float32) * 4 - 2).astype(np.float32)
    P = ops.compactify_ternary(torch.from_numpy(W).cuda())
    ref = T.pack(W)
    assert np.array_equal(P.cpu().numpy(), ref)
    back = ops.expand_ternary(P, list(shape))
    assert np.array_equal(back.cpu().numpy(), T.unpack(ref, shape))


def test_nonfinite_and_huge_values(ops):
    W = np.array([[np.inf, -np.inf, np.nan, 3e9, -3e9, 2.5, -2.5, 0.4, 0.5, -0.5, 1.5, 0.49999997]],
                 dtype=np.float32).T.copy()
    P = ops.compactify_ternary(torch.from_numpy(W).cuda())
    assert np.array_equal(P.cpu().numpy(), T.pack(W))


def test_full_size_roundtrip(ops):
    """BASELINE GEMV weight (11008 x 4096): pack -> unpack is the identity on ternary data, idempotent on repack."""
    gen = torch.Generator(device="cuda").manual_seed(0)
    u = torch.rand(11008, 4096, generator=gen, device="cuda")
    W = torch.where(u < 0.3, -1.0, torch.where(u < 0.7, 0.0, 1.0))
    P = ops.compactify_ternary(W)
    assert tuple(P.shape) == (4096, 688)
    back = ops.expand_ternary(P, [11008, 4096])
    assert torch.equal(back, W)
    assert torch.equal(ops.compactify_ternary(back), P)
    # a 256-row slab against the oracle
    sl = W[:256].cpu().numpy()
    assert np.array_equal(ops.compactify_ternary(W[:256].contiguous()).cpu().numpy(), T.pack(sl))
