"""Multi-GPU plumbing for the paths that shard naturally (one process per GPU, torch.distributed over NCCL).

The reference is single-device; these are the three partitionings its workloads admit without changing results:

  * data-parallel QAT: every rank runs the full model on its slice of the batch; ONE all-reduce per step over a flat
    fp32 bucket that the parameters' .grad tensors are views of (`FlatGradBucket`);
  * column-sharded ternary linear: rank r owns output channels [n0_r, n1_r) of the packed weights, computes its
    column block with the local GEMM and the blocks are all-gathered (`ColumnShardedLinear`);
  * element / batch sharding with no data-path collective: `shard_range` (soft-step over a flat tensor, inference
    over a batch); the soft-step loss scalar needs one scalar all-reduce.

Nothing here launches kernels of its own; the collectives are torch.distributed's (NCCL on GPUs, gloo in CPU tests).
"""
import torch
import torch.distributed as dist


def world():
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def shard_range(n, rank, world_size, align=1):
    """Contiguous slice [begin, end) of n items for `rank`; slice boundaries are multiples of `align`."""
    units = (n + align - 1) // align
    base, extra = divmod(units, world_size)
    begin_u = rank * base + min(rank, extra)
    end_u = begin_u + base + (1 if rank < extra else 0)
    return min(begin_u * align, n), min(end_u * align, n)


class FlatGradBucket:
    """All gradients of a model in one flat fp32 buffer, so a data-parallel step needs a single all-reduce.

    After construction every parameter's .grad is a view into `self.flat`; backward accumulates straight into it.
    `zero()` replaces optimizer.zero_grad(set_to_none=True), which would detach the views."""

    def __init__(self, params):
        self.params = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("FlatGradBucket: no trainable parameters")
        dev, total = self.params[0].device, 0
        self.offsets = []
        for p in self.params:
            if p.device != dev or p.dtype != torch.float32:
                raise ValueError("FlatGradBucket: parameters must be fp32 and on one device")
            self.offsets.append(total)
            total += (p.numel() + 3) // 4 * 4           # 16-byte aligned slices
        self.flat = torch.zeros(total, dtype=torch.float32, device=dev)
        for p, off in zip(self.params, self.offsets):
            p.grad = self.flat[off:off + p.numel()].view_as(p)

    def zero(self):
        self.flat.zero_()

    def allreduce_mean(self, group=None):
        """Average the gradients over the ranks in place (sum all-reduce, then one scale)."""
        _, n = world()
        if n == 1:
            return None
        work = dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group)
        self.flat.mul_(1.0 / n)
        return work


class ColumnShardedLinear:
    """y = x @ T^T for a ternary weight whose output channels are split over the ranks.

    `packed` is the reference-layout packed weight [K, ceil(N/16)] of the FULL matrix (every rank may hold it, or
    only its own slice via `from_shard`); shard boundaries are multiples of 128 channels (the GEMM's tile height,
    and a multiple of the 16-channel packing word).  `matmul(x, packed_shard, n_shard)` is the local product; the
    default runs the CUDA GEMM."""

    ALIGN = 128

    def __init__(self, packed, n_total, scale=None, bias=None, rank=None, world_size=None, matmul=None):
        r, w = world()
        self.rank = r if rank is None else rank
        self.world = w if world_size is None else world_size
        self.n_total = int(n_total)
        self.bounds = [shard_range(self.n_total, i, self.world, self.ALIGN) for i in range(self.world)]
        n0, n1 = self.bounds[self.rank]
        self.n0, self.n1 = n0, n1
        q0, q1 = n0 // 16, (n1 + 15) // 16
        self.packed_shard = packed[:, q0:q1].contiguous()
        self.scale = None if scale is None else scale[n0:n1].contiguous()
        self.bias = None if bias is None else bias[n0:n1].contiguous()
        self._matmul = matmul
        self._wt = None

    def local(self, x):
        """Column block [M, n1 - n0] of this rank."""
        n = self.n1 - self.n0
        if self._matmul is not None:
            return self._matmul(x, self.packed_shard, n, self.scale, self.bias)
        from . import ops
        if self._wt is None:
            self._wt = ops.prepack(self.packed_shard, n, ops.FMT_BF16)
        return ops.ternary_gemm(x, self._wt, n, self.scale, self.bias, out_dtype=x.dtype
                                if x.dtype in (torch.bfloat16, torch.float32) else torch.bfloat16)

    def __call__(self, x, group=None, chunks=1, blocked=False):
        """Full output on every rank.  chunks > 1 splits the rows so that the all-gather of one chunk overlaps the
        GEMM of the next (equal shards only).  blocked=True returns the column blocks as [world, M, n_shard] without
        the final interleaving copy (a consumer that walks K in blocks can use them as they are)."""
        if self.world == 1:
            y = self.local(x)
            return y.unsqueeze(0) if blocked else y
        widths = [b[1] - b[0] for b in self.bounds]
        widest = max(widths)
        equal = all(wd == widest for wd in widths)
        m = x.shape[0]
        if chunks > 1 and equal and m >= chunks:
            first = self.local(x[:1])
            gathered = torch.empty((self.world, m, widest), dtype=first.dtype, device=first.device)
            edges = [m * i // chunks for i in range(chunks + 1)]
            works = []
            for i in range(chunks):
                r0, r1 = edges[i], edges[i + 1]
                y_c = self.local(x[r0:r1]).contiguous()
                stage = torch.empty((self.world * (r1 - r0), widest), dtype=y_c.dtype, device=y_c.device)
                works.append((dist.all_gather_into_tensor(stage, y_c, group=group, async_op=True), stage, r0, r1))
            for work, stage, r0, r1 in works:
                work.wait()
                gathered[:, r0:r1, :].copy_(stage.view(self.world, r1 - r0, widest))
            return gathered if blocked else gathered.permute(1, 0, 2).reshape(m, self.n_total)
        send = self.local(x).contiguous()
        if send.shape[1] != widest:      # collectives want equal shapes: the ragged last shard is padded for the trip
            send = torch.nn.functional.pad(send, (0, widest - send.shape[1]))
        stacked = torch.empty((self.world * send.shape[0], widest), dtype=send.dtype, device=send.device)
        dist.all_gather_into_tensor(stacked, send, group=group)      # rank blocks concatenated along dim 0
        gathered = stacked.view(self.world, send.shape[0], widest)
        if blocked and equal:
            return gathered
        if equal:
            return gathered.permute(1, 0, 2).reshape(send.shape[0], self.n_total)
        return torch.cat([gathered[r, :, :wd] for r, wd in enumerate(widths)], dim=1)


def allreduce_scalar(t, group=None):
    """Sum a 0-d tensor (for instance the soft-step loss of a sharded weight tensor) over the ranks, in place."""
    _, n = world()
    if n > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t
