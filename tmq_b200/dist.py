"""Multi-GPU plumbing for the paths that shard naturally (one process per GPU, torch.distributed over NCCL).

The reference is single-device; these are the three partitionings its workloads admit without changing results:

  * data-parallel QAT: every rank runs the full model on its slice of the batch; ONE all-reduce per step over a flat
    fp32 bucket that the parameters' .grad tensors are views of (`FlatGradBucket`);
  * column-sharded ternary linear: rank r owns output channels [n0_r, n1_r) of the packed weights, computes its
    column block with the local GEMM and the blocks are all-gathered (`ColumnShardedLinear`);
  * element / batch sharding with no data-path collective: `shard_range` (soft-step over a flat tensor, inference
    over a batch); the soft-step loss scalar needs one scalar all-reduce.

The collectives are torch.distributed's (NCCL on GPUs, gloo in CPU tests); the one fused step is the column-sharded
linear's GEMM, whose epilogue stores its block into every rank's result buffer (ColumnShardedLinear.fused).
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
    """All gradients of a model in one flat fp32 buffer, so a data-parallel step needs no per-tensor collectives.

    After construction every parameter's .grad is a view into `self.flat`; backward accumulates straight into it.
    `zero()` replaces optimizer.zero_grad(set_to_none=True), which would detach the views.

    bucket_bytes=None: ONE all-reduce over the whole buffer in allreduce_mean().  With a size, the buffer is cut into
    contiguous buckets walking the parameters from the last to the first (the order backward produces gradients in);
    a bucket's all-reduce is launched asynchronously from a post-accumulate hook the moment its last gradient has
    landed, so the collectives of the late layers run under the backward pass of the early ones and
    allreduce_mean() only waits."""

    def __init__(self, params, bucket_bytes=None):
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
        self.buckets = []                                # (begin, end) element ranges of self.flat, last layers first
        self._works, self._left, self._hooks = [], [], []
        if bucket_bytes is not None:
            end, count, owner = total, 0, {}
            for i in range(len(self.params) - 1, -1, -1):
                owner[i] = len(self.buckets)
                count += 1
                if (end - self.offsets[i]) * 4 >= bucket_bytes or i == 0:
                    self.buckets.append((self.offsets[i], end))
                    self._left.append(count)
                    end, count = self.offsets[i], 0
            self._sizes = list(self._left)
            self._works = [None] * len(self.buckets)
            for i, p in enumerate(self.params):
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(owner[i])))

    def _make_hook(self, b):
        def hook(_param):
            self._left[b] -= 1
            if self._left[b] == 0 and world()[1] > 1:
                lo, hi = self.buckets[b]
                self._works[b] = dist.all_reduce(self.flat[lo:hi], op=dist.ReduceOp.SUM, async_op=True)
        return hook

    def zero(self):
        self.flat.zero_()

    def allreduce_mean(self, group=None):
        """Average the gradients over the ranks in place (sum all-reduce(s), then one scale)."""
        _, n = world()
        if n == 1:
            if self.buckets:
                self._left = list(self._sizes)
            return None
        if not self.buckets:
            dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group)
        else:
            for b, (lo, hi) in enumerate(self.buckets):
                if self._works[b] is None:           # a parameter took no part in this backward: reduce its bucket now
                    self._works[b] = dist.all_reduce(self.flat[lo:hi], op=dist.ReduceOp.SUM, group=group, async_op=True)
            for b in range(len(self.buckets)):
                self._works[b].wait()
                self._works[b] = None
            self._left = list(self._sizes)
        self.flat.mul_(1.0 / n)
        return None


class PeerBuffer:
    """One CUDA tensor of the same shape on every rank of a single node, each mapped into every other rank's address
    space (torch symmetric memory), so that a kernel on one GPU can store straight into the others' copies over NVLink.
    `ptrs[r]` is the device address of rank r's tensor as seen from THIS process.  Raises when symmetric memory is not
    available; callers then keep to the NCCL route.  There is deliberately no second mapping route: handles exported
    through torch's CUDA IPC storage sharing are opened in the exporting device's context, and a kernel running on
    another device faulted on such a pointer."""

    def __init__(self, shape, dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm
        self.rank, self.world = world()
        self.tensor = symm.empty(tuple(shape), dtype=dtype, device=device)
        self._handle = symm.rendezvous(self.tensor, dist.group.WORLD if group is None else group)
        self.ptrs = [int(p) for p in self._handle.buffer_ptrs]
        if len(self.ptrs) != self.world or self.ptrs[self.rank] != self.tensor.data_ptr():
            raise RuntimeError("PeerBuffer: symmetric memory returned an unexpected mapping")
        self.kind = "symmetric_memory"


class ColumnShardedLinear:
    """y = x @ T^T for a ternary weight whose output channels are split over the ranks.

    `packed` is the reference-layout packed weight [K, ceil(N/16)] of the FULL matrix; shard boundaries are multiples
    of 128 channels (the GEMM's tile height, and a multiple of the 16-channel packing word).
    `matmul(x, packed_shard, n_shard, scale, bias)` is the local product; the default runs the CUDA GEMM, whose epilogue
    writes this rank's column block straight into its slot of the gather buffer, so the all-gather runs in place and no
    block is copied before or after the collective."""

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
        self._peer = {}              # rows -> two alternating PeerBuffers holding the full [rows, n_total] result on every rank
        self._turn = {}
        self._flag = None

    def _out_dtype(self, x):
        return x.dtype if x.dtype in (torch.bfloat16, torch.float32) else torch.bfloat16

    def local(self, x, out=None):
        """Column block [M, n1 - n0] of this rank, written into `out` (rows may be wider than the block) when given."""
        n = self.n1 - self.n0
        if self._matmul is not None:
            y = self._matmul(x, self.packed_shard, n, self.scale, self.bias)
            if out is None:
                return y
            out[:, :n].copy_(y)
            return out[:, :n]
        from . import ops
        if self._wt is None:
            self._wt = ops.prepack(self.packed_shard, n, ops.FMT_BF16)
        return ops.ternary_gemm(x, self._wt, n, self.scale, self.bias, out_dtype=self._out_dtype(x),
                                out=None if out is None else out[:, :n])

    def prepare_fused(self, rows, device, group=None):
        """The two alternating result buffers of `rows` rows for fused(), mapped between the ranks on first use (a
        collective call)."""
        pair = self._peer.get(rows)
        if pair is None:
            pair = self._peer[rows] = [PeerBuffer((rows, self.n_total), torch.bfloat16, device, group) for _ in range(2)]
            self._flag = torch.zeros(1, dtype=torch.int32, device=device)
            self._turn[rows] = 0
        return pair

    def fused(self, x, group=None):
        """Full row-major [M, n_total] bf16 result on every rank with GEMM and all-gather as ONE kernel: the epilogue
        of this rank's GEMM stores its column block into every rank's result buffer (peer mappings, plain stores over
        NVLink), so the transfer overlaps the multiplication tile by tile and nothing is copied afterwards.  One tiny
        all-reduce after the launch tells every rank that all blocks have landed.  Results alternate between two
        buffers: a rank can only start call i + 1 after every rank has passed the all-reduce of call i, i.e. after every
        rank's stream is done with result i - 1, which is the buffer call i + 1 overwrites.  The returned tensor is
        therefore valid until the next-but-one call with the same row count."""
        from . import ops
        if self.world == 1:
            return self.local(x)
        if x.dtype != torch.bfloat16:
            raise RuntimeError("ColumnShardedLinear.fused: bf16 activations only")
        m = x.shape[0]
        pair = self.prepare_fused(m, x.device, group)
        pb = pair[self._turn[m]]
        self._turn[m] ^= 1                      # per row count: each pair alternates on its own
        if self._wt is None:
            self._wt = ops.prepack(self.packed_shard, self.n1 - self.n0, ops.FMT_BF16)
        order = [self.rank] + [r for r in range(self.world) if r != self.rank]
        dsts = [pb.ptrs[r] + self.n0 * 2 for r in order]
        ops.ternary_gemm_bcast(x, self._wt, self.n1 - self.n0, dsts, self.n_total, self.scale, self.bias)
        dist.all_reduce(self._flag, group=group)
        return pb.tensor

    def __call__(self, x, group=None, chunks=1, blocked=False):
        """Full output on every rank.  chunks > 1 splits the rows so that the all-gather of one chunk runs under the
        GEMM of the next.  blocked=True returns the column blocks as they arrive, [chunks, world, M / chunks, widest]
        (chunks == 1: [world, M, widest]), without the final interleaving copy - a consumer that walks K in blocks
        can use them as they are; otherwise the result is the row-major [M, N] matrix."""
        if self.world == 1:
            y = self.local(x)
            return y.unsqueeze(0) if blocked else y
        widths = [b[1] - b[0] for b in self.bounds]
        widest = max(widths)
        m = x.shape[0]
        if chunks < 1 or m % chunks != 0:
            chunks = 1
        rows = m // chunks
        buf = torch.empty((chunks, self.world, rows, widest), dtype=self._out_dtype(x), device=x.device)
        works = []
        for c in range(chunks):
            mine = buf[c, self.rank]                                         # this rank's slot of the gather buffer
            self.local(x[c * rows:(c + 1) * rows], out=mine)
            if widths[self.rank] != widest:
                mine[:, widths[self.rank]:].zero_()                          # ragged last shard: defined padding
            works.append(dist.all_gather_into_tensor(buf[c].view(self.world * rows, widest), mine, group=group,
                                                     async_op=True))         # in place: input is a slice of the output
        for w_ in works:
            w_.wait()
        if blocked:
            return buf if chunks > 1 else buf[0]
        if all(wd == widest for wd in widths):
            return buf.permute(0, 2, 1, 3).reshape(m, self.n_total)
        full = buf.permute(0, 2, 1, 3).reshape(m, self.world, widest)
        return torch.cat([full[:, r, :wd] for r, wd in enumerate(widths)], dim=1)


def allreduce_scalar(t, group=None):
    """Sum a 0-d tensor (for instance the soft-step loss of a sharded weight tensor) over the ranks, in place."""
    _, n = world()
    if n > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t
