"""Operator layer: the functions TMQ's layers call, with the reference's names and argument meaning, backed by the
C ABI of libtmq_b200.so.

Mirrors the pybind surface of the reference (`tmq_cuda`, tmq/tmq_cuda.cu:800-809, and `tmq_native`,
tmq/tmq_native.cpp:550-555): inputs are borrowed, outputs are freshly allocated on the input's device, wrong
devices / dtypes raise RuntimeError, the unimplemented half-precision paths raise ValueError.  Unlike the reference
the calls run on the current stream of the tensor's device and check contiguity.  This module only moves
pointers; every computation happens in the CUDA library, and nothing here works without it.
"""
import ctypes

import torch

from . import _lib
from ._lib import check, lib

_scratch = {}


def _stream(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _require_cuda_f32(t, name):
    if not isinstance(t, torch.Tensor) or t.device.type != "cuda":
        raise RuntimeError(f"{name}: expected a CUDA tensor")
    if t.dtype == torch.float16:
        raise ValueError("Not implemented yet")
    if t.dtype != torch.float32:
        raise ValueError("Expected either a float16 or a float32 tensor as input/output")
    return t if t.is_contiguous() else t.contiguous()


def reduce_scratch(device):
    """Scratch of the two-stage reductions for the CURRENT stream of `device` (zeroed once; the kernels leave it
    zeroed).  Calls that share a scratch buffer must be ordered on one stream, so every stream gets its own: a
    reduction on a side stream can then never meet one on the caller's stream in the same partial sums."""
    device = torch.device(device)
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (index, torch.cuda.current_stream(index).cuda_stream)
    buf = _scratch.get(key)
    if buf is None:
        buf = torch.zeros(lib().tmq_reduce_scratch_bytes(), dtype=torch.uint8, device=torch.device("cuda", index))
        _scratch[key] = buf
    return buf


# ------------------------------------------------------------------------------------------------ soft-step

def fwd_softstep(weights, digamma):
    w = _require_cuda_f32(weights, "fwd_softstep")
    out = torch.empty_like(w)
    with torch.cuda.device(w.device):
        check(lib().tmq_softstep_fwd(_ptr(w), _ptr(out), w.numel(), float(digamma), _stream(w)), "fwd_softstep")
    return out


def bwd_softstep(weights, digamma, scale, grad):
    w = _require_cuda_f32(weights, "bwd_softstep")
    g = _require_cuda_f32(grad, "bwd_softstep")
    if g.shape != w.shape:
        g = g.expand_as(w).contiguous()
    out = torch.empty_like(w)
    with torch.cuda.device(w.device):
        check(lib().tmq_softstep_bwd(_ptr(w), _ptr(g), _ptr(out), w.numel(), float(digamma), float(scale), _stream(w)),
              "bwd_softstep")
    return out


def fwd_softstep_derivative(weights, digamma, strength):
    w = _require_cuda_f32(weights, "fwd_softstep_derivative")
    out = torch.empty_like(w)
    with torch.cuda.device(w.device):
        check(lib().tmq_softstep_deriv_fwd(_ptr(w), _ptr(out), w.numel(), float(digamma), float(strength), _stream(w)),
              "fwd_softstep_derivative")
    return out


def bwd_softstep_derivative(weights, digamma, strength, grad):
    w = _require_cuda_f32(weights, "bwd_softstep_derivative")
    g = _require_cuda_f32(grad, "bwd_softstep_derivative")
    if g.shape != w.shape or not g.is_contiguous():
        g = g.expand_as(w).contiguous()
    out = torch.empty_like(w)
    with torch.cuda.device(w.device):
        check(lib().tmq_softstep_deriv_bwd(_ptr(w), _ptr(g), _ptr(out), w.numel(), float(digamma), float(strength),
                                           _stream(w)), "bwd_softstep_derivative")
    return out


def clamp(weights, lo, hi, out=None):
    w = _require_cuda_f32(weights, "clamp")
    out = torch.empty_like(w) if out is None else out
    with torch.cuda.device(w.device):
        check(lib().tmq_clamp(_ptr(w), _ptr(out), w.numel(), float(lo), float(hi), _stream(w)), "clamp")
    return out


def qloss_sum(weights, sharpness, strength):
    """fp64 0-d tensor: sum of the loss integrand over the tensor, never materialised."""
    w = _require_cuda_f32(weights, "qloss_sum")
    out = torch.empty((), dtype=torch.float64, device=w.device)
    scratch = reduce_scratch(w.device)
    with torch.cuda.device(w.device):
        check(lib().tmq_qloss_sum(_ptr(w), w.numel(), float(sharpness), float(strength), _ptr(out), _ptr(scratch),
                                  scratch.numel(), _stream(w)), "qloss_sum")
    return out


def fused_step(weights, grad, digamma, sharpness, strength, lo, hi, scale=1.0, gq=None, out=None):
    """One pass: (softstep(w), total gradient wrt w, clamp(w), fp64 loss sum).  `out` may carry preallocated
    (y, gw, wc, loss) buffers."""
    w = _require_cuda_f32(weights, "fused_step")
    g = _require_cuda_f32(grad, "fused_step")
    n = w.numel()
    if out is None:
        out = (torch.empty_like(w), torch.empty_like(w), torch.empty_like(w),
               torch.empty((), dtype=torch.float64, device=w.device))
    y, gw, wc, loss = out
    if gq is None:
        gq = float(torch.tensor(1.0, dtype=torch.float32) / torch.tensor(float(n), dtype=torch.float32))
    scratch = reduce_scratch(w.device)
    with torch.cuda.device(w.device):
        check(lib().tmq_softstep_fused_step(_ptr(w), _ptr(g), _ptr(y), _ptr(gw), _ptr(wc), _ptr(loss), n, float(digamma),
                                            float(scale), float(sharpness), float(strength), float(gq), float(lo),
                                            float(hi), _ptr(scratch), scratch.numel(), _stream(w)), "fused_step")
    return y, gw, wc, loss


_host_pipes = {}


class _HostPipe:
    """Streams, events and device staging buffers of fused_step_host for one (device, chunk size)."""

    SLOTS = 3

    def __init__(self, device, chunk):
        self.device, self.chunk = device, chunk
        with torch.cuda.device(device):
            self.s_in, self.s_k, self.s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
            self.buf = [[torch.empty(chunk, dtype=torch.float32, device=device) for _ in range(5)]
                        for _ in range(self.SLOTS)]           # per slot: w, g, y, gw, wc
            self.ev_in = [torch.cuda.Event() for _ in range(self.SLOTS)]
            self.ev_k = [torch.cuda.Event() for _ in range(self.SLOTS)]
            self.ev_out = [torch.cuda.Event() for _ in range(self.SLOTS)]
            self.loss = torch.zeros(1, dtype=torch.float64, device=device)


def fused_step_host(hw, hg, hy, hgw, hwc, digamma, sharpness, strength, lo, hi, scale=1.0, gq=None, device="cuda",
                    chunk_elems=1 << 22):
    """The fused element pass on HOST buffers: hw, hg (inputs) and hy, hgw, hwc (outputs) are flat float32 CPU tensors,
    pinned for full speed.  The tensors are cut into chunks that flow through three streams - host-to-device copies,
    the kernel, device-to-host copies - so that the two PCIe directions and the kernel overlap; at most three chunks of
    staging live on the device.  Returns the loss sum as a Python float (per-chunk fp64 sums added in chunk order) after
    every output has arrived: the call is synchronous."""
    for t in (hw, hg, hy, hgw, hwc):
        if t.dtype != torch.float32 or t.device.type != "cpu" or not t.is_contiguous() or t.numel() != hw.numel():
            raise RuntimeError("fused_step_host: expected equally sized contiguous float32 CPU tensors")
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    n = hw.numel()
    chunk = int(min(max(chunk_elems, 1 << 16), max(n, 1)))
    pipe = _host_pipes.get((device.index, chunk))
    if pipe is None:
        pipe = _HostPipe(device, chunk)
        _host_pipes[(device.index, chunk)] = pipe
    if gq is None:
        gq = float(torch.tensor(1.0, dtype=torch.float32) / torch.tensor(float(n), dtype=torch.float32))
    nchunks = (n + chunk - 1) // chunk
    if pipe.loss.numel() < nchunks:
        pipe.loss = torch.zeros(nchunks, dtype=torch.float64, device=device)
    hw1, hg1, hy1, hgw1, hwc1 = (t.view(-1) for t in (hw, hg, hy, hgw, hwc))
    with torch.cuda.device(device):
        start = torch.cuda.Event()
        start.record()
        for s in (pipe.s_in, pipe.s_k, pipe.s_out):
            s.wait_event(start)                   # everything the caller queued before this call comes first
        for c in range(nchunks):
            a, b = c * chunk, min(n, (c + 1) * chunk)
            m, slot = b - a, c % pipe.SLOTS
            dw, dg, dy, dgw, dwc = (t[:m] for t in pipe.buf[slot])
            if c >= pipe.SLOTS:
                pipe.s_in.wait_event(pipe.ev_out[slot])   # the slot's previous outputs have left the device
            with torch.cuda.stream(pipe.s_in):
                dw.copy_(hw1[a:b], non_blocking=True)
                dg.copy_(hg1[a:b], non_blocking=True)
                pipe.ev_in[slot].record()
            pipe.s_k.wait_event(pipe.ev_in[slot])
            with torch.cuda.stream(pipe.s_k):
                fused_step(dw, dg, digamma, sharpness, strength, lo, hi, scale=scale, gq=gq,
                           out=(dy, dgw, dwc, pipe.loss[c]))
                pipe.ev_k[slot].record()
            pipe.s_out.wait_event(pipe.ev_k[slot])
            with torch.cuda.stream(pipe.s_out):
                hy1[a:b].copy_(dy, non_blocking=True)
                hgw1[a:b].copy_(dgw, non_blocking=True)
                hwc1[a:b].copy_(dwc, non_blocking=True)
                pipe.ev_out[slot].record()
        pipe.s_out.synchronize()
        return float(pipe.loss[:nchunks].cpu().sum().item()) if nchunks > 1 else float(pipe.loss[0].item())


def selftest_const_div(digamma, device="cuda"):
    cnt = torch.zeros((), dtype=torch.int64, device=device)
    with torch.cuda.device(cnt.device):
        check(lib().tmq_selftest_const_div(float(digamma), _ptr(cnt), _stream(cnt)), "selftest_const_div")
    return int(cnt.item())


def selftest_div(per_b, b_begin=0, b_count=9 << 23, device="cuda"):
    """Mismatches of the range-specialised division against IEEE division (see tmq_selftest_div)."""
    cnt = torch.zeros((), dtype=torch.int64, device=device)
    with torch.cuda.device(cnt.device):
        check(lib().tmq_selftest_div(int(per_b), int(b_begin), int(b_count), _ptr(cnt), _stream(cnt)), "selftest_div")
    return int(cnt.item())


# ------------------------------------------------------------------------------------------------ multi-tensor

class MultiTensorPlan:
    """Device-resident table over a fixed list of weight tensors (one per registered layer) so that loss, its
    gradient and the clamp run as ONE launch each instead of one per layer."""

    def __init__(self, weights):
        assert len(weights) > 0
        self.device = weights[0].device
        for w in weights:
            if w.device != self.device or w.device.type != "cuda" or w.dtype != torch.float32 or not w.is_contiguous():
                raise RuntimeError("MultiTensorPlan: weights must be contiguous fp32 tensors on one CUDA device")
        self.ptrs = [w.data_ptr() for w in weights]
        self.shapes = [tuple(w.shape) for w in weights]
        # outputs of the gradient kernel live in one flat buffer, each tensor's slice 16-byte aligned
        self.offsets, total = [], 0
        for w in weights:
            self.offsets.append(total)
            total += (w.numel() + 3) // 4 * 4
        self.flat_elems = total
        n = len(weights)
        arr = (_lib.MtTensor * n)()
        for i, w in enumerate(weights):
            arr[i].w = w.data_ptr()
            arr[i].out = None
            arr[i].n = w.numel()
            arr[i].out_offset = self.offsets[i]
        nbytes = lib().tmq_mt_plan_bytes(arr, n)
        host = torch.empty(nbytes, dtype=torch.uint8)
        nchunks = ctypes.c_int(0)
        check(lib().tmq_mt_plan_build(arr, n, ctypes.c_void_p(host.data_ptr()), nbytes, ctypes.byref(nchunks)),
              "mt_plan_build")
        self.ntensors, self.nchunks = n, nchunks.value
        self.table = host.to(self.device)

    def matches(self, weights):
        return (len(weights) == len(self.ptrs) and all(w.data_ptr() == p for w, p in zip(weights, self.ptrs))
                and all(tuple(w.shape) == s for w, s in zip(weights, self.shapes)))

    def qloss(self, sharpness, strength):
        """fp64 0-d tensor: sum over tensors of mean(strength * S'(w; sharpness))."""
        out = torch.empty((), dtype=torch.float64, device=self.device)
        scratch = reduce_scratch(self.device)
        with torch.cuda.device(self.device):
            check(lib().tmq_mt_qloss(_ptr(self.table), self.ntensors, self.nchunks, float(sharpness), float(strength),
                                     _ptr(out), _ptr(scratch), scratch.numel(), _stream(out)), "mt_qloss")
        return out

    def qloss_bwd(self, sharpness, strength, upstream=None):
        """Gradients of qloss() wrt every tensor (fresh storage per call), scaled by the fp32 0-d `upstream`."""
        up = None
        if upstream is not None:
            up = upstream.to(device=self.device, dtype=torch.float32).reshape(()).contiguous()
        flat = torch.empty(self.flat_elems, dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            check(lib().tmq_mt_qloss_bwd(_ptr(self.table), self.ntensors, self.nchunks, float(sharpness),
                                         float(strength), _ptr(up) if up is not None else None, _ptr(flat),
                                         _stream(self.table)), "mt_qloss_bwd")
        grads = []
        for off, shape in zip(self.offsets, self.shapes):
            n = 1
            for d in shape:
                n *= d
            grads.append(flat[off:off + n].view(shape))
        return grads

    def clamp_(self, lo, hi):
        with torch.cuda.device(self.device):
            check(lib().tmq_mt_clamp(_ptr(self.table), self.ntensors, self.nchunks, float(lo), float(hi),
                                     _stream(self.table)), "mt_clamp")


# ------------------------------------------------------------------------------------------------ packing

class MultiTensorAdam:
    """torch.optim.Adam (no weight decay, no amsgrad) for a fixed list of fp32 CUDA parameters as ONE launch per step,
    with the QAT clamp fused in for the parameters listed in `clamp_params` (one more launch for the others).
    Gradients live in a flat buffer (each parameter's .grad is a view into it, as with dist.FlatGradBucket - pass that
    bucket to share its buffer), the moments in two more flat buffers."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, clamp_params=(), clamp=(-1.0, 1.0), bucket=None):
        self.params = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("MultiTensorAdam: no trainable parameters")
        self.lr, self.betas, self.eps, self.clamp, self.steps = float(lr), (float(betas[0]), float(betas[1])), float(eps), clamp, 0
        dev = self.params[0].device
        for p in self.params:
            if p.device != dev or dev.type != "cuda" or p.dtype != torch.float32 or not p.is_contiguous():
                raise RuntimeError("MultiTensorAdam: parameters must be contiguous fp32 tensors on one CUDA device")
        self.device = dev
        if bucket is not None:
            if [id(p) for p in bucket.params] != [id(p) for p in self.params]:
                raise ValueError("MultiTensorAdam: the bucket must hold the same parameters in the same order")
            self.offsets, self.grad = list(bucket.offsets), bucket.flat
        else:
            self.offsets, total = [], 0
            for p in self.params:
                self.offsets.append(total)
                total += (p.numel() + 3) // 4 * 4
            self.grad = torch.zeros(total, dtype=torch.float32, device=dev)
            for p, off in zip(self.params, self.offsets):
                p.grad = self.grad[off:off + p.numel()].view_as(p)
        self.exp_avg = torch.zeros_like(self.grad)
        self.exp_avg_sq = torch.zeros_like(self.grad)
        clamp_ids = {id(p) for p in clamp_params}
        groups = ([i for i, p in enumerate(self.params) if id(p) in clamp_ids],
                  [i for i, p in enumerate(self.params) if id(p) not in clamp_ids])
        self.groups = groups
        self.plans = [self._plan(idx) if idx else None for idx in groups]     # [clamped, plain]

    def _plan(self, idx):
        n = len(idx)
        arr = (_lib.MtTensor * n)()
        for j, i in enumerate(idx):
            p = self.params[i]
            arr[j].w = p.data_ptr()
            arr[j].out = self.grad.data_ptr() + 4 * self.offsets[i]
            arr[j].n = p.numel()
            arr[j].out_offset = self.offsets[i]
        nbytes = lib().tmq_mt_plan_bytes(arr, n)
        host = torch.empty(nbytes, dtype=torch.uint8)
        nchunks = ctypes.c_int(0)
        check(lib().tmq_mt_plan_build(arr, n, ctypes.c_void_p(host.data_ptr()), nbytes, ctypes.byref(nchunks)),
              "mt_plan_build")
        return host.to(self.device), n, nchunks.value, [self.params[i].data_ptr() for i in idx]

    def zero_grad(self):
        self.grad.zero_()

    @torch.no_grad()
    def step(self):
        for p, off in zip(self.params, self.offsets):
            if p.grad is None or p.grad.data_ptr() != self.grad.data_ptr() + 4 * off:
                raise RuntimeError("MultiTensorAdam: a parameter's .grad no longer views the flat gradient buffer "
                                   "(use zero_grad() of this object, not set_to_none)")
        self.steps += 1
        for k, plan in enumerate(self.plans):
            if plan is None:
                continue
            table, n, nchunks, ptrs = plan
            if any(q != r for q, r in zip(ptrs, [self.params[i].data_ptr() for i in self.groups[k]])):
                raise RuntimeError("MultiTensorAdam: a parameter's storage was rebound since construction")
            with torch.cuda.device(self.device):
                check(lib().tmq_mt_adam_clamp(_ptr(table), n, nchunks, _ptr(self.exp_avg), _ptr(self.exp_avg_sq), self.lr,
                                              self.betas[0], self.betas[1], self.eps, self.steps, 1 if k == 0 else 0,
                                              float(self.clamp[0]), float(self.clamp[1]), _stream(self.grad)),
                      "mt_adam_clamp")


def _work_device(t):
    """Packing runs on the GPU; host tensors make a round trip through the current device."""
    if t.device.type == "cuda":
        return t.device
    if not torch.cuda.is_available():
        raise _lib.TmqError("tmq_b200 needs a CUDA device: packing runs in the CUDA library and there is no CPU path")
    return torch.device("cuda", torch.cuda.current_device())


def compactify_ternary(tensor):
    """[N,K] or [O,I,ky,kx] float32|int32|int8 -> int32 packed [K, ceil(N/16)] or [I,ky,kx,ceil(O/16)] on the
    input's device (tmq/tmq_native.cpp:418-425)."""
    if tensor.dim() not in (2, 4):
        raise RuntimeError("compactify_ternary: expected a 2-D or 4-D tensor")
    fn = {torch.float32: "tmq_pack2b_f32", torch.int32: "tmq_pack2b_i32", torch.int8: "tmq_pack2b_i8"}.get(tensor.dtype)
    if fn is None:
        raise ValueError("Cannot handle the supplied data-type")
    dev = _work_device(tensor)
    w = tensor.detach().to(dev).contiguous()
    N = w.shape[0]
    K = w.numel() // N if N else 0
    Q = (N + 15) // 16
    out_shape = (K, Q) if w.dim() == 2 else (w.shape[1], w.shape[2], w.shape[3], Q)
    out = torch.empty(out_shape, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        check(getattr(lib(), fn)(_ptr(w), _ptr(out), N, K, _stream(w)), "compactify_ternary")
    return out.to(tensor.device)


def expand_ternary(packed, orig_shape, entropy_decode=False):
    """Packed int32 -> float32 {-1,0,+1} tensor of `orig_shape` (tmq/tmq_native.cpp:516-544; 2-D uses the true
    inverse of the packer, which the reference's 2-D routine is not)."""
    if entropy_decode:
        from .codec import decompress_ternary
        packed = decompress_ternary(packed, orig_shape)
    if packed.dtype != torch.int32:
        raise RuntimeError("expand_ternary: expected an int32 tensor")
    orig_shape = [int(s) for s in orig_shape]
    if len(orig_shape) not in (2, 4):
        raise ValueError("Shape needs to be of dim 2 or 4")
    N = orig_shape[0]
    K = 1
    for s in orig_shape[1:]:
        K *= s
    if packed.numel() != K * ((N + 15) // 16):
        raise RuntimeError("expand_ternary: packed tensor does not match the original shape")
    dev = _work_device(packed)
    p = packed.detach().to(dev).contiguous()
    out = torch.empty(orig_shape, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(lib().tmq_unpack2b_f32(_ptr(p), _ptr(out), N, K, _stream(p)), "expand_ternary")
    return out.to(packed.device)


# ------------------------------------------------------------------------------------------------ ternary GEMM

FMT_BF16, FMT_I8 = 0, 1
_status = {}
_watch = {}


def gemm_status_word(device):
    """Per-device int32 the GEMM kernels report bounded-wait failures into (0 = healthy)."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    buf = _status.get(key)
    if buf is None:
        buf = torch.zeros(1, dtype=torch.int32, device=device)
        _status[key] = buf
    return buf


def _raise_status(device, code):
    gemm_status_word(device).zero_()           # re-arm: the word is sticky, every launch skips while it is non-zero
    raise _lib.TmqError(f"ternary GEMM kernel reported status {code}: {lib().tmq_status_string(code).decode()}; "
                        "results produced on this device since the previous check are invalid")


def check_gemm_status(device="cuda"):
    """Synchronising check: raises if any GEMM / GEMV / convolution launch on this device gave up on a device-side
    wait, and re-arms the status word."""
    code = int(gemm_status_word(device).item())
    if code != 0:
        _raise_status(device, code)


class _StatusWatch:
    """Non-blocking watch over a device's status word.  A kernel that gives up on a bounded wait makes every later
    launch skip its work (the word is sticky) while the C calls keep returning TMQ_OK, so somebody has to look: every
    `EVERY` launches the word is copied to pinned host memory behind the work already queued, and the next operator
    call that finds the copy finished raises if it is non-zero.  No synchronisation is added; a failure surfaces
    within about 2 * EVERY operator calls instead of never."""

    EVERY = 32

    def __init__(self, device):
        self.device = device
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event = torch.cuda.Event()
        self.pending = False
        self.launches = 0

    def note_launch(self):
        if self.pending and self.event.query():
            self.pending = False
            code = int(self.host[0])
            if code != 0:
                _raise_status(self.device, code)
        self.launches += 1
        if not self.pending and self.launches % self.EVERY == 1 and not torch.cuda.is_current_stream_capturing():
            self.host.copy_(gemm_status_word(self.device), non_blocking=True)
            self.event.record()
            self.pending = True


def _launched(device):
    """Book-keeping after a tensor-core launch on `device` (see _StatusWatch)."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    w = _watch.get(key)
    if w is None:
        w = _watch[key] = _StatusWatch(torch.device("cuda", key))
    w.note_launch()


def prepack_row_words(k, fmt):
    """Row stride (int32 words) of the row-major prepacked formats for K = k: the K/16 words (K rounded up to 64) plus
    the padding that keeps rows copied into shared memory free of bank conflicts."""
    return int(lib().tmq_prepack_row_words(int(k), int(fmt) & 1))


def prepack(packed, columns, fmt=FMT_BF16):
    """Reference-layout packed weights int32 [K, ceil(N/16)] (or the 4-D conv form) -> prepacked int32
    [N, prepack_row_words(K, fmt)] in the bit order the GEMM kernels decode (fmt: FMT_BF16 or FMT_I8).  Done once per
    weight tensor."""
    if packed.dtype != torch.int32 or packed.device.type != "cuda":
        raise RuntimeError("prepack: expected a CUDA int32 tensor")
    N = int(columns)
    Q = (N + 15) // 16
    p = packed.contiguous().view(-1, Q)
    K = p.shape[0]
    if fmt not in (FMT_BF16, FMT_I8):
        raise ValueError("prepack: fmt must be FMT_BF16 or FMT_I8")
    out = torch.empty((N, lib().tmq_prepack_row_words(K, int(fmt))), dtype=torch.int32, device=p.device)
    with torch.cuda.device(p.device):
        check(lib().tmq_prepack(_ptr(p), _ptr(out), N, K, int(fmt), _stream(p)), "prepack")
    return out


GEMV_ROWS = 16      # activation rows one skinny-kernel launch takes (1 .. 8: one MMA tile, 9 .. 16: two)


def _pick_path(path, M):
    """auto: up to 24 rows go through the skinny kernel (one pass of up to 16 rows, or two), anything taller through the
    tiled tensor-core kernel (measured on 11008 x 4096: 17 rows 15.3 us skinny / 18.8 us tiled, 32 rows 20.8 / 18.8)."""
    if path != "auto":
        return path
    if M <= GEMV_ROWS + 8:
        return "gemv"
    return "tiles"


def _skinny_passes(call, M):
    """Runs call(m0, rows) over the M rows in passes of up to GEMV_ROWS; a pass the resident kernel cannot take (one
    SM's share of the weights beyond its shared-memory budget) is split into the 8-row passes of the streaming kernel."""
    m0 = 0
    while m0 < M:
        rows = min(GEMV_ROWS, M - m0)
        rc = call(m0, rows)
        if rc == -6 and rows > 8:
            rc = call(m0, 8)
            if rc == 0:
                rc = call(m0 + 8, rows - 8)
        check(rc, "ternary_gemv")
        m0 += rows


def _check_weights(name, wt, N, K, fmt):
    if wt is None or wt.dtype != torch.int32 or wt.dim() != 2 or wt.shape[0] != N or not wt.is_contiguous() \
            or wt.shape[1] != lib().tmq_prepack_row_words(K, fmt):
        raise RuntimeError(f"{name}: prepacked weights do not match the problem shape")


def ternary_gemm(x, wt, columns, scale=None, bias=None, out_dtype=torch.bfloat16, path="auto", out=None):
    """Y = scale * (x @ T^T) + bias with x bf16 [M, K]; fp32 accumulation; Y is bf16 or fp32 [M, N].
    wt: prepack(..., FMT_BF16).  path: "auto", or pin "tiles" (tiled tcgen05 GEMM) or "gemv" (warp-level MMA skinny
    kernel, 8 rows per pass).  out: optional preallocated [M, >= N] tensor of the output dtype whose rows may be
    strided (a column block of a wider matrix); it is written in place and returned."""
    if x.dtype != torch.bfloat16 or x.device.type != "cuda" or x.dim() != 2:
        raise RuntimeError("ternary_gemm: expected a 2-D CUDA bf16 activation tensor")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("ternary_gemm: output dtype must be bfloat16 or float32")
    x = x.contiguous()
    M, K = x.shape
    N = int(columns)
    _check_weights("ternary_gemm", wt, N, K, FMT_BF16)
    if out is None:
        y = torch.empty((M, N), dtype=out_dtype, device=x.device)
    else:
        if out.dtype != out_dtype or out.device != x.device or out.dim() != 2 or tuple(out.shape) != (M, N) \
                or out.stride(1) != 1 or out.stride(0) < N:
            raise RuntimeError("ternary_gemm: `out` must be an [M, N] tensor of the output dtype with unit column stride")
        y = out
    ldy = y.stride(0) if M > 1 else max(N, y.stride(0))
    if M == 0:
        return y
    sc = None if scale is None else scale.to(device=x.device, dtype=torch.float32).contiguous()
    bi = None if bias is None else bias.to(device=x.device, dtype=torch.float32).contiguous()
    psc, pbi = (_ptr(sc) if sc is not None else None), (_ptr(bi) if bi is not None else None)
    f32 = 1 if out_dtype == torch.float32 else 0
    path = _pick_path(path, M)
    st = gemm_status_word(x.device)
    with torch.cuda.device(x.device):
        if path == "gemv":
            esz = y.element_size()
            _skinny_passes(lambda m0, rows: lib().tmq_ternary_gemv_bf16(
                ctypes.c_void_p(x.data_ptr() + m0 * K * 2), _ptr(wt), psc, pbi, ctypes.c_void_p(y.data_ptr() + m0 * ldy * esz),
                rows, N, K, ldy, f32, _ptr(st), _stream(x)), M)
        elif path == "tiles":
            need = int(lib().tmq_ternary_gemm_workspace_bytes(M, N, K, 0))     # > 0: skinny, K is split over CTAs
            if need:
                ws = torch.empty(need, dtype=torch.uint8, device=x.device)     # stream-ordered caching allocator
                check(lib().tmq_ternary_gemm_bf16_splitk(_ptr(x), _ptr(wt), psc, pbi, _ptr(y), M, N, K, ldy, f32, _ptr(ws),
                                                         need, _ptr(st), _stream(x)), "ternary_gemm")
            else:
                check(lib().tmq_ternary_gemm_bf16(_ptr(x), _ptr(wt), psc, pbi, _ptr(y), M, N, K, ldy, f32, _ptr(st),
                                                  _stream(x)), "ternary_gemm")
        else:
            raise ValueError(f"ternary_gemm: unknown path {path!r}")
    _launched(x.device)
    return y


def ternary_gemm_bcast(x, wt, columns, dst_ptrs, ldy, scale=None, bias=None):
    """ternary_gemm (bf16 in, bf16 out, tiled kernel) whose epilogue stores the [M, columns] block at every address of
    `dst_ptrs` (device addresses, this GPU's buffer first, then peer mappings of other GPUs' buffers; row stride `ldy`
    elements everywhere): GEMM and all-gather of a column-sharded linear in one kernel.  The caller orders buffer
    reuse and completion across the ranks (see dist.ColumnShardedLinear.fused)."""
    if x.dtype != torch.bfloat16 or x.device.type != "cuda" or x.dim() != 2:
        raise RuntimeError("ternary_gemm_bcast: expected a 2-D CUDA bf16 activation tensor")
    x = x.contiguous()
    M, K = x.shape
    N = int(columns)
    _check_weights("ternary_gemm_bcast", wt, N, K, FMT_BF16)
    if not 1 <= len(dst_ptrs) <= 8 or int(ldy) < N:
        raise RuntimeError("ternary_gemm_bcast: 1 .. 8 destinations with a row stride of at least `columns`")
    if M == 0:
        return
    sc = None if scale is None else scale.to(device=x.device, dtype=torch.float32).contiguous()
    bi = None if bias is None else bias.to(device=x.device, dtype=torch.float32).contiguous()
    arr = (ctypes.c_void_p * len(dst_ptrs))(*[int(p) for p in dst_ptrs])
    st = gemm_status_word(x.device)
    with torch.cuda.device(x.device):
        check(lib().tmq_ternary_gemm_bf16_bcast(_ptr(x), _ptr(wt), _ptr(sc) if sc is not None else None,
                                                _ptr(bi) if bi is not None else None, arr, len(dst_ptrs), M, N, K, int(ldy),
                                                _ptr(st), _stream(x)), "ternary_gemm_bcast")
    _launched(x.device)


def ternary_gemm_i8(x, wt, columns, path="auto"):
    """Exact int32 Y = x @ T^T with x int8 [M, K]; wt: prepack(..., FMT_I8)."""
    if x.dtype != torch.int8 or x.device.type != "cuda" or x.dim() != 2:
        raise RuntimeError("ternary_gemm_i8: expected a 2-D CUDA int8 activation tensor")
    x = x.contiguous()
    M, K = x.shape
    N = int(columns)
    _check_weights("ternary_gemm_i8", wt, N, K, FMT_I8)
    y = torch.empty((M, N), dtype=torch.int32, device=x.device)
    if M == 0:
        return y
    path = _pick_path(path, M)
    st = gemm_status_word(x.device)
    with torch.cuda.device(x.device):
        if path == "gemv":
            _skinny_passes(lambda m0, rows: lib().tmq_ternary_gemv_i8(
                ctypes.c_void_p(x.data_ptr() + m0 * K), _ptr(wt), ctypes.c_void_p(y.data_ptr() + m0 * N * 4), rows, N, K, N,
                _ptr(st), _stream(x)), M)
        elif path == "tiles":
            need = int(lib().tmq_ternary_gemm_workspace_bytes(M, N, K, 1))
            if need:
                ws = torch.empty(need, dtype=torch.uint8, device=x.device)
                check(lib().tmq_ternary_gemm_i8_splitk(_ptr(x), _ptr(wt), _ptr(y), M, N, K, N, _ptr(ws), need, _ptr(st),
                                                       _stream(x)), "ternary_gemm_i8")
            else:
                check(lib().tmq_ternary_gemm_i8(_ptr(x), _ptr(wt), _ptr(y), M, N, K, N, _ptr(st), _stream(x)),
                      "ternary_gemm_i8")
        else:
            raise ValueError(f"ternary_gemm_i8: unknown path {path!r}")
    _launched(x.device)
    return y


GEMV_BATCH_MAX = 16   # matrices one batched skinny launch takes (TMQ_GEMV_BATCH_MAX)


def _pointer_array(tensors):
    """Host array of device pointers (None -> NULL) for the batched entry points."""
    arr = (ctypes.c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = None if t is None else t.data_ptr()
    return arr


def ternary_gemv_batched(x, wts, columns, scales=None, biases=None, out_dtype=torch.bfloat16, outs=None):
    """Several ternary matrices of one shape against M <= 8 activation rows each, GEMV_BATCH_MAX matrices per launch.

    x: bf16 or int8, [M, K] (all matrices share it: query / key / value, gate / up) or [len(wts), M, K] (one block per
    matrix: experts, independent layers).  wts: prepacked weights (FMT_BF16 for bf16 x, FMT_I8 for int8 x), all
    [columns, prepack_row_words(K)].  scales / biases: per-matrix fp32 [columns] tensors or None (bf16 only).
    Returns the list of [M, columns] results (bf16 / fp32 for bf16 x, exact int32 for int8 x); against
    ternary_gemm(..., path="gemv") per matrix only the fp32 summation order differs.  outs: optional preallocated contiguous results."""
    i8 = x.dtype == torch.int8
    if x.dtype not in (torch.bfloat16, torch.int8) or x.device.type != "cuda" or x.dim() not in (2, 3):
        raise RuntimeError("ternary_gemv_batched: expected CUDA bf16 or int8 activations, [M, K] or [matrices, M, K]")
    n = len(wts)
    x = x.contiguous()
    if x.dim() == 3 and x.shape[0] != n:
        raise RuntimeError("ternary_gemv_batched: one activation block per matrix expected")
    M, K = x.shape[-2:]
    N = int(columns)
    if M > 8:
        raise RuntimeError("ternary_gemv_batched: at most 8 activation rows per matrix")
    dtype = torch.int32 if i8 else out_dtype
    if not i8 and out_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("ternary_gemv_batched: output dtype must be bfloat16 or float32")
    for w in wts:
        _check_weights("ternary_gemv_batched", w, N, K, FMT_I8 if i8 else FMT_BF16)
    if outs is None:
        whole = torch.empty((n, M, N), dtype=dtype, device=x.device)
        outs = list(whole.unbind(0))
    elif len(outs) != n or any(o.dtype != dtype or tuple(o.shape) != (M, N) or not o.is_contiguous() or o.device != x.device
                               for o in outs):
        raise RuntimeError("ternary_gemv_batched: `outs` must be contiguous [M, N] tensors of the output dtype")
    if n == 0 or M == 0:
        return outs
    def f32(ts):
        return None if ts is None else [None if t is None else t.to(device=x.device, dtype=torch.float32).contiguous()
                                        for t in ts]
    scales, biases = f32(scales), f32(biases)
    stride = M * K if x.dim() == 3 else 0
    esz = x.element_size()
    st = gemm_status_word(x.device)
    with torch.cuda.device(x.device):
        for j0 in range(0, n, GEMV_BATCH_MAX):
            j1 = min(n, j0 + GEMV_BATCH_MAX)
            xp = ctypes.c_void_p(x.data_ptr() + j0 * stride * esz)
            W, Y = _pointer_array(wts[j0:j1]), _pointer_array(outs[j0:j1])
            if i8:
                rc = lib().tmq_ternary_gemv_batched_i8(xp, stride, W, Y, j1 - j0, M, N, K, N, _ptr(st), _stream(x))
            else:
                S = _pointer_array(scales[j0:j1]) if scales is not None else None
                B = _pointer_array(biases[j0:j1]) if biases is not None else None
                rc = lib().tmq_ternary_gemv_batched_bf16(xp, stride, W, S, B, Y, j1 - j0, M, N, K, N,
                                                         1 if dtype == torch.float32 else 0, _ptr(st), _stream(x))
            if rc == -6:      # one SM's share of a matrix exceeds the shared-memory budget: one launch per matrix
                for j in range(j0, j1):
                    xj = x[j] if x.dim() == 3 else x
                    if i8:
                        outs[j].copy_(ternary_gemm_i8(xj, wts[j], N, path="gemv"))
                    else:
                        ternary_gemm(xj, wts[j], N, None if scales is None else scales[j],
                                     None if biases is None else biases[j], dtype, path="gemv", out=outs[j])
            else:
                check(rc, "ternary_gemv_batched")
            _launched(x.device)
    return outs


def qat_linear_forward(x, weight, bias, hardness):
    """Training forward of a quantisation-aware Linear layer, x @ S(weight)^T + bias, with the soft staircase S evaluated
    inside the tensor-core GEMM's operand producers (never materialised).  x: CUDA bf16 [..., K] with K % 8 == 0;
    weight: the latent fp32 [N, K] tensor; bias: fp32 [N] or None.  Returns fp32 [..., N]."""
    if x.dtype != torch.bfloat16 or x.device.type != "cuda":
        raise RuntimeError("qat_linear_forward: expected CUDA bf16 activations")
    if weight.dtype != torch.float32 or weight.dim() != 2 or weight.device != x.device:
        raise RuntimeError("qat_linear_forward: expected a 2-D fp32 weight tensor on the activations' device")
    N, K = weight.shape
    if x.shape[-1] != K:
        raise RuntimeError("qat_linear_forward: activation width does not match the weights")
    lead = x.shape[:-1]
    x2 = x.reshape(-1, K).contiguous()
    w = weight.contiguous()
    M = x2.shape[0]
    y = torch.empty((M, N), dtype=torch.float32, device=x.device)
    if M == 0:
        return y.view(*lead, N)
    b = None if bias is None else bias.to(device=x.device, dtype=torch.float32).contiguous()
    st = gemm_status_word(x.device)
    need = int(lib().tmq_qat_linear_workspace_bytes(M, N, K))      # partial sums when K is split over several CTAs
    ws = torch.empty(need, dtype=torch.uint8, device=x.device) if need else None   # stream-ordered caching allocator
    with torch.cuda.device(x.device):
        check(lib().tmq_qat_linear_fwd_bf16(_ptr(x2), _ptr(w), _ptr(b) if b is not None else None, _ptr(y), M, N, K, N,
                                            float(hardness), _ptr(ws) if ws is not None else None, need, _ptr(st),
                                            _stream(x)), "qat_linear_forward")
    _launched(x.device)
    return y.view(*lead, N)


HAVE_IMPLICIT_CONV = True


def conv_patches(x, kernel, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
    """fp32 NCHW image batch -> bf16 patch matrix [B*OH*OW, Kp] in (ky, kx, c) order, K zero-padded to a multiple
    of 8; for layers whose channel count the implicit convolution cannot take."""
    if x.dtype != torch.float32 or x.device.type != "cuda" or x.dim() != 4:
        raise RuntimeError("conv_patches: expected a 4-D CUDA fp32 NCHW tensor")
    x = x.contiguous()
    b, c, h, w = x.shape
    (ky, kx), (sy, sx), (py, px), (dy, dx) = kernel, stride, padding, dilation
    oh = (h + 2 * py - dy * (ky - 1) - 1) // sy + 1
    ow = (w + 2 * px - dx * (kx - 1) - 1) // sx + 1
    kp = (ky * kx * c + 7) // 8 * 8
    out = torch.empty((b * oh * ow, kp), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().tmq_conv_patches_bf16(_ptr(x), _ptr(out), b, c, h, w, ky, kx, sy, sx, py, px, dy, dx, kp, _stream(x)),
              "conv_patches")
    return out, (b, oh, ow)


def ternary_conv2d_nhwc(x, wt, columns, kernel, stride=(1, 1), padding=(0, 0), dilation=(1, 1), scale=None, bias=None,
                        relu=False, residual=None, out_dtype=None):
    """Implicit-GEMM convolution on NHWC activations [B, H, W, C] (C % 64 == 0) -> NHWC [B, OH, OW, N].
    bf16 x: wt = prepack(FMT_BF16) of the packed weight with rows in (ky, kx, c) order; output bf16 (default) or fp32
    (out_dtype=torch.float32: no output rounding).  int8 x: wt = prepack(FMT_I8) of the same rows; exact int32 output,
    no scale / bias / residual / ReLU."""
    if x.device.type != "cuda" or x.dim() != 4 or not x.is_contiguous() or x.dtype not in (torch.bfloat16, torch.int8):
        raise RuntimeError("ternary_conv2d_nhwc: expected a contiguous 4-D CUDA bf16 or int8 NHWC tensor")
    i8 = x.dtype == torch.int8
    b, h, w, c = x.shape
    (ky, kx), (sy, sx), (py, px), (dy, dx) = kernel, stride, padding, dilation
    n = int(columns)
    if c % 64 != 0:
        raise RuntimeError("ternary_conv2d_nhwc: the channel count must be a multiple of 64")
    fmt = FMT_I8 if i8 else FMT_BF16
    if wt.dtype != torch.int32 or wt.shape[0] != n or wt.shape[1] != prepack_row_words(ky * kx * c, fmt):
        raise RuntimeError("ternary_conv2d_nhwc: prepacked weights do not match the problem shape")
    if out_dtype is None:
        out_dtype = torch.int32 if i8 else torch.bfloat16
    if out_dtype != (torch.int32 if i8 else out_dtype) or out_dtype not in (torch.bfloat16, torch.float32, torch.int32):
        raise ValueError("ternary_conv2d_nhwc: bf16 activations give bf16 or fp32, int8 activations int32")
    if i8 and (scale is not None or bias is not None or residual is not None or relu):
        raise ValueError("ternary_conv2d_nhwc: the int8 form returns the bare int32 sums")
    oh = (h + 2 * py - dy * (ky - 1) - 1) // sy + 1
    ow = (w + 2 * px - dx * (kx - 1) - 1) // sx + 1
    y = torch.empty((b, oh, ow, n), dtype=out_dtype, device=x.device)
    sc, bi = _opt_f32(scale, x.device), _opt_f32(bias, x.device)
    if residual is not None and (residual.dtype != torch.bfloat16 or tuple(residual.shape) != tuple(y.shape)
                                 or not residual.is_contiguous()):
        raise RuntimeError("ternary_conv2d_nhwc: the residual must be a contiguous bf16 tensor of the output's shape")
    st = gemm_status_word(x.device)
    geom = (b, h, w, c, n, ky, kx, sy, sx, py, px, dy, dx)
    with torch.cuda.device(x.device):
        if i8:
            check(lib().tmq_ternary_conv2d_i8(_ptr(x), _ptr(wt), _ptr(y), *geom, _ptr(st), _stream(x)), "ternary_conv2d_i8")
        else:
            fn = lib().tmq_ternary_conv2d_bf16_f32out if out_dtype == torch.float32 else lib().tmq_ternary_conv2d_bf16
            check(fn(_ptr(x), _ptr(wt), _ptr(sc) if sc is not None else None, _ptr(bi) if bi is not None else None,
                     _ptr(residual) if residual is not None else None, _ptr(y), *geom, 1 if relu else 0, _ptr(st),
                     _stream(x)), "ternary_conv2d_nhwc")
    _launched(x.device)
    return y


def conv_rows_kkc(packed, cin, ky, kx, terms=1, pad_to=8):
    """Packed convolution weights (reference layout: rows in (c, ky, kx) order, [cin * ky * kx, ceil(N/16)] or the 4-D form)
    -> the row order the implicit GEMM walks, (ky, kx, c), channel runs contiguous as in NHWC.  terms = 3 repeats each
    tap's channel block three times (for activations split into three bf16 terms along the channels); the row count is
    padded with zero rows to a multiple of `pad_to`."""
    rows = packed.contiguous().view(-1, packed.shape[-1])
    taps = int(ky) * int(kx)
    if rows.shape[0] != int(cin) * taps:
        raise RuntimeError("conv_rows_kkc: packed weights do not match the kernel geometry")
    r = rows.view(int(cin), taps, -1).transpose(0, 1)                  # [tap, c, Q]
    if terms > 1:
        r = r.unsqueeze(1).expand(taps, terms, int(cin), r.shape[-1])  # [tap, term, c, Q]
    r = r.reshape(-1, rows.shape[-1])
    pad = (-r.shape[0]) % int(pad_to)
    if pad:
        r = torch.nn.functional.pad(r, (0, 0, 0, pad))
    return r.contiguous()


def conv_rows_skkc(packed, cin, ky, kx):
    """Packed convolution weights (reference layout, rows in (c, ky, kx) order) -> rows in (64-channel slice, ky, kx,
    channel within the slice) order: the K order of the stride-1 shifted-window kernel, which takes all taps of one
    channel slice with a single copy."""
    rows = packed.contiguous().view(-1, packed.shape[-1])
    taps, cin = int(ky) * int(kx), int(cin)
    if rows.shape[0] != cin * taps or cin % 64 != 0:
        raise RuntimeError("conv_rows_skkc: packed weights do not match the kernel geometry (channels % 64 == 0)")
    r = rows.view(cin // 64, 64, taps, -1).permute(0, 2, 1, 3)         # [slice, tap, c64, Q]
    return r.reshape(-1, rows.shape[-1]).contiguous()


def conv_rows_stem(packed, cin, ky, kx, sx):
    """Packed weights of a few-channel convolution -> the K order of the descriptor-patch stem kernel: (filter row,
    [kx positions x CP channels] zero-padded to a multiple of 16), CP = 8 / sx channel slots per pixel.  None when the
    layer is outside that kernel's reach (sx not 1 or 2, more than CP channels)."""
    cin, ky, kx, sx = int(cin), int(ky), int(kx), int(sx)
    k_rows = int(lib().tmq_stem_rows_k(cin, ky, kx, sx))
    if k_rows == 0:
        return None
    cp = 8 // sx
    per_row = k_rows // ky
    rows = packed.contiguous().view(-1, packed.shape[-1])
    if rows.shape[0] != cin * ky * kx:
        raise RuntimeError("conv_rows_stem: packed weights do not match the kernel geometry")
    e = torch.arange(per_row, device=rows.device)
    kxi, c = e // cp, e % cp
    valid = (kxi < kx) & (c < cin)
    r = torch.arange(ky, device=rows.device).view(-1, 1)
    src = (c.clamp(max=cin - 1) * (ky * kx)).view(1, -1) + r * kx + kxi.clamp(max=kx - 1).view(1, -1)     # [ky, per_row]
    out = rows.index_select(0, src.reshape(-1)).view(ky, per_row, -1)
    out = torch.where(valid.view(1, -1, 1), out, torch.zeros_like(out))
    return out.reshape(k_rows, -1).contiguous()


def ternary_conv2d_stem_rows(x, wt, columns, kernel, stride=(1, 1), padding=(0, 0), scale=None, bias=None, relu=False,
                             pool=False):
    """Few-channel convolution with the patches read straight out of a bf16 copy of the input rows in shared memory (no
    patch matrix, no operand tile): x fp32 NCHW [B, C, H, W], wt = prepack(conv_rows_stem(...), FMT_BF16) -> bf16 NHWC.
    pool=True fuses ReLU and a 3 x 3 / stride 2 / padding 1 max pooling into the epilogue (64 output channels, even output
    height and width): the convolution's own output never reaches memory and the result is [B, OH/2, OW/2, 64].
    None when the shape is outside the kernel's limits."""
    if x.dtype != torch.float32 or x.device.type != "cuda" or x.dim() != 4:
        raise RuntimeError("ternary_conv2d_stem_rows: expected a 4-D CUDA fp32 NCHW tensor")
    x = x.contiguous()
    b, c, h, w = x.shape
    (ky, kx), (sy, sx), (py, px) = kernel, stride, padding
    n = int(columns)
    k_rows = int(lib().tmq_stem_rows_k(c, ky, kx, sx))
    if k_rows == 0:
        return None
    if wt.dtype != torch.int32 or wt.shape[0] != n or wt.shape[1] != prepack_row_words(k_rows, FMT_BF16):
        raise RuntimeError("ternary_conv2d_stem_rows: prepacked weights do not match the problem shape")
    oh, ow = (h + 2 * py - ky) // sy + 1, (w + 2 * px - kx) // sx + 1
    if pool and (oh % 2 or ow % 2):
        return None
    y = torch.empty((b, oh // 2, ow // 2, n) if pool else (b, oh, ow, n), dtype=torch.bfloat16, device=x.device)
    sc, bi = _opt_f32(scale, x.device), _opt_f32(bias, x.device)
    st = gemm_status_word(x.device)
    with torch.cuda.device(x.device):
        if pool:
            rc = lib().tmq_ternary_conv2d_stem_rows_pool_bf16(_ptr(x), _ptr(wt), _ptr(sc) if sc is not None else None,
                                                              _ptr(bi) if bi is not None else None, _ptr(y), b, c, h, w, n,
                                                              ky, kx, sy, sx, py, px, _ptr(st), _stream(x))
        else:
            rc = lib().tmq_ternary_conv2d_stem_rows_bf16(_ptr(x), _ptr(wt), _ptr(sc) if sc is not None else None,
                                                         _ptr(bi) if bi is not None else None, _ptr(y), b, c, h, w, n, ky,
                                                         kx, sy, sx, py, px, 1 if relu else 0, _ptr(st), _stream(x))
    if rc == -6:
        return None
    check(rc, "ternary_conv2d_stem_rows")
    _launched(x.device)
    return y


def ternary_conv2d_s1(x, wt, columns, kernel, padding=(0, 0), dilation=(1, 1), scale=None, bias=None, relu=False,
                      residual=None):
    """Unit-stride implicit-GEMM convolution on bf16 NHWC activations [B, H, W, C] (C % 64 == 0) with the input tile
    resident in shared memory for all filter taps; wt = prepack(conv_rows_skkc(...), FMT_BF16).  Returns bf16 NHWC, or
    None when the geometry is outside this kernel's limits (the caller then takes ternary_conv2d_nhwc)."""
    if x.dtype != torch.bfloat16 or x.device.type != "cuda" or x.dim() != 4 or not x.is_contiguous():
        raise RuntimeError("ternary_conv2d_s1: expected a contiguous 4-D CUDA bf16 NHWC tensor")
    b, h, w, c = x.shape
    (ky, kx), (py, px), (dy, dx) = kernel, padding, dilation
    n = int(columns)
    if c % 64 != 0 or ky * kx > 9:
        return None
    if wt.dtype != torch.int32 or wt.shape[0] != n or wt.shape[1] != prepack_row_words(ky * kx * c, FMT_BF16):
        raise RuntimeError("ternary_conv2d_s1: prepacked weights do not match the problem shape")
    oh, ow = h + 2 * py - dy * (ky - 1), w + 2 * px - dx * (kx - 1)
    if oh <= 0 or ow <= 0:
        raise RuntimeError("ternary_conv2d_s1: empty output")
    y = torch.empty((b, oh, ow, n), dtype=torch.bfloat16, device=x.device)
    sc, bi = _opt_f32(scale, x.device), _opt_f32(bias, x.device)
    if residual is not None and (residual.dtype != torch.bfloat16 or tuple(residual.shape) != tuple(y.shape)
                                 or not residual.is_contiguous()):
        raise RuntimeError("ternary_conv2d_s1: the residual must be a contiguous bf16 tensor of the output's shape")
    st = gemm_status_word(x.device)
    with torch.cuda.device(x.device):
        rc = lib().tmq_ternary_conv2d_s1_bf16(_ptr(x), _ptr(wt), _ptr(sc) if sc is not None else None,
                                              _ptr(bi) if bi is not None else None,
                                              _ptr(residual) if residual is not None else None, _ptr(y), b, h, w, c, n, ky,
                                              kx, py, px, dy, dx, 1 if relu else 0, _ptr(st), _stream(x))
    if rc == -6:
        return None
    check(rc, "ternary_conv2d_s1")
    _launched(x.device)
    return y


def split_f32(x2d, terms=3, kp=None):
    """fp32 [M, K] -> bf16 [M, terms * kp]: terms = 1 rounds, terms = 3 is the exact split x = lo + mid + hi (smallest
    term first) with term t in columns [t * kp, t * kp + K); kp >= K pads every term with zero columns."""
    if x2d.dtype != torch.float32 or x2d.device.type != "cuda" or x2d.dim() != 2:
        raise RuntimeError("split_f32: expected a 2-D CUDA float32 tensor")
    x2d = x2d.contiguous()
    m, k = x2d.shape
    kp = k if kp is None else int(kp)
    out = torch.empty((m, terms * kp), dtype=torch.bfloat16, device=x2d.device)
    if m:
        with torch.cuda.device(x2d.device):
            check(lib().tmq_split_f32_bf16(_ptr(x2d), _ptr(out), m, k, kp, int(terms), _stream(x2d)), "split_f32")
    return out


def nchw_to_nhwc_bf16(x, terms=1):
    """fp32 NCHW [B, C, H, W] (contiguous) -> bf16 NHWC [B, H, W, terms * C] in one pass (terms as in split_f32)."""
    if x.dtype != torch.float32 or x.device.type != "cuda" or x.dim() != 4:
        raise RuntimeError("nchw_to_nhwc_bf16: expected a 4-D CUDA float32 tensor")
    x = x.contiguous()
    b, c, h, w = x.shape
    y = torch.empty((b, h, w, terms * c), dtype=torch.bfloat16, device=x.device)
    if x.numel():
        with torch.cuda.device(x.device):
            check(lib().tmq_nchw_f32_to_nhwc_bf16(_ptr(x), _ptr(y), b, c, h, w, int(terms), _stream(x)), "nchw_to_nhwc_bf16")
    return y


def avgpool_nhwc(x):
    """Global average pooling of a contiguous bf16 NHWC tensor [B, H, W, C] (C even) -> bf16 [B, C], fp32 sums."""
    if x.dtype != torch.bfloat16 or x.device.type != "cuda" or x.dim() != 4 or not x.is_contiguous():
        raise RuntimeError("avgpool_nhwc: expected a contiguous 4-D CUDA bf16 NHWC tensor")
    b, h, w, c = x.shape
    y = torch.empty((b, c), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().tmq_avgpool_nhwc_bf16(_ptr(x), _ptr(y), b, h * w, c, _stream(x)), "avgpool_nhwc")
    return y


def ternary_conv2d_stem(x, wt, columns, kernel, stride=(1, 1), padding=(0, 0), scale=None, bias=None, relu=False):
    """Fused convolution for layers with few input channels: x fp32 NCHW [B, C, H, W]; wt = prepack(FMT_BF16) of the
    packed weights with rows in (ky, kx, c) order -> bf16 NHWC [B, OH, OW, N].  Returns None when the shape is outside the
    kernel's limits (the caller then builds patches and runs the GEMM)."""
    if x.dtype != torch.float32 or x.device.type != "cuda" or x.dim() != 4:
        raise RuntimeError("ternary_conv2d_stem: expected a 4-D CUDA fp32 NCHW tensor")
    x = x.contiguous()
    b, c, h, w = x.shape
    (ky, kx), (sy, sx), (py, px) = kernel, stride, padding
    n = int(columns)
    k_rows = None
    for cand in range(ky * kx * c, ky * kx * c + 64):          # the prepacked K may carry a few zero rows of padding
        if wt.shape[1] == prepack_row_words(cand, FMT_BF16):
            k_rows = cand
            break
    if wt.dtype != torch.int32 or wt.shape[0] != n or k_rows is None:
        raise RuntimeError("ternary_conv2d_stem: prepacked weights do not match the problem shape")
    oh, ow = (h + 2 * py - ky) // sy + 1, (w + 2 * px - kx) // sx + 1
    y = torch.empty((b, oh, ow, n), dtype=torch.bfloat16, device=x.device)
    sc, bi = _opt_f32(scale, x.device), _opt_f32(bias, x.device)
    st = gemm_status_word(x.device)
    with torch.cuda.device(x.device):
        rc = lib().tmq_ternary_conv2d_stem_bf16(_ptr(x), _ptr(wt), _ptr(sc) if sc is not None else None,
                                                _ptr(bi) if bi is not None else None, _ptr(y), b, c, h, w, n, ky, kx, sy, sx,
                                                py, px, k_rows, 1 if relu else 0, _ptr(st), _stream(x))
    if rc == -6:
        return None
    check(rc, "ternary_conv2d_stem")
    _launched(x.device)
    return y


def maxpool2d_nhwc(x, kernel, stride, padding, relu=False):
    """Max pooling on a contiguous bf16 NHWC tensor [B, H, W, C] (C % 8 == 0), torch's max_pool2d semantics; relu=True
    also applies max(0, .), i.e. folds a ReLU that preceded the pooling."""
    if x.dtype != torch.bfloat16 or x.device.type != "cuda" or x.dim() != 4 or not x.is_contiguous():
        raise RuntimeError("maxpool2d_nhwc: expected a contiguous 4-D CUDA bf16 NHWC tensor")
    b, h, w, c = x.shape
    k, s, p = int(kernel), int(stride), int(padding)
    oh, ow = (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1
    y = torch.empty((b, oh, ow, c), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().tmq_maxpool2d_nhwc_bf16(_ptr(x), _ptr(y), b, h, w, c, k, s, p, 1 if relu else 0, _stream(x)),
              "maxpool2d_nhwc")
    return y


class MaxPool2dTrain(torch.autograd.Function):
    """max_pool2d (square window, no dilation, floor mode) for fp32 CUDA activations in channels-last layout, forward and
    backward as two streaming kernels (the backward gathers: deterministic, no atomics).  Same values, winners and
    gradients as torch's."""

    @staticmethod
    def forward(ctx, x, k, s, p):
        b, c, h, w = x.shape
        xn = x.permute(0, 2, 3, 1)                                   # NHWC view of the channels-last tensor
        oh, ow = (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1
        y = torch.empty((b, c, oh, ow), dtype=torch.float32, device=x.device, memory_format=torch.channels_last)
        idx = torch.empty((b, oh, ow, c), dtype=torch.int8, device=x.device)
        with torch.cuda.device(x.device):
            check(lib().tmq_maxpool2d_nhwc_f32_fwd(_ptr(xn), _ptr(y), _ptr(idx), b, h, w, c, k, s, p, _stream(x)),
                  "maxpool2d_train")
        ctx.save_for_backward(idx)
        ctx.geom = (b, c, h, w, k, s, p)
        return y

    @staticmethod
    def backward(ctx, gy):
        (idx,) = ctx.saved_tensors
        b, c, h, w, k, s, p = ctx.geom
        gy = gy.contiguous(memory_format=torch.channels_last)
        gx = torch.empty((b, c, h, w), dtype=torch.float32, device=gy.device, memory_format=torch.channels_last)
        with torch.cuda.device(gy.device):
            check(lib().tmq_maxpool2d_nhwc_f32_bwd(_ptr(gy), _ptr(idx), _ptr(gx), b, h, w, c, k, s, p, _stream(gy)),
                  "maxpool2d_train")
        return gx, None, None, None


def maxpool2d_train(x, kernel, stride, padding):
    """Training max pooling: the library's kernels for fp32 CUDA tensors in channels-last layout with C % 4 == 0, torch's
    own max_pool2d for anything else."""
    k, s, p = int(kernel), int(stride), int(padding)
    if (x.dim() == 4 and x.is_cuda and x.dtype == torch.float32 and x.shape[1] % 4 == 0 and k <= 11 and 2 * p <= k
            and x.is_contiguous(memory_format=torch.channels_last) and x.shape[2] + 2 * p >= k and x.shape[3] + 2 * p >= k):
        return MaxPool2dTrain.apply(x, k, s, p)
    return torch.nn.functional.max_pool2d(x, k, s, p)


# ---- depthwise convolutions ------------------------------------------------------------------------------------------

def _dw_args(name, x, weights):
    if x.dtype != torch.float32 or x.device.type != "cuda":
        raise RuntimeError(f"{name}: expected a CUDA float32 activation tensor")
    if weights.dtype != torch.int32 or weights.device != x.device:
        raise RuntimeError(f"{name}: expected int32 packed weights on the activations' device")
    return x.contiguous(), weights.contiguous()


def _opt_f32(t, device):
    return None if t is None else t.to(device=device, dtype=torch.float32).contiguous()


def ternary_dwconv2d(x, weights, kernel, stride=(1, 1), padding=(0, 0), dilation=(1, 1), scale=None, bias=None):
    """Depthwise ternary convolution straight from the image: x fp32 NCHW [B, C, H, W], weights = packed
    [1, ky, kx, ceil(C/16)] (the reference's compact form of a [C, 1, ky, kx] kernel) -> fp32 [B, C, OH, OW] with torch
    conv2d's output size; optional per-channel scale and bias."""
    x, weights = _dw_args("ternary_dwconv2d", x, weights)
    if x.dim() != 4:
        raise RuntimeError("ternary_dwconv2d: expected a 4-D NCHW tensor")
    b, c, h, w = x.shape
    (ky, kx), (sy, sx), (py, px), (dy, dx) = kernel, stride, padding, dilation
    if weights.numel() != ky * kx * ((c + 15) // 16):
        raise RuntimeError("ternary_dwconv2d: packed weights do not match the channel count and kernel size")
    oh = (h + 2 * py - dy * (ky - 1) - 1) // sy + 1
    ow = (w + 2 * px - dx * (kx - 1) - 1) // sx + 1
    y = torch.empty((b, c, oh, ow), dtype=torch.float32, device=x.device)
    sc, bi = _opt_f32(scale, x.device), _opt_f32(bias, x.device)
    with torch.cuda.device(x.device):
        check(lib().tmq_ternary_dwconv2d_f32(_ptr(x), _ptr(weights), _ptr(sc) if sc is not None else None,
                                             _ptr(bi) if bi is not None else None, _ptr(y), b, c, h, w, ky, kx, sy, sx,
                                             py, px, dy, dx, _stream(x)), "ternary_dwconv2d")
    return y


def ternary_dwconvtrans2d(x, weights, kernel, stride=(1, 1), padding=(0, 0), dilation=(1, 1), output_padding=(0, 0),
                          scale=None, bias=None):
    """Depthwise ternary transposed convolution straight from the image (torch conv_transpose2d's output size)."""
    x, weights = _dw_args("ternary_dwconvtrans2d", x, weights)
    if x.dim() != 4:
        raise RuntimeError("ternary_dwconvtrans2d: expected a 4-D NCHW tensor")
    b, c, h, w = x.shape
    (ky, kx), (sy, sx), (py, px), (dy, dx), (opy, opx) = kernel, stride, padding, dilation, output_padding
    if weights.numel() != ky * kx * ((c + 15) // 16):
        raise RuntimeError("ternary_dwconvtrans2d: packed weights do not match the channel count and kernel size")
    oh = (h - 1) * sy - 2 * py + dy * (ky - 1) + 1 + opy
    ow = (w - 1) * sx - 2 * px + dx * (kx - 1) + 1 + opx
    y = torch.empty((b, c, oh, ow), dtype=torch.float32, device=x.device)
    sc, bi = _opt_f32(scale, x.device), _opt_f32(bias, x.device)
    with torch.cuda.device(x.device):
        check(lib().tmq_ternary_dwconvtrans2d_f32(_ptr(x), _ptr(weights), _ptr(sc) if sc is not None else None,
                                                  _ptr(bi) if bi is not None else None, _ptr(y), b, c, h, w, ky, kx, sy,
                                                  sx, py, px, dy, dx, opy, opx, _stream(x)), "ternary_dwconvtrans2d")
    return y


# ---- the reference's operator names (tmq/tmq_cuda.cu:800-809), same argument meaning ----------------------------------

def ternary_dwconv_cuda(x, weights, kx, ky, channels):
    """x fp32 [B, 1, P, kx*ky*C] / [B, P, kx*ky*C] / [P, kx*ky*C] (taps outermost, channels fastest) -> the same rank
    with `channels` as the last dimension [tmq/tmq_cuda.cu:607-644].  Every batch element is processed (the
    reference's launch only covers the first)."""
    x, weights = _dw_args("ternary_dwconv_cuda", x, weights)
    ntaps, c = int(kx) * int(ky), int(channels)
    if x.dim() not in (2, 3, 4) or (x.dim() == 4 and x.shape[1] != 1) or x.shape[-1] != ntaps * c:
        raise RuntimeError("ternary_dwconv_cuda: expected [.., pixels, kx*ky*channels] activations")
    if weights.numel() != ntaps * ((c + 15) // 16):
        raise RuntimeError("ternary_dwconv_cuda: packed weights do not match the channel count and kernel size")
    y = torch.empty(tuple(x.shape[:-1]) + (c,), dtype=torch.float32, device=x.device)
    rows = x.numel() // (ntaps * c)
    if rows:
        with torch.cuda.device(x.device):
            check(lib().tmq_ternary_dwconv_patches_f32(_ptr(x), _ptr(weights), _ptr(y), rows, c, ntaps, _stream(x)),
                  "ternary_dwconv_cuda")
    return y


def ternary_dwconvtrans_cuda(x, weights, kx, ky):
    """x fp32 [B, 1, P, C] / [B, P, C] / [P, C], weights packed [1, ky, kx, ceil(C/16)] -> [.., C*kx*ky, P] columns for
    F.fold [tmq/tmq_cuda.cu:647-686]."""
    x, weights = _dw_args("ternary_dwconvtrans_cuda", x, weights)
    if x.dim() not in (2, 3, 4) or (x.dim() == 4 and x.shape[1] != 1):
        raise RuntimeError("ternary_dwconvtrans_cuda: expected [.., pixels, channels] activations")
    ntaps, c, p = int(kx) * int(ky), int(x.shape[-1]), int(x.shape[-2])
    if weights.dim() != 4 or tuple(weights.shape) != (1, int(ky), int(kx), (c + 15) // 16):
        raise RuntimeError("ternary_dwconvtrans_cuda: expected packed weights of shape [1, ky, kx, ceil(C/16)]")
    b = x.numel() // (p * c)
    y = torch.empty(tuple(x.shape[:-2]) + (c * ntaps, p), dtype=torch.float32, device=x.device)
    if x.numel():
        with torch.cuda.device(x.device):
            check(lib().tmq_ternary_dwconvtrans_patches_f32(_ptr(x), _ptr(weights), _ptr(y), b, p, c, ntaps, _stream(x)),
                  "ternary_dwconvtrans_cuda")
    return y


_f32_weights = {}      # (id of the weight tensor, columns, k) -> (tensor, version, data_ptr, shape, stacked prepack)


def _stacked_prepack(weights, columns, k8):
    """Three stacked copies of the packed weights in the kernels' layout, cached per weight TENSOR OBJECT: the entry
    keeps the tensor alive (so its id cannot be recycled) and is rebuilt when the tensor's version counter, storage or
    shape changed.  A fresh tensor object (for instance `param.data`, which makes a new one on every access) is a
    cache miss: slower, never stale."""
    key = (id(weights), int(columns), k8)
    hit = _f32_weights.get(key)
    tag = (weights._version, weights.data_ptr(), tuple(weights.shape))
    if hit is None or hit[0] is not weights or hit[1] != tag:
        if len(_f32_weights) >= 32:
            _f32_weights.clear()
        p = weights.contiguous().view(-1, weights.shape[-1])
        if k8 > p.shape[0]:
            p = torch.nn.functional.pad(p, (0, 0, 0, k8 - p.shape[0]))
        hit = (weights, tag, prepack(torch.cat([p, p, p], dim=0), columns, FMT_BF16))
        _f32_weights[key] = hit
    return hit[2]


def ternary_gemm_f32(x2d, weights, columns, scale=None, bias=None):
    """fp32 activations [M, K] x reference-layout packed weights int32 [K, ceil(N/16)] -> fp32 [M, N].  x is split
    exactly into three bf16 terms (hi + mid + lo) that ride along K against three stacked copies of the weights:
    every product is exact, accumulation is fp32 on the tensor cores."""
    if x2d.dtype != torch.float32 or x2d.device.type != "cuda" or x2d.dim() != 2:
        raise RuntimeError("ternary_gemm_f32: expected a 2-D CUDA float32 tensor")
    if weights.dtype != torch.int32 or weights.device != x2d.device:
        raise RuntimeError("ternary_gemm_f32: expected int32 packed weights on the activations' device")
    k = x2d.shape[1]
    rows = weights.numel() // weights.shape[-1]
    if rows != k:
        raise RuntimeError("ternary_gemm_f32: activation width does not match the packed weights")
    kp = (k + 7) // 8 * 8
    return ternary_gemm(split_f32(x2d, 3, kp), _stacked_prepack(weights, columns, kp), int(columns), scale, bias,
                        out_dtype=torch.float32)


def ternary_mmm_cuda(x, weights, columns):
    """x fp32 [M, K] / [B, M, K] / [1, B, M, K], weights int32 [K, ceil(N/16)] -> fp32 [.., M, N]
    [tmq/tmq_cuda.cu:478-549]; one launch for the whole batch."""
    if x.dim() not in (2, 3, 4) or (x.dim() == 4 and x.shape[0] != 1):
        raise RuntimeError("ternary_mmm_cuda: expected [M, K], [B, M, K] or [1, B, M, K] activations")
    y = ternary_gemm_f32(x.contiguous().view(-1, x.shape[-1]), weights, columns)
    return y.view(tuple(x.shape[:-1]) + (int(columns),))


def ternary_mvm_cuda(x, weights, columns):
    """x fp32 [K] / [1, K] / [1, 1, K] / [1, 1, 1, K] -> fp32 [.., N] [tmq/tmq_cuda.cu:563-603]."""
    if x.dim() not in (1, 2, 3, 4) or any(int(s) != 1 for s in x.shape[:-1]):
        raise RuntimeError("ternary_mvm_cuda: expected a single activation row")
    y = ternary_gemm_f32(x.contiguous().view(1, -1), weights, columns)
    return y.view(tuple(x.shape[:-1]) + (int(columns),))
