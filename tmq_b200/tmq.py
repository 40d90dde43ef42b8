"""TMQ's Python API on top of the B200 kernels: same names, signatures and behaviour as the reference's
`tmq/tmq.py`, with the hot paths re-plumbed onto libtmq_b200.so.

What is kept (reference file:line in brackets): `QuantMode`, `TensorType` [tmq/tmq.py:49-72],
`QuantizationScheduleBuilder` [:75-82], `QuantizationControl` [:85-310], the autograd functions `SoftStep`
[:315-438] and `SoftStepDerivative` [:441-493], the layer drop-ins `Linear` [:573-765], `Conv2d` [:769-973],
`ConvTranspose2d` [:978-1087], and the model-level helpers `quantize_weights`, `quantize_model`,
`compressed_state_dict`, `prepare_compressed_load`, `load_compressed_state_dict`, `expand_compact_layers`
[:1090-1319], including the state-dict metadata keys `tmq.tensor_type`, `tmq.shape`, `tmq.quant`.

What differs, on purpose:
  * the soft-step functions, the quantization loss, the clamp, packing and compact inference run in the CUDA
    library; tensors must live on a CUDA device (there is no CPU path in this package);
  * `QuantizationControl.quantization_loss()` and `.clamp()` issue ONE launch over all registered layers;
  * compact inference works for any number of rows / any batch, fuses `post_scale` and bias into the GEMM epilogue,
    accepts fp32 (exact three-way bf16 split), bf16 and int8 activations, and convolutions go through the same
    tensor-core GEMM; `Linear.forward` does not dump tensors to /tmp [tmq/tmq.py:624-635];
  * `expand_compact_layers` on 2-D weights returns the true inverse of the packer.
"""
import fnmatch
from enum import Enum

import torch
from torch import nn
from torch.autograd.function import Function

from . import codec, ops
from ._lib import lib as _load_library

_load_library()  # fail loudly at import when the CUDA library has not been built
CUDA_EXT_AVAILABLE = True
NATIVE_EXT_AVAILABLE = True

# operator names the reference imports from its extensions, re-exported for code that used them directly
fwd_softstep = ops.fwd_softstep
bwd_softstep = ops.bwd_softstep
fwd_softstep_derivative = ops.fwd_softstep_derivative
bwd_softstep_derivative = ops.bwd_softstep_derivative
compactify_ternary = ops.compactify_ternary
expand_ternary = ops.expand_ternary
compress_ternary = codec.compress_ternary
decompress_ternary = codec.decompress_ternary


class QuantMode(Enum):
    NONE = 0
    TERNARY = 1
    TWO_BIT = 2
    THREE_BIT = 3
    FOUR_BIT = 4
    FIVE_BIT = 5
    SIX_BIT = 6
    EIGHT_BIT = 8


class TensorType(Enum):
    FLOAT_32BIT = 0
    FLOAT_16BIT = 1
    COMPACT_TERNARY_32BIT = 2
    COMPRESSED_TERNARY_32BIT = 3


class QuantizationScheduleBuilder:
    @staticmethod
    def default_schedule(max_epochs: int):
        assert max_epochs >= 50, "Need at least 50 epochs for a default schedule"
        return (int(max_epochs * 0.3), int(max_epochs * 0.8), int(max_epochs * 0.875), int(max_epochs * 0.93),
                max_epochs)


def _require_cuda(t, what):
    if t.device.type != "cuda":
        raise RuntimeError(f"{what}: tmq_b200 runs on CUDA tensors only (got a {t.device.type} tensor); "
                           "move the model to a CUDA device")


class QuantizationControl:
    """Schedules the hardness (`digamma`) and the loss penalty per epoch and fans `clamp`, `quantize` and
    `quantization_loss` out over every registered layer [tmq/tmq.py:85-310]."""

    def __init__(self, epoch_knots=None, digamma_range=(0.1, 6), qpenalty_range=None, quant_mode=QuantMode.TERNARY,
                 post_scale=False, init_range=None, device="cpu"):
        assert epoch_knots is None or len(epoch_knots) == 5
        assert len(digamma_range) == 2, "Need to supply a start/end value for the digamma parameter of the softstep function"
        assert digamma_range[0] >= 0.05, "Initial digamma value must be >= 0.05"
        assert digamma_range[0] <= 1, "Initial digamma value must be <= 1"
        assert digamma_range[1] <= 20.0, "Final digamma value must be <= 20"
        assert digamma_range[1] >= 3, "Final digamma value must be >= 3"
        assert digamma_range[0] <= digamma_range[1], "Please supply a valid range for digamma"
        self._warmup_epochs = 7
        if epoch_knots is not None:
            assert epoch_knots[0] >= self._warmup_epochs + 5, \
                "At least %d epochs required to reach halfway point" % (self._warmup_epochs + 5)
            self.max_epochs = epoch_knots[4]
        else:
            self.max_epochs = 0
        self.quantization = quant_mode
        self.epoch_knots = epoch_knots
        self.post_scale = post_scale
        self.digamma_start = max(0.05, digamma_range[0])
        self.digamma_end = max(3, digamma_range[1])
        self.digamma = self.digamma_start
        self.qpenalty = qpenalty_range[0] if qpenalty_range is not None else 0
        self.qpenalty_sharpness = 5.0
        self.inference_mode = self.max_epochs == 0
        self.device = device
        self._registry = {}
        self._last_cycle = -1
        self._digamma_cycle_start = 0
        self._digamma_cycle_end = 0
        self._cycle_len = 15
        if quant_mode == QuantMode.TERNARY:
            self.clamp_values = (-1., 1.)
        else:
            bits = int(quant_mode.value)
            self.clamp_values = (-2 ** bits, (2 ** bits) - 1)
        self.init_range = init_range if init_range is not None else self.clamp_values
        if qpenalty_range is not None:
            assert len(qpenalty_range) == 2, "Quantization penalty needs to supply a range"
            self.qpenalty_range = qpenalty_range
        else:
            self.qpenalty_range = (0, 0)
        self._plan = None

    # ---- schedule ------------------------------------------------------------------------------------------------

    @staticmethod
    def _blend(e_from, e_to, e, v_from, v_to):
        frac = min(1, max(0, (e - e_from) / (e_to - e_from)))
        return frac * v_to + (1 - frac) * v_from

    def _segment(self, e):
        """Index of the schedule segment epoch e falls in: 0..3 before the knots 0..3, 4 from knot 3 on."""
        knots = self.epoch_knots
        if e >= knots[3]:
            return 4
        seg = 0
        while seg < 3 and e >= knots[seg]:
            seg += 1
        return seg

    def _ramp(self, seg, e):
        """Un-cycled hardness ramp: start -> 3 over segment 0, 3 -> end over segment 1, end afterwards."""
        if seg >= 2:
            return self.digamma_end
        if seg == 0:
            return self._blend(self._warmup_epochs, self.epoch_knots[0], e, self.digamma_start, 3.0)
        return self._blend(self.epoch_knots[0], self.epoch_knots[1], e, 3.0, self.digamma_end)

    def step(self, epoch):
        """Advance `digamma` and `qpenalty` to `epoch`; stateful (cycle restarts), call once per epoch in order."""
        if self.epoch_knots is None:
            return
        if epoch >= self.epoch_knots[3]:
            self.qpenalty = self.qpenalty_range[1]
            self.digamma = self.digamma_end
            return
        if epoch <= self._warmup_epochs:
            return
        seg = self._segment(epoch)
        first_cycle_ready = seg != 0 or epoch >= self._warmup_epochs + self._cycle_len
        if self._last_cycle == -1 and first_cycle_ready:
            # open a new cycle: drop to 45 % of the ramp and climb to where the ramp will be one cycle later
            ahead = self._segment(epoch + self._cycle_len)
            if ahead < 4:
                self._digamma_cycle_start = max(self.digamma_start, self._ramp(seg, epoch) * 0.45)
                self._digamma_cycle_end = self._ramp(ahead, epoch + self._cycle_len)
                self._last_cycle = epoch
                self.digamma = self._digamma_cycle_start
        elif epoch < self._warmup_epochs + self._cycle_len:
            self.digamma = self._ramp(seg, epoch)
        elif epoch <= self._last_cycle + self._cycle_len:
            self.digamma = self._blend(self._last_cycle, self._last_cycle + self._cycle_len, epoch,
                                       self._digamma_cycle_start, self._digamma_cycle_end)
        else:
            self._last_cycle = -1
        if seg >= 2:
            self.qpenalty = self._blend(self.epoch_knots[2], self.epoch_knots[3], epoch, self.qpenalty_range[0],
                                        self.qpenalty_range[1])

    def inference(self):
        self.inference_mode = True

    def register_node(self, name, node):
        self._registry[name] = node
        self._plan = None

    # ---- all-layer operations: one launch each -----------------------------------------------------------------------

    def _float_weights(self):
        ws = []
        for node in self._registry.values():
            w = node.weight
            if w.dtype == torch.float32:
                _require_cuda(w, "QuantizationControl")
                ws.append(w)
        return ws

    def _multi_tensor_plan(self, weights):
        datas = [w.data if w.data.is_contiguous() else None for w in weights]
        if any(d is None for d in datas):
            raise RuntimeError("QuantizationControl: layer weights must be contiguous")
        if self._plan is None or not self._plan.matches(datas):
            self._plan = ops.MultiTensorPlan(datas)
        return self._plan

    def clamp(self, slack=0):
        """Clamp every registered weight to the quantization range (widened by `slack`), in place, in one launch."""
        lo, hi = self.clamp_values[0] - slack, self.clamp_values[1] + slack
        weights = self._float_weights()
        if weights:
            self._multi_tensor_plan(weights).clamp_(lo, hi)

    def collect_grad_norms(self):
        norms = {}
        for name, node in self._registry.items():
            if node.weight.grad is not None:
                norms[name] = node.weight.grad.norm()
        return norms

    def quantize(self):
        """Snap every registered weight onto the staircase levels (final step, not for checkpoints)."""
        for node in self._registry.values():
            node.weight.data = torch.round(SoftStep.map(node.weight.data, self))

    def quantization_loss(self, penalty=None):
        """Sum over layers of mean(penalty * S'(w; sharpness)): one fused reduction launch, differentiable."""
        strength = penalty if penalty is not None else self.qpenalty
        weights = self._float_weights()
        if not weights:
            return None
        return _AllLayerQuantLoss.apply(self, float(self.qpenalty_sharpness), float(strength), *weights)


class _AllLayerQuantLoss(Function):
    """Fused replacement of the per-layer `torch.mean(SoftStepDerivative.apply(...))` + Python sum
    [tmq/tmq.py:298-310, :698-699, :889-891]."""

    @staticmethod
    def forward(ctx, ctrl, sharpness, strength, *weights):
        plan = ctrl._multi_tensor_plan(weights)
        ctx.plan, ctx.sharpness, ctx.strength = plan, sharpness, strength
        return plan.qloss(sharpness, strength).to(torch.float32)

    @staticmethod
    def backward(ctx, grad_output):
        grads = ctx.plan.qloss_bwd(ctx.sharpness, ctx.strength, grad_output)
        return (None, None, None, *grads)


class SoftStep(Function):
    """Differentiable staircase (piecewise rational polynomial) applied to the weights [tmq/tmq.py:315-438]."""

    @staticmethod
    @torch.no_grad()
    def map(weight: torch.Tensor, ctrl: QuantizationControl) -> torch.Tensor:
        assert ctrl, "Control instance is required"
        d = ctrl.digamma
        base = torch.floor(weight.data)
        arg = d * weight.data - d * base - d / 2.0
        return SoftStep.sigmoid(arg) / (2.0 * SoftStep.scalar_sigmoid(d / 2)) + 0.5 + base

    @staticmethod
    @torch.no_grad()
    def dmap(weight: torch.Tensor, ctrl: QuantizationControl) -> torch.Tensor:
        assert ctrl, "Control instance is required"
        d = ctrl.digamma
        arg = weight.data * d - d * torch.floor(weight.data) - d / 2
        return d * SoftStep.dsigmoid(arg) / (2.0 * SoftStep.scalar_sigmoid(d / 2))

    @staticmethod
    def sigmoid(input: torch.Tensor) -> torch.Tensor:
        x = torch.clamp(input, -3.0, 3.0)
        sq = x * x
        return x * (sq + 27.0) / (27.0 + sq * 9.0)

    @staticmethod
    def dsigmoid(input: torch.Tensor) -> torch.Tensor:
        x = torch.clamp(input, -3.0, 3.0)
        sq = x * x
        return ((sq - 9) * (sq - 9)) / (9 * (3 + sq) * (3 + sq))

    @staticmethod
    def d2sigmoid(input: torch.Tensor) -> torch.Tensor:
        x = torch.clamp(input, -3.0, 3.0)
        sq = x * x
        den = sq + 3
        return 16 * x * (sq - 9) / (3 * den * den * den)

    @staticmethod
    def scalar_sigmoid(input: float) -> float:
        x = min(3.0, max(-3.0, input))
        sq = x * x
        return x * (sq + 27.0) / (27.0 + sq * 9.0)

    @staticmethod
    def scalar_dsigmoid(input: float) -> float:
        x = min(3.0, max(-3.0, input))
        sq = x * x
        return ((sq - 9) * (sq - 9)) / (9 * (3 + sq) * (3 + sq))

    @staticmethod
    def forward(ctx, weight, scale, ctrl):
        _require_cuda(weight, "SoftStep")
        ctx.ctrl = ctrl
        ctx.scale = scale
        ctx.save_for_backward(weight)
        return ops.fwd_softstep(weight.data, ctrl.digamma)

    @staticmethod
    def backward(ctx, grad_output):
        weight = ctx.saved_tensors[0]
        return ops.bwd_softstep(weight.data, ctx.ctrl.digamma, ctx.scale, grad_output), None, None


class FusedSoftLinear(Function):
    """x @ SoftStep(weight)^T + bias for bf16 activations with the staircase fused into the GEMM's weight-operand load
    (ops.qat_linear_forward); the two passes it replaces are SoftStep.apply + F.linear [tmq/tmq.py:637-659].  The
    backward pass recomputes the staircase with the elementwise kernels."""

    @staticmethod
    def forward(ctx, x, weight, bias, ctrl):
        ctx.ctrl = ctrl
        ctx.has_bias = bias is not None
        ctx.save_for_backward(x, weight)
        return ops.qat_linear_forward(x.data, weight.data, None if bias is None else bias.data, ctrl.digamma)

    @staticmethod
    def backward(ctx, grad_output):
        x, weight = ctx.saved_tensors
        d = ctx.ctrl.digamma
        g = grad_output.reshape(-1, grad_output.shape[-1]).float()
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            gx = (g @ ops.fwd_softstep(weight.data, d)).to(x.dtype).view(x.shape)
        if ctx.needs_input_grad[1]:
            gw = ops.bwd_softstep(weight.data, d, 1.0, g.t() @ x.reshape(-1, x.shape[-1]).float())
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = g.sum(0)
        return gx, gw, gb, None


class SoftStepDerivative(Function):
    """First derivative of the staircase, the integrand of the quantization loss [tmq/tmq.py:441-493]."""

    @staticmethod
    def forward(ctx, weight, digamma, strength):
        _require_cuda(weight, "SoftStepDerivative")
        ctx.save_for_backward(weight)
        ctx.digamma = digamma
        ctx.strength = strength
        return ops.fwd_softstep_derivative(weight.data, digamma, strength)

    @staticmethod
    def backward(ctx, grad_output):
        weight = ctx.saved_tensors[0]
        return ops.bwd_softstep_derivative(weight.data, ctx.digamma, ctx.strength, grad_output), None, None


class _LayerQuantLoss(Function):
    """mean(strength * S'(w; sharpness)) of ONE tensor without materialising the integrand."""

    @staticmethod
    def forward(ctx, weight, sharpness, strength):
        _require_cuda(weight, "quantization_loss")
        ctx.save_for_backward(weight)
        ctx.sharpness, ctx.strength = sharpness, strength
        return (ops.qloss_sum(weight.data, sharpness, strength) / weight.numel()).to(torch.float32)

    @staticmethod
    def backward(ctx, grad_output):
        weight = ctx.saved_tensors[0]
        g = (grad_output / weight.numel()).to(torch.float32).expand(weight.shape)
        return ops.bwd_softstep_derivative(weight.data, ctx.sharpness, ctx.strength, g), None, None


_VARIANCE = {QuantMode.TERNARY: 2.0 / 3.0, QuantMode.TWO_BIT: (2 * 2 * 2 + 2 + 1) / 6.0,
             QuantMode.THREE_BIT: (2 * 4 * 4 + 4 + 1) / 6.0, QuantMode.FOUR_BIT: (2 * 8 * 8 + 8 + 1) / 6.0,
             QuantMode.FIVE_BIT: (2 * 16 * 16 + 16 + 1) / 6.0, QuantMode.SIX_BIT: (2 * 32 * 32 + 32 + 1) / 6.0,
             QuantMode.EIGHT_BIT: (2 * 128 * 128 + 128 + 1) / 6.0}


def _pair(v):
    return tuple(v) if isinstance(v, (tuple, list)) else (v, v)


class TMQLayer:
    """Shared state and behaviour of the quantization-aware layers [tmq/tmq.py:496-570]."""

    def __init__(self, ctrl=None, quant_mode=QuantMode.NONE, tensor_type=TensorType.FLOAT_32BIT, device=None):
        self._ctrl = ctrl
        self.quantization = quant_mode
        self.tensor_type = tensor_type
        self._device = device
        self.compact = False
        self.original_shape = None
        self.post_scale_imm = 1.0
        self.post_scale = None
        self.layer_name = None
        self._scale_dirty = True
        self._prepacked = {}

    def compact_inference_mode(self):
        self.training = False
        self.compact = True

    def quantization_loss(self, strength, sharpness):
        return _LayerQuantLoss.apply(self.weight, float(sharpness), float(strength))

    def quantize(self):
        self.weight.data = torch.round(self.weight.data).float()

    @torch.no_grad()
    def clamp(self, limits=(-1., 1.)):
        _require_cuda(self.weight, "clamp")
        ops.clamp(self.weight.data, limits[0], limits[1], out=self.weight.data)

    def _update_scale(self):
        if self._scale_dirty and self.post_scale is not None:
            self.post_scale_imm = self.post_scale.item()
            self._scale_dirty = False

    def _variance_estimate(self) -> float:
        return _VARIANCE.get(self.quantization, 1.0)

    def _soft_weight(self):
        """Weights as the forward pass sees them: through the staircase while training with a controller."""
        assert self._ctrl or not self.training, "Quantization controller required for training"
        self._update_scale()
        if self._ctrl is not None and not self._ctrl.inference_mode:
            return SoftStep.apply(self.weight, 1.0, self._ctrl)
        return self.weight

    # ---- compact inference helpers -------------------------------------------------------------------------------------

    def _cached_layout(self, key, build):
        """Kernel-side layout of the packed weights under `key`, built by build() on first use and whenever the packed
        tensor changes."""
        # identity of the packed tensor: the Parameter object (kept alive by the cache entry, so its id cannot be
        # recycled), its in-place version counter (copy_ / load_state_dict bump it; `.data` would always read 0), and
        # the storage it points at (module.to(...) rebinds .data under the same Parameter)
        p = self.weight
        tag = (id(p), p._version, p.data_ptr(), tuple(p.shape), str(p.device))
        hit = self._prepacked.get(key)
        if hit is not None and hit[0][0] != tag[0]:
            self._prepacked.clear()               # a different Parameter was bound: every cached layout is stale
            hit = None
        if hit is None or hit[0] != tag:
            hit = (tag, build(), p)
            self._prepacked[key] = hit
        return hit[1]

    def _prepacked_weights(self, fmt, k_repeat=1, k_each=None):
        """GEMM layout of the layer's packed matrix.  k_repeat = 3 stacks three copies along K (each zero-padded to
        k_each rows) for the exact fp32 path."""
        def build():
            packed = self._packed_matrix()
            if k_each is not None and k_each > packed.shape[0]:
                packed = torch.nn.functional.pad(packed, (0, 0, 0, k_each - packed.shape[0]))
            if k_repeat > 1:
                packed = torch.cat([packed] * k_repeat, dim=0)
            return ops.prepack(packed, self._gemm_columns(), fmt)
        return self._cached_layout((fmt, k_repeat, k_each), build)

    def _gemm_columns(self):
        """Output width N of the layer's GEMM."""
        return int(self.original_shape[0])

    def _packed_matrix(self):
        """The layer's weights as the 2-D reference-layout packed matrix int32 [K, ceil(N/16)] of its GEMM."""
        w = self.weight.data
        return w.contiguous().view(-1, w.shape[-1])

    def _compact_matmul(self, x2d, fuse=True):
        """[M, K] activations x packed weights -> [M, N] with post_scale and bias fused into the epilogue (fuse=False:
        the bare product).  fp32 in -> fp32 out (exact split), bf16 in -> bf16 out, int8 in -> int32 out (no scale /
        bias)."""
        n_out = self._gemm_columns()
        k = x2d.shape[1]
        scale = None
        if fuse and self.post_scale_imm != 1.0:
            scale = torch.full((n_out,), float(self.post_scale_imm), dtype=torch.float32, device=x2d.device)
        bias = getattr(self, "bias", None) if fuse else None
        if x2d.dtype == torch.int8:
            pad = (-k) % 16
            if pad:
                x2d = torch.nn.functional.pad(x2d, (0, pad))
            wt = self._prepacked_weights(ops.FMT_I8)
            if wt.shape[1] != ops.prepack_row_words(x2d.shape[1], ops.FMT_I8):
                raise RuntimeError("compact inference: activation width does not match the packed weights")
            return ops.ternary_gemm_i8(x2d, wt, n_out)
        if x2d.dtype == torch.bfloat16:
            pad = (-k) % 8
            if pad:
                x2d = torch.nn.functional.pad(x2d, (0, pad))
            return ops.ternary_gemm(x2d, self._prepacked_weights(ops.FMT_BF16), n_out, scale, bias,
                                    out_dtype=torch.bfloat16)
        if x2d.dtype != torch.float32:
            raise RuntimeError("compact inference: activations must be float32, bfloat16 or int8")
        # fp32 activations: x = hi + mid + lo with three bf16 terms is exact, so is every product with {-1,0,1};
        # the three terms ride along K against three stacked copies of the weights, accumulation is fp32
        kp = (k + 7) // 8 * 8
        x3 = ops.split_f32(x2d, 3, kp)                      # one kernel: [M, 3 * kp] bf16
        return ops.ternary_gemm(x3, self._prepacked_weights(ops.FMT_BF16, k_repeat=3, k_each=kp), n_out,
                                scale, bias, out_dtype=torch.float32)

    def _load_compact_metadata(self, state_dict, prefix, local_metadata):
        """Second half of `_load_from_state_dict`: interpret the tmq.* metadata [tmq/tmq.py:748-765, :956-973]."""
        if "tmq.quant" in local_metadata and "tmq.tensor_type" in local_metadata:
            self.tensor_type = TensorType(local_metadata["tmq.tensor_type"])
            self.original_shape = local_metadata["tmq.shape"]
            stored = state_dict[prefix + "weight"]
            if self.tensor_type == TensorType.COMPRESSED_TERNARY_32BIT:
                self.weight = nn.Parameter(decompress_ternary(stored, self.original_shape), requires_grad=False)
                self.tensor_type = TensorType.COMPACT_TERNARY_32BIT
                self.compact = True
            elif self.tensor_type == TensorType.COMPACT_TERNARY_32BIT:
                self.weight = nn.Parameter(stored, requires_grad=False)
                self.compact = True
            else:
                self.compact = False
            self.quantization = QuantMode(local_metadata["tmq.quant"])
            self.training = False if self.compact else self.training
        else:
            self.compact = False


class Linear(nn.Module, TMQLayer):
    """Quantization-aware drop-in for nn.Linear [tmq/tmq.py:573-765]."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None,
                 ctrl: QuantizationControl = None, quant_mode=QuantMode.NONE, post_scale=False):
        super(Linear, self).__init__()
        TMQLayer.__init__(self, ctrl, quant_mode, TensorType.FLOAT_32BIT, device)
        self.weight = nn.Parameter()
        self._in_features = in_features
        self._out_features = out_features
        self._init_weights(bias, device)
        self.original_shape = self.weight.shape
        self.post_scale_imm = 1.0 / (self._in_features * self._variance_estimate()) if post_scale else 1.0
        self.post_scale = nn.Parameter(torch.tensor(self.post_scale_imm), requires_grad=False)
        self.bn = None

    def __repr__(self):
        if len(self.original_shape) == 2:
            return "Linear(%d,%d) [tmq]" % tuple(self.original_shape) + " <%s>" % self.layer_name
        return "Linear(???) [tmq] <%s>" % self.layer_name

    def disable_bias(self):
        self.bias = None

    def implicit_bn(self):
        self.bn = nn.BatchNorm1d(self._out_features)

    def forward(self, x):
        if self.compact:
            return self.compact_forward(x)
        if (x.dtype == torch.bfloat16 and x.is_cuda and self._ctrl is not None and not self._ctrl.inference_mode
                and x.shape[-1] % 8 == 0):
            # bf16 activations (not a reference configuration: its fp32 weights would refuse them): one fused kernel
            self._update_scale()
            out = FusedSoftLinear.apply(x, self.weight, None if self.post_scale_imm != 1.0 else self.bias, self._ctrl)
            if self.post_scale_imm != 1.0:
                out = self.post_scale * out
                if self.bias is not None:
                    out = self.bias + out
            return self.bn(out) if self.bn is not None else out
        w = self._soft_weight()
        if self.post_scale_imm != 1.0:
            out = self.post_scale * torch.nn.functional.linear(x, w, None)
            if self.bias is not None:
                out = self.bias + out
        else:
            out = torch.nn.functional.linear(x, w, self.bias)
        return self.bn(out) if self.bn is not None else out

    forward_wrap = forward

    @torch.no_grad()
    def compact_forward(self, x):
        """Inference from the packed weights, any leading dimensions [tmq/tmq.py:662-688 handles one row only]."""
        assert self.training == False, "Compact inference is not supported in training mode"
        assert self.weight.data.dtype == torch.int32, "Compact inference requires 32-bit integer words"
        _require_cuda(x, "compact_forward")
        self._update_scale()
        lead = x.shape[:-1]
        out = self._compact_matmul(x.reshape(-1, x.shape[-1]))
        out = out.view(*lead, out.shape[-1])
        return self.bn(out) if self.bn is not None else out

    @classmethod
    def from_linear(cls, source: nn.Linear, name: str, ctrl: QuantizationControl):
        assert ctrl, "Control instance is required"
        obj = cls(source.in_features, source.out_features, source.bias is not None, ctrl=ctrl,
                  device=source.weight.device, quant_mode=ctrl.quantization, post_scale=ctrl.post_scale)
        obj.layer_name = name
        ctrl.register_node(name, obj)
        return obj

    @torch.no_grad()
    def _init_weights(self, bias, device):
        # weights start uniform in [-1, 1), bias at zero; whatever the source layer held is discarded
        self.bias = nn.Parameter(torch.zeros(self._out_features).to(device), requires_grad=True) if bias else None
        w = 2.0 * (torch.rand(self._out_features, self._in_features) - 0.5)
        self.weight = nn.Parameter(w.to(device), requires_grad=True)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                              error_msgs):
        super(Linear, self)._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys,
                                                  unexpected_keys, error_msgs)
        self._load_compact_metadata(state_dict, prefix, local_metadata)


class Conv2d(nn.Module, TMQLayer):
    """Quantization-aware drop-in for nn.Conv2d [tmq/tmq.py:769-973]."""

    def __init__(self, in_channels, out_channels, kernel, stride=1, padding=0, groups=1, dilation=1, bias=True,
                 device=None, ctrl=None, quant_mode=QuantMode.NONE, post_scale=False):
        super(Conv2d, self).__init__()
        TMQLayer.__init__(self, ctrl, quant_mode, TensorType.FLOAT_32BIT, device)
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel = kernel
        self.stride = stride
        self.padding = padding
        self.groups = groups
        self.dilation = dilation
        self._init_weights(bias, device)
        self.original_shape = self.weight.shape
        self.post_scale_imm = 1.0 / (self._fan_in * self._variance_estimate()) if post_scale else 1.0
        self.post_scale = nn.Parameter(torch.tensor(self.post_scale_imm), requires_grad=False)

    def __repr__(self):
        return "Conv2d(%d,%d,%d,%d) [tmq]" % tuple(self.original_shape) + " <%s>" % self.layer_name

    def to(self, *args, **kwargs):
        me = super().to(*args, **kwargs)
        me.post_scale_imm = me.post_scale.item()
        return me

    def _conv(self, x, w, bias):
        return torch.nn.functional.conv2d(x, w, bias, self.stride, self.padding, dilation=self.dilation,
                                          groups=self.groups)

    def forward(self, x):
        if self.compact:
            return self.compact_forward(x)
        w = self._soft_weight()
        if self.post_scale_imm != 1.0:
            out = self.post_scale * self._conv(x, w, None)
            return self.bias + out if self.bias is not None else out
        return self._conv(x, w, self.bias)

    @torch.no_grad()
    def compact_forward(self, x):
        """Convolution from packed weights with the output geometry of F.conv2d.  Channel counts that are a multiple of
        64 run as an implicit GEMM (bf16, int8 or - exactly - fp32 activations); few-channel layers with bf16
        activations run the fused stem kernel; depthwise layers their own kernel; the rest falls back to explicit
        patches.  Reference path: unfold + CUDA-core GEMM + fold [tmq/tmq.py:822-871]."""
        assert not self.training, "Compact inference is not supported in training mode"
        assert self.weight.data.dtype == torch.int32, "Compact inference requires 32-bit integer words"
        _require_cuda(x, "compact_forward")
        self._update_scale()
        if x.dim() == 3:
            return self.compact_forward(x.unsqueeze(0)).squeeze(0)
        if x.dim() != 4:
            raise Exception("Expected a 3D tensor")
        b, c, h, w = x.shape
        (ky, kx), (sy, sx) = _pair(self.kernel), _pair(self.stride)
        (py, px), (dy, dx) = _pair(self.padding), _pair(self.dilation)
        if self.groups != 1:
            # depthwise: straight from the image, no unfold / fold [tmq/tmq.py:849-854]
            assert self.groups == self.original_shape[0] == c, \
                "Grouped convolutions are only supported for group == channels"
            if x.dtype != torch.float32:
                raise RuntimeError("compact inference of depthwise convolutions takes float32 activations")
            scale = None
            if self.post_scale_imm != 1.0:
                scale = torch.full((c,), float(self.post_scale_imm), dtype=torch.float32, device=x.device)
            return ops.ternary_dwconv2d(x, self.weight.data, (ky, kx), (sy, sx), (py, px), (dy, dx), scale, self.bias)
        if c != int(self.original_shape[1]):
            raise RuntimeError("compact inference: channel count does not match the packed weights")
        if c % 64 == 0 and x.dtype in (torch.bfloat16, torch.float32, torch.int8):
            return self._implicit_forward(x, (ky, kx), (sy, sx), (py, px), (dy, dx))
        if x.dtype == torch.bfloat16 and (dy, dx) == (1, 1):
            y = self._few_channel_forward(x, (ky, kx), (sy, sx), (py, px))
            if y is not None:
                return y
        return self._patch_forward(x, (ky, kx), (sy, sx), (py, px), (dy, dx))

    def _epilogue_scale(self, n_out, device):
        if self.post_scale_imm == 1.0:
            return None
        return torch.full((n_out,), float(self.post_scale_imm), dtype=torch.float32, device=device)

    def _implicit_forward(self, x, kernel, stride, padding, dilation):
        """Implicit GEMM on the tensor cores, no patch matrix.  The result is NHWC in memory and returned as the NCHW
        view of it (torch's channels_last), which the next compact layer takes without a copy.
        bf16 -> bf16; int8 -> exact int32 sums (no scale / bias); fp32 -> fp32 through the exact three-term split of
        the activations along the channels (three stacked copies of the weights per filter tap)."""
        b, c, h, w = x.shape
        n_out = int(self.original_shape[0])
        (ky, kx) = kernel
        terms = 3 if x.dtype == torch.float32 else 1
        fmt = ops.FMT_I8 if x.dtype == torch.int8 else ops.FMT_BF16
        nhwc = x.permute(0, 2, 3, 1)
        if x.dtype == torch.float32:
            if nhwc.is_contiguous():                       # channels_last fp32: split the pixel rows in place
                xin = ops.split_f32(nhwc.reshape(b * h * w, c), 3, c).view(b, h, w, 3 * c)
            else:
                xin = ops.nchw_to_nhwc_bf16(x, 3)
        else:
            xin = nhwc if nhwc.is_contiguous() else nhwc.contiguous()
        if x.dtype == torch.bfloat16 and stride == (1, 1) and ky * kx <= 9:
            wt1 = self._cached_layout(("conv_s1",), lambda: ops.prepack(
                ops.conv_rows_skkc(self.weight.data, c, ky, kx), n_out, ops.FMT_BF16))
            y = ops.ternary_conv2d_s1(xin, wt1, n_out, kernel, padding, dilation, self._epilogue_scale(n_out, x.device),
                                      self.bias)
            if y is not None:
                return y.permute(0, 3, 1, 2)
        wt = self._cached_layout(("conv", fmt, terms), lambda: ops.prepack(
            ops.conv_rows_kkc(self.weight.data, c, ky, kx, terms, pad_to=1), n_out, fmt))
        if x.dtype == torch.int8:
            y = ops.ternary_conv2d_nhwc(xin, wt, n_out, kernel, stride, padding, dilation)
        else:
            y = ops.ternary_conv2d_nhwc(xin, wt, n_out, kernel, stride, padding, dilation,
                                        self._epilogue_scale(n_out, x.device), self.bias,
                                        out_dtype=torch.float32 if terms == 3 else torch.bfloat16)
        return y.permute(0, 3, 1, 2)

    def _few_channel_forward(self, x, kernel, stride, padding):
        """Layers with few input channels (an image stem) and bf16 activations: the fused kernel that keeps the patches
        on chip.  None when the geometry is outside that kernel's limits."""
        b, c, h, w = x.shape
        n_out = int(self.original_shape[0])
        (ky, kx) = kernel
        def rows_layout():
            rows = ops.conv_rows_stem(self.weight.data, c, ky, kx, stride[1])
            return None if rows is None else ops.prepack(rows, n_out, ops.FMT_BF16)
        wt_rows = self._cached_layout(("stem_rows",), rows_layout)
        if wt_rows is not None:
            y = ops.ternary_conv2d_stem_rows(x.float(), wt_rows, n_out, kernel, stride, padding,
                                             self._epilogue_scale(n_out, x.device), self.bias)
            if y is not None:
                return y.permute(0, 3, 1, 2)
        wt = self._cached_layout(("stem",), lambda: ops.prepack(
            ops.conv_rows_kkc(self.weight.data, c, ky, kx, 1, pad_to=8), n_out, ops.FMT_BF16))
        y = ops.ternary_conv2d_stem(x.float(), wt, n_out, kernel, stride, padding,
                                    self._epilogue_scale(n_out, x.device), self.bias)
        return None if y is None else y.permute(0, 3, 1, 2)

    def _patch_forward(self, x, kernel, stride, padding, dilation):
        """Fallback for what the kernels above do not take (channel counts that are no multiple of 64 with fp32 or int8
        activations, dilated few-channel layers): explicit patches (torch's unfold) through the ternary GEMM, exact for
        fp32 [the reference's only route, tmq/tmq.py:857-863]."""
        b, c, h, w = x.shape
        (ky, kx), (sy, sx), (py, px), (dy, dx) = kernel, stride, padding, dilation
        h_out = (h + 2 * py - dy * (ky - 1) - 1) // sy + 1
        w_out = (w + 2 * px - dx * (kx - 1) - 1) // sx + 1
        if ky == 1 and kx == 1 and py == 0 and px == 0:
            cols = x[:, :, ::sy, ::sx].permute(0, 2, 3, 1).reshape(b * h_out * w_out, c)
        else:
            cols = torch.nn.functional.unfold(x, kernel_size=(ky, kx), dilation=(dy, dx), stride=(sy, sx),
                                              padding=(py, px))            # [B, C*ky*kx, L], (c, ky, kx) order
            cols = cols.transpose(1, 2).reshape(b * h_out * w_out, c * ky * kx)
        k = cols.shape[1]
        align = 16 if cols.dtype == torch.int8 else 8
        if k % align:
            cols = torch.nn.functional.pad(cols, (0, align - k % align))
        out = self._compact_matmul(cols.contiguous())
        return out.view(b, h_out, w_out, -1).permute(0, 3, 1, 2)

    @classmethod
    def from_conv2d(cls, source: nn.Conv2d, name: str, ctrl: QuantizationControl):
        assert ctrl, "Controller required"
        obj = cls(source.in_channels, source.out_channels, source.kernel_size, stride=source.stride,
                  padding=source.padding, groups=source.groups, dilation=source.dilation,
                  bias=source.bias is not None, device=source.weight.device, ctrl=ctrl,
                  quant_mode=ctrl.quantization, post_scale=ctrl.post_scale)
        obj.layer_name = name
        ctrl.register_node(name, obj)
        return obj

    def _weight_shape(self):
        ky, kx = _pair(self.kernel)
        return [self.out_channels, self.in_channels // self.groups, ky, kx]

    @torch.no_grad()
    def _init_weights(self, bias, device):
        ky, kx = _pair(self.kernel)
        self._fan_in = ky * kx * self.in_channels
        self._fan_out = ky * kx * self.out_channels
        w = 2.0 * (torch.rand(self._weight_shape()) - 0.5)
        self.weight = nn.Parameter(w.to(device), requires_grad=True)
        self.bias = nn.Parameter(torch.zeros(self.out_channels).to(device), requires_grad=True) if bias else None

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                              error_msgs):
        super(Conv2d, self)._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys,
                                                  unexpected_keys, error_msgs)
        self._load_compact_metadata(state_dict, prefix, local_metadata)


class ConvTranspose2d(Conv2d):
    """Quantization-aware drop-in for nn.ConvTranspose2d (training path) [tmq/tmq.py:978-1087]."""

    def __init__(self, in_channels, out_channels, kernel, stride=1, padding=0, output_padding=0, groups=1, bias=True,
                 dilation=1, device=None, ctrl=None, quant_mode=QuantMode.NONE, post_scale=False):
        super(ConvTranspose2d, self).__init__(in_channels, out_channels, kernel, stride, padding, groups, dilation,
                                              bias, device, ctrl, quant_mode, post_scale)
        self.output_padding = output_padding

    def __repr__(self):
        return "ConvTranspose2d(%d,%d,%d,%d) [tmq] " % tuple(self.original_shape) + " <%s>" % self.layer_name

    def _weight_shape(self):
        ky, kx = _pair(self.kernel)
        return [self.in_channels, self.out_channels // self.groups, ky, kx]

    def _conv(self, x, w, bias):
        return torch.nn.functional.conv_transpose2d(x, w, bias, self.stride, self.padding, dilation=self.dilation,
                                                    groups=self.groups)

    def _gemm_columns(self):
        ky, kx = _pair(self.kernel)
        return int(self.original_shape[1]) * ky * kx

    def _packed_matrix(self):
        """groups == 1: out[pixel][(o, ky, kx)] = sum_i x[pixel][i] * w[i][o][ky][kx], so the GEMM's weight matrix is
        [N = (o, ky, kx)][K = i]; the stored packed tensor [o, ky, kx, ceil(i/16)] is re-packed along N once."""
        w4 = ops.expand_ternary(self.weight.data, list(self.original_shape))          # fp32 [i, o, ky, kx]
        return ops.compactify_ternary(w4.reshape(w4.shape[0], -1).t().contiguous())    # [K = i, ceil(N/16)]

    @torch.no_grad()
    def compact_forward(self, x):
        """Transposed convolution from packed weights with torch conv_transpose2d's output geometry.  Depthwise
        (groups == channels): one gather kernel straight from the image.  groups == 1: tensor-core GEMM to columns,
        then F.fold [tmq/tmq.py:1007-1042; the reference passes mismatched operands to its GEMM there]."""
        assert not self.training, "Compact inference is not supported in training mode"
        assert self.weight.data.dtype == torch.int32, "Compact inference requires 32-bit integer words"
        _require_cuda(x, "compact_forward")
        self._update_scale()
        if x.dim() == 3:
            return self.compact_forward(x.unsqueeze(0)).squeeze(0)
        if x.dim() != 4:
            raise Exception("Expected a 3D tensor")
        if x.dtype != torch.float32:
            raise RuntimeError("compact inference of transposed convolutions takes float32 activations")
        b, c, h, w = x.shape
        (ky, kx), (sy, sx) = _pair(self.kernel), _pair(self.stride)
        (py, px), (dy, dx) = _pair(self.padding), _pair(self.dilation)
        opy, opx = _pair(self.output_padding)
        assert self.groups == 1 or self.groups == self.in_channels, \
            "Grouped transpose convolutions are only supported for channels == groupsize"
        n_out = int(self.original_shape[1]) * self.groups
        scale = None
        if self.post_scale_imm != 1.0:
            scale = torch.full((n_out,), float(self.post_scale_imm), dtype=torch.float32, device=x.device)
        if self.groups != 1:
            assert int(self.original_shape[1]) == 1, "depthwise transposed convolutions keep the channel count"
            return ops.ternary_dwconvtrans2d(x, self.weight.data, (ky, kx), (sy, sx), (py, px), (dy, dx), (opy, opx),
                                             scale, self.bias)
        h_out = (h - 1) * sy - 2 * py + dy * (ky - 1) + 1 + opy
        w_out = (w - 1) * sx - 2 * px + dx * (kx - 1) + 1 + opx
        cols = self._compact_matmul(x.permute(0, 2, 3, 1).reshape(b * h * w, c), fuse=False)    # [B*H*W, O*ky*kx]
        final = torch.nn.functional.fold(cols.view(b, h * w, -1).transpose(1, 2), output_size=(h_out, w_out),
                                         kernel_size=(ky, kx), dilation=(dy, dx), stride=(sy, sx), padding=(py, px))
        if scale is not None:
            final = final * self.post_scale_imm
        if self.bias is not None:
            final = self.bias.view(1, -1, 1, 1) + final
        return final

    @classmethod
    def from_transconv2d(cls, source: nn.ConvTranspose2d, name: str, ctrl: QuantizationControl):
        assert ctrl, "Controller required"
        obj = cls(source.in_channels, source.out_channels, source.kernel_size, stride=source.stride,
                  padding=source.padding, output_padding=source.output_padding, groups=source.groups,
                  dilation=source.dilation, bias=source.bias is not None, device=ctrl.device, ctrl=ctrl,
                  quant_mode=ctrl.quantization, post_scale=ctrl.post_scale)
        obj.layer_name = name
        ctrl.register_node(name, obj)
        return obj


# ---- model-level helpers ----------------------------------------------------------------------------------------------

def _tmq_layers(module, prefix=""):
    """(dotted name, parent, attribute name, layer) for every TMQ layer; does not descend into TMQ layers."""
    for name, sub in module.named_children():
        full = prefix + "." + name if prefix != "" else name
        if isinstance(sub, TMQLayer):
            yield full, module, name, sub
        else:
            yield from _tmq_layers(sub, full)


def quantize_weights(module: nn.Module):
    """Round the fp32 weights of every TMQ layer to integers, in place [tmq/tmq.py:1090-1111]."""
    for _, sub in module.named_modules():
        if isinstance(sub, TMQLayer):
            if sub.weight.data.dtype == torch.float16:
                raise Exception("FP16 data is currently not supported")
            if sub.weight.data.dtype == torch.float32:
                sub.weight = nn.Parameter(torch.round(sub.weight.data), requires_grad=sub.weight.requires_grad)


def quantize_model(module: nn.Module, ctrl: QuantizationControl, prefix="", exclude=[]):
    """Swap nn.Linear / nn.Conv2d / nn.ConvTranspose2d children for their quantization-aware versions, in place.
    `exclude` holds dotted names and `*` wildcards; weights are re-initialised [tmq/tmq.py:1114-1180]."""
    assert ctrl, "Must supply a quantization control instance"
    exact = [e for e in exclude if "*" not in e]
    globs = [e for e in exclude if "*" in e]
    _swap_children(module, ctrl, prefix, exact, globs)


def _swap_children(module, ctrl, prefix, exact, globs):
    for name, sub in module.named_children():
        if sub is module:
            continue
        dotted = prefix + "." + name if prefix != "" else name
        if dotted in exact:
            print("Skipping excluded layer %s" % dotted)
            continue
        if any(fnmatch.fnmatch(dotted, g) for g in globs):
            print("Skipping excluded layer %s" % dotted)
        else:
            registry_name = prefix + "." + name        # top-level layers keep the leading dot of the reference
            if isinstance(sub, nn.Linear):
                setattr(module, name, Linear.from_linear(sub, registry_name, ctrl))
            elif isinstance(sub, nn.ConvTranspose2d):
                setattr(module, name, ConvTranspose2d.from_transconv2d(sub, registry_name, ctrl))
            elif isinstance(sub, nn.Conv2d):
                setattr(module, name, Conv2d.from_conv2d(sub, registry_name, ctrl))
        _swap_children(sub, ctrl, dotted, exact, globs)


def compressed_state_dict(module: nn.Module, strong=False, remove_prefix=""):
    """State dict with the TMQ layers' weights bit-stuffed (int32, 16 per word) or, with `strong`, range coded
    (int8 stream); the model itself is switched to compact inference [tmq/tmq.py:1183-1248]."""
    layers = list(_tmq_layers(module))
    for _, _, _, layer in layers:
        if not hasattr(layer, "tensor_type"):
            continue
        if getattr(layer, "original_shape", None) is None:
            layer.original_shape = layer.weight.shape
        if not strong and layer.tensor_type != TensorType.COMPACT_TERNARY_32BIT:
            layer.weight = nn.Parameter(compactify_ternary(layer.weight.data), requires_grad=False)
            layer.tensor_type = TensorType.COMPACT_TERNARY_32BIT
        elif strong and layer.tensor_type != TensorType.COMPRESSED_TERNARY_32BIT:
            already_packed = layer.tensor_type == TensorType.COMPACT_TERNARY_32BIT
            stream = compress_ternary(layer.weight.data, layer.original_shape, already_packed)
            layer._stream_device = layer.weight.device
            layer.weight = nn.Parameter(stream, requires_grad=False)
            layer.tensor_type = TensorType.COMPRESSED_TERNARY_32BIT
    state = module.state_dict()
    for full, _, _, layer in layers:
        layer.compact_inference_mode()
        meta = state._metadata[full]
        meta["tmq.tensor_type"] = layer.tensor_type.value
        meta["tmq.shape"] = layer.original_shape
        meta["tmq.quant"] = layer.quantization.value
        if layer.tensor_type == TensorType.COMPRESSED_TERNARY_32BIT:
            # keep the live model usable: back to the packed form (on the device the layer lived on)
            packed = decompress_ternary(layer.weight.data, layer.original_shape)
            layer.weight = nn.Parameter(packed.to(getattr(layer, "_stream_device", packed.device)), requires_grad=False)
            layer.tensor_type = TensorType.COMPACT_TERNARY_32BIT
    return state


def prepare_compressed_load(module: nn.Module, state_dict):
    _size_weights_for_load(module, state_dict)


def load_compressed_state_dict(module: nn.Module, state_dict):
    """Load a dict produced by compressed_state_dict; range-coded weights are decoded to the packed form."""
    _size_weights_for_load(module, state_dict)
    module.load_state_dict(state_dict, strict=False)


def _size_weights_for_load(module, state_dict):
    meta = state_dict._metadata
    for full, _, _, layer in _tmq_layers(module):
        layer.layer_name = full
        if full not in meta:
            continue
        kind = TensorType(meta[full]["tmq.tensor_type"])
        if kind in (TensorType.COMPACT_TERNARY_32BIT, TensorType.COMPRESSED_TERNARY_32BIT):
            stored = state_dict[full + ".weight"]
            layer.weight = nn.Parameter(torch.empty(stored.shape, dtype=stored.dtype), requires_grad=False)
        else:
            layer.compact = False


def expand_compact_layers(module: nn.Module, for_training=False):
    """Turn packed / range-coded TMQ layers back into fp32 {-1, 0, +1} weights, in place [tmq/tmq.py:1296-1319]."""
    for _, sub in module.named_modules():
        if not (isinstance(sub, TMQLayer) and hasattr(sub, "tensor_type") and hasattr(sub, "original_shape")):
            continue
        if sub.tensor_type in (TensorType.COMPRESSED_TERNARY_32BIT, TensorType.COMPACT_TERNARY_32BIT):
            coded = sub.tensor_type == TensorType.COMPRESSED_TERNARY_32BIT
            full = expand_ternary(sub.weight.data, sub.original_shape, coded)
            sub.weight = nn.Parameter(full, requires_grad=for_training)
            sub.tensor_type = TensorType.FLOAT_32BIT
            sub.compact = False
