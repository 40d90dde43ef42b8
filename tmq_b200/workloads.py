"""The ResNet-18 workloads of the baseline configuration, built from the public API only.

  * `build_resnet18(num_classes)`         torchvision ResNet-18 with every conv / fc layer swapped for its TMQ layer,
                                          fc without bias but with its own BatchNorm (the reference's sample set-up,
                                          samples/resnet_train.py:344-358)
  * `qat_step(...)`                       one QAT step: forward, cross-entropy + quantization loss, backward,
                                          (all-reduce), optimizer, clamp (samples/resnet_train.py:102-160)
  * `PackedResNet18`                      inference from packed weights: BatchNorm folded into per-channel scale/bias of
                                          the conv epilogue, bf16 NHWC activations, convolutions as implicit GEMMs
"""
import torch
from torch import nn

from . import dist as tdist
from . import ops
from . import tmq as api


class TrainMaxPool(nn.Module):
    """nn.MaxPool2d(kernel, stride, padding) whose forward / backward run the library's streaming kernels on fp32
    channels-last CUDA activations (torch's own otherwise)."""

    def __init__(self, kernel_size, stride, padding):
        super().__init__()
        self.kernel_size, self.stride, self.padding = kernel_size, stride, padding

    def forward(self, x):
        return ops.maxpool2d_train(x, self.kernel_size, self.stride, self.padding)


def build_resnet18(num_classes=101, ctrl=None, max_epochs=50, qpenalty_range=(0.0, 1e-3)):
    import torchvision
    model = torchvision.models.resnet18(num_classes=num_classes)
    if ctrl is None:
        ctrl = api.QuantizationControl(epoch_knots=api.QuantizationScheduleBuilder.default_schedule(max_epochs),
                                       qpenalty_range=qpenalty_range)
    api.quantize_model(model, ctrl)
    model.maxpool = TrainMaxPool(3, 2, 1)        # same layer, faster kernels when the activations are channels-last
    model.fc.disable_bias()
    model.fc.implicit_bn()
    return model, ctrl


def fused_optimizer(model, ctrl, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, bucket=None):
    """ops.MultiTensorAdam over the model's parameters with the QAT clamp fused in for every registered TMQ layer."""
    lo, hi = ctrl.clamp_values
    return ops.MultiTensorAdam(model.parameters(), lr=lr, betas=betas, eps=eps, bucket=bucket,
                               clamp_params=[node.weight for node in ctrl._registry.values()], clamp=(lo, hi))


def qat_step(model, ctrl, optimizer, x, y, bucket=None):
    """One training step on this rank's slice of the batch.  With a FlatGradBucket the gradients are averaged over
    the ranks with a single all-reduce before the optimizer runs.  `optimizer` may be an ops.MultiTensorAdam (see
    fused_optimizer): it then also performs the clamp.  Returns (loss, cross-entropy, quantization loss)."""
    fused = isinstance(optimizer, ops.MultiTensorAdam)
    if bucket is not None:
        bucket.zero()
    elif fused:
        optimizer.zero_grad()
    else:
        optimizer.zero_grad(set_to_none=True)
    if x.dim() == 4 and x.is_cuda:
        # channels-last activations: cuDNN's tensor-core convolutions then run without layout conversions around every
        # layer (ResNet-18, batch 256: 40.6 -> 19.6 ms per step, same arithmetic, loss equal to 3e-4 relative); the
        # weights stay contiguous, which the multi-tensor soft-step / clamp / loss kernels require
        x = x.contiguous(memory_format=torch.channels_last)
    logits = model(x)
    ce = nn.functional.cross_entropy(logits, y)
    ql = ctrl.quantization_loss()
    loss = ce + ql if ql is not None else ce
    loss.backward()
    if bucket is not None:
        bucket.allreduce_mean()
    optimizer.step()
    if not fused:
        ctrl.clamp()
    return loss.detach(), ce.detach(), (ql.detach() if ql is not None else None)


# ---- packed inference ----------------------------------------------------------------------------------------------------

def _fold_bn(bn, conv_bias=None, post_scale=1.0):
    """BatchNorm (eval) after a bias-free linear map -> per-channel (scale, bias) of that map's epilogue."""
    inv = torch.rsqrt(bn.running_var.float() + bn.eps)
    gamma = bn.weight.float() if bn.weight is not None else torch.ones_like(inv)
    beta = bn.bias.float() if bn.bias is not None else torch.zeros_like(inv)
    scale = gamma * inv * post_scale
    bias = beta - bn.running_mean.float() * gamma * inv
    if conv_bias is not None:
        bias = bias + conv_bias.float() * gamma * inv
    return scale.contiguous(), bias.contiguous()


class PackedConv:
    """A ternary convolution with folded BatchNorm, run from packed weights on bf16 NHWC activations."""

    def __init__(self, layer, bn, relu):
        assert layer.weight.dtype == torch.int32, "layer must be in compact form (compressed_state_dict)"
        self.cout, self.cin, self.ky, self.kx = [int(v) for v in layer.original_shape]
        self.stride, self.padding = api._pair(layer.stride), api._pair(layer.padding)
        self.dilation = api._pair(layer.dilation)
        self.relu = relu
        self.layer = layer
        self.scale, self.bias = _fold_bn(bn, getattr(layer, "bias", None), float(layer.post_scale_imm))
        # the implicit GEMM walks K as (ky, kx, c): channel runs are contiguous in NHWC
        self.K = self.cin * self.ky * self.kx
        self.implicit = (self.cin % 64 == 0)
        self.wt = ops.prepack(ops.conv_rows_kkc(layer.weight.data, self.cin, self.ky, self.kx, 1, pad_to=8), self.cout,
                              ops.FMT_BF16)
        # few-channel layers: the K order of the descriptor-patch stem kernel, where it covers the layer
        self.wt_rows = None
        if not self.implicit and self.dilation == (1, 1):
            rows = ops.conv_rows_stem(layer.weight.data, self.cin, self.ky, self.kx, self.stride[1])
            if rows is not None:
                self.wt_rows = ops.prepack(rows, self.cout, ops.FMT_BF16)
        # unit-stride layers also get the slice-major layout of the shifted-window kernel
        self.wt_s1 = None
        if self.implicit and self.stride == (1, 1) and self.ky * self.kx <= 9:
            self.wt_s1 = ops.prepack(ops.conv_rows_skkc(layer.weight.data, self.cin, self.ky, self.kx), self.cout,
                                     ops.FMT_BF16)

    def from_images_pooled(self, images):
        """Stem + ReLU + 3 x 3 / 2 / 1 max pooling as one kernel, or None when the layer is outside its limits."""
        if self.wt_rows is None or not self.relu:
            return None
        return ops.ternary_conv2d_stem_rows(images, self.wt_rows, self.cout, (self.ky, self.kx), self.stride, self.padding,
                                            self.scale, self.bias, relu=True, pool=True)

    def from_images(self, images, defer_relu=False):
        """Stem route: fp32 NCHW images -> bf16 NHWC feature map, patches built by a kernel (no torch glue).
        defer_relu: leave the activation to the caller (a max pooling that follows applies it for free)."""
        relu = self.relu and not defer_relu
        if self.wt_rows is not None:
            y = ops.ternary_conv2d_stem_rows(images, self.wt_rows, self.cout, (self.ky, self.kx), self.stride, self.padding,
                                             self.scale, self.bias, relu=relu)
            if y is not None:
                return y
        if self.dilation == (1, 1):
            y = ops.ternary_conv2d_stem(images, self.wt, self.cout, (self.ky, self.kx), self.stride, self.padding,
                                        self.scale, self.bias, relu=relu)
            if y is not None:
                return y
        a, (b, oh, ow) = ops.conv_patches(images, (self.ky, self.kx), self.stride, self.padding, self.dilation)
        y = ops.ternary_gemm(a, self.wt, self.cout, self.scale, self.bias).view(b, oh, ow, self.cout)
        return torch.relu_(y) if relu else y

    def __call__(self, x_nhwc, residual=None):
        """x_nhwc: bf16 [B, H, W, C] contiguous -> bf16 [B, OH, OW, Cout]; the optional residual is added before the
        ReLU inside the convolution's epilogue."""
        if not self.implicit:
            raise RuntimeError("PackedConv: this layer's channel count needs the from_images() route")
        if self.wt_s1 is not None:
            y = ops.ternary_conv2d_s1(x_nhwc, self.wt_s1, self.cout, (self.ky, self.kx), self.padding, self.dilation,
                                      self.scale, self.bias, relu=self.relu, residual=residual)
            if y is not None:
                return y
        return ops.ternary_conv2d_nhwc(x_nhwc, self.wt, self.cout, (self.ky, self.kx), self.stride, self.padding,
                                       self.dilation, self.scale, self.bias, relu=self.relu, residual=residual)


class PackedResNet18:
    """ResNet-18 inference from packed ternary weights; input NCHW fp32/bf16 images, output fp32 logits."""

    def __init__(self, model):
        model.eval()
        self.conv1 = PackedConv(model.conv1, model.bn1, relu=True)
        self.blocks = []
        for stage in (model.layer1, model.layer2, model.layer3, model.layer4):
            for blk in stage:
                down = None
                if blk.downsample is not None:
                    down = PackedConv(blk.downsample[0], blk.downsample[1], relu=False)
                self.blocks.append((PackedConv(blk.conv1, blk.bn1, relu=True), PackedConv(blk.conv2, blk.bn2, relu=True),
                                    down))
        fc = model.fc
        assert fc.weight.dtype == torch.int32
        self.fc_n, self.fc_k = [int(v) for v in fc.original_shape]
        self.fc_scale, self.fc_bias = _fold_bn(fc.bn, getattr(fc, "bias", None), float(fc.post_scale_imm))
        packed = fc.weight.data
        self.fc_wt = ops.prepack(packed, self.fc_n, ops.FMT_BF16)

    @torch.no_grad()
    def __call__(self, images, trace=None):
        """trace(name, layer, input, residual, output), when given, sees every layer's actual operands (layerwise
        checks); `layer` is the PackedConv, or None for the pooling layers and the classifier."""
        def seen(name, layer, x_in, res, y):
            if trace is not None:
                trace(name, layer, x_in, res, y)
            return y
        images = images.float()
        x = self.conv1.from_images_pooled(images) if trace is None else None      # stem, ReLU and pooling in one kernel
        if x is None:                                                              # layerwise trace, or outside its limits
            x = seen("conv1", self.conv1, images, None, self.conv1.from_images(images, defer_relu=True))   # bf16 NHWC
            x = seen("maxpool", None, x, None, ops.maxpool2d_nhwc(x, 3, 2, 1, relu=True))   # ReLU folded into the pooling
        for i, (c1, c2, down) in enumerate(self.blocks):
            identity = x if down is None else seen(f"block{i}.down", down, x, None, down(x))
            mid = seen(f"block{i}.conv1", c1, x, None, c1(x))
            x = seen(f"block{i}.conv2", c2, mid, identity, c2(mid, residual=identity))
        pooled = seen("avgpool", None, x, None, ops.avgpool_nhwc(x))                   # [B, 512] bf16, fp32 sums
        return seen("fc", None, pooled, None, ops.ternary_gemm(pooled, self.fc_wt, self.fc_n, self.fc_scale,
                                                               self.fc_bias, out_dtype=torch.float32))


class GraphedInference:
    """A PackedResNet18 pass captured into a CUDA graph for one input shape: the 22 launches of a pass replay as one
    graph launch, which is what small per-GPU batches need (at 32 images a pass is 22 kernels of ~15 us each and the
    host cannot issue them that fast one by one).  Call with a tensor of the captured shape; the logits come back in a
    tensor that the next call overwrites."""

    def __init__(self, net, example):
        self.net = net
        self.static_in = example.float().clone()
        stream = torch.cuda.Stream(device=example.device)
        stream.wait_stream(torch.cuda.current_stream(example.device))
        with torch.cuda.stream(stream):
            for _ in range(2):                       # warm up: lazy initialisation must not be captured
                net(self.static_in)
        torch.cuda.current_stream(example.device).wait_stream(stream)
        torch.cuda.synchronize(example.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.static_out = net(self.static_in)

    def __call__(self, images):
        if images.shape != self.static_in.shape or images.device != self.static_in.device:
            raise RuntimeError("GraphedInference: input shape or device differs from the captured one")
        self.static_in.copy_(images)                  # also converts bf16 / fp16 images to the captured fp32 input
        self.graph.replay()
        return self.static_out


def shard_batch(x, rank=None, world_size=None):
    """This rank's contiguous slice of a batch (batch-sharded inference needs no collective)."""
    r, w = tdist.world()
    r = r if rank is None else rank
    w = w if world_size is None else world_size
    b, e = tdist.shard_range(x.shape[0], r, w)
    return x[b:e]
