"""Convolution through the reference's own layer API, and the two ResNet-18 configurations at the sizes they are quoted on.

  * tmq.Conv2d.compact_forward (the method the reference implements as F.unfold + ternary_mmm_cuda + reshape,
    tmq/tmq.py:822-871) routes to the implicit-GEMM kernels: bf16, int8 and - exactly - fp32 activations, NCHW and
    channels_last inputs; no unfold anywhere in a ResNet-18 under bf16;
  * the convolution's int8 and fp32-output forms through the C ABI, before any output rounding;
  * packed ResNet-18 inference at the benchmarked configuration (batch 256, 224 x 224, weights at P = .35/.3/.35): every
    layer against fp64 torch on that layer's actual input, plus a sampled end-to-end check;
  * the ResNet-18 QAT step against the reference's own CPU run (tests/golden/resnet_qat_step.npz)."""
import os

import numpy as np
import pytest
import torch
from torch import nn

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from tmq_b200 import ops
    return ops


@pytest.fixture(scope="module")
def tmq():
    import tmq_b200
    return tmq_b200


def _ternary(shape, gen, p=(0.35, 0.3, 0.35)):
    u = torch.rand(shape, generator=gen)
    return torch.where(u < p[0], -1.0, torch.where(u < p[0] + p[1], 0.0, 1.0))


def _compact_conv(tmq, cin, cout, k, stride, padding, dilation, gen, bias=True):
    layer = tmq.Conv2d(cin, cout, k, stride=stride, padding=padding, dilation=dilation, bias=bias, ctrl=None,
                       quant_mode=tmq.QuantMode.TERNARY)
    with torch.no_grad():
        layer.weight.copy_(_ternary(layer.weight.shape, gen))
        if bias:
            layer.bias.copy_(torch.randn(cout, generator=gen))
    layer.cuda().eval()
    w = layer.weight.detach().clone()
    holder = nn.Sequential()
    holder.add_module("conv", layer)
    tmq.compressed_state_dict(holder)
    assert layer.compact and layer.weight.dtype == torch.int32
    return layer, w


GEOMS = [(64, 64, 3, 1, 1, 1, 12, 12), (64, 128, 3, 2, 1, 1, 15, 13), (128, 72, 1, 2, 0, 1, 14, 14),
         (64, 96, 3, 1, 2, 2, 10, 11), (256, 128, 3, 1, 1, 1, 7, 7)]


@pytest.mark.parametrize("geom", GEOMS)
def test_compact_forward_takes_the_implicit_kernels(tmq, ops, geom, monkeypatch):
    cin, cout, k, s, p, d, h, w = geom
    gen = torch.Generator().manual_seed(sum(geom))
    layer, wgt = _compact_conv(tmq, cin, cout, k, s, p, d, gen)

    def no_unfold(*a, **kw):
        raise AssertionError("compact_forward materialised patches")
    monkeypatch.setattr(torch.nn.functional, "unfold", no_unfold)
    x32 = torch.randn(3, cin, h, w, generator=gen).cuda()
    ref = nn.functional.conv2d(x32.double(), wgt.double(), layer.bias.double(), s, p, d)
    # fp32 activations: exact products, fp32 accumulation -> fp32 GEMM accuracy, no bf16 rounding anywhere
    y32 = layer(x32)
    ops.check_gemm_status()
    assert y32.dtype == torch.float32 and y32.shape == ref.shape
    assert float((y32.double() - ref).abs().max()) <= 2e-5 * float(ref.abs().max())
    assert torch.equal(layer(x32.contiguous(memory_format=torch.channels_last)), y32)
    # bf16 activations, both memory layouts, same bits; result is channels_last
    xb = x32.to(torch.bfloat16)
    refb = nn.functional.conv2d(xb.double(), wgt.double(), layer.bias.double(), s, p, d)
    yb = layer(xb)
    assert yb.dtype == torch.bfloat16 and yb.is_contiguous(memory_format=torch.channels_last)
    tol = 2.0 ** -7 * refb.abs() + 1e-4 * refb.abs().max()
    assert bool(((yb.double() - refb).abs() <= tol).all())
    assert torch.equal(layer(xb.contiguous(memory_format=torch.channels_last)), yb)
    # int8 activations: exact integers, bias not applied (the bare sums, as for Linear)
    xi = torch.randint(-127, 128, (3, cin, h, w), generator=gen, dtype=torch.int8).cuda()
    yi = layer(xi)
    refi = nn.functional.conv2d(xi.double(), wgt.double(), None, s, p, d)
    assert yi.dtype == torch.int32 and torch.equal(yi.double(), refi)
    ops.check_gemm_status()


def test_post_scale_and_three_d_input(tmq, ops):
    gen = torch.Generator().manual_seed(5)
    layer = tmq.Conv2d(64, 64, 3, padding=1, bias=False, ctrl=None, quant_mode=tmq.QuantMode.TERNARY, post_scale=True)
    with torch.no_grad():
        layer.weight.copy_(_ternary(layer.weight.shape, gen))
    layer.cuda().eval()
    wgt = layer.weight.detach().clone()
    holder = nn.Sequential(layer)
    tmq.compressed_state_dict(holder)
    x = torch.randn(64, 9, 9, generator=gen).cuda()
    ref = nn.functional.conv2d(x.double().unsqueeze(0), wgt.double(), None, 1, 1)[0] * layer.post_scale_imm
    y = layer(x)
    assert y.shape == ref.shape and float((y.double() - ref).abs().max()) <= 2e-5 * float(ref.abs().max())


def test_conv_abi_int8_and_fp32_output_before_rounding(ops):
    """tmq_ternary_conv2d_i8: bit-exact; tmq_ternary_conv2d_bf16_f32out: rel 1e-3 of the fp64 result asked for, 1e-5 met."""
    gen = torch.Generator().manual_seed(8)
    for (b, c, h, w, n, k, s, p, d) in [(2, 64, 9, 11, 64, 3, 1, 1, 1), (1, 192, 8, 8, 80, 3, 2, 1, 1), (2, 128, 7, 7, 136, 1, 1, 0, 1)]:
        wgt = _ternary((n, c, k, k), gen)
        rows = ops.compactify_ternary(wgt.cuda())
        xb = torch.randn(b, c, h, w, generator=gen).to(torch.bfloat16).cuda()
        scale = (torch.rand(n, generator=gen) * 0.09 + 0.01).cuda()
        bias = torch.randn(n, generator=gen).cuda()
        wt = ops.prepack(ops.conv_rows_kkc(rows, c, k, k), n, ops.FMT_BF16)
        y = ops.ternary_conv2d_nhwc(xb.permute(0, 2, 3, 1).contiguous(), wt, n, (k, k), (s, s), (p, p), (d, d), scale, bias,
                                    out_dtype=torch.float32)
        ref = nn.functional.conv2d(xb.double(), wgt.double().cuda(), None, s, p, d) * scale.double().view(1, -1, 1, 1) \
            + bias.double().view(1, -1, 1, 1)
        err = (y.permute(0, 3, 1, 2).double() - ref).abs()
        rms = ref.pow(2).mean().sqrt()
        assert bool((err <= 1e-3 * torch.maximum(ref.abs(), rms)).all())
        assert bool((err <= 1e-5 * torch.maximum(ref.abs(), rms)).all())
        xi = torch.randint(-127, 128, (b, c, h, w), generator=gen, dtype=torch.int8).cuda()
        wt8 = ops.prepack(ops.conv_rows_kkc(rows, c, k, k, pad_to=1), n, ops.FMT_I8)
        yi = ops.ternary_conv2d_nhwc(xi.permute(0, 2, 3, 1).contiguous(), wt8, n, (k, k), (s, s), (p, p), (d, d))
        refi = nn.functional.conv2d(xi.double(), wgt.double().cuda(), None, s, p, d)
        assert torch.equal(yi.permute(0, 3, 1, 2).double(), refi)
    ops.check_gemm_status()


def test_layout_kernels(ops):
    gen = torch.Generator().manual_seed(13)
    x = torch.randn(37, 50, generator=gen) * torch.exp(torch.randn(37, 50, generator=gen) * 4)
    x[0, :4] = torch.tensor([0.0, -0.0, 1.0, 3.0e38])
    s = ops.split_f32(x.cuda(), 3, 56)
    assert s.shape == (37, 168)
    lo, mid, hi = s[:, :50].float(), s[:, 56:106].float(), s[:, 112:162].float()
    assert torch.equal(hi + mid + lo, x.cuda())                                   # three bf16 terms rebuild the fp32 value
    assert torch.equal(hi, x.cuda().to(torch.bfloat16).float())                   # smallest term first, leading term last
    assert float(s[:, 50:56].abs().max()) == 0.0 and float(s[:, 162:].abs().max()) == 0.0
    assert torch.equal(ops.split_f32(x.cuda(), 1), x.cuda().to(torch.bfloat16))
    img = torch.randn(3, 70, 9, 5, generator=gen).cuda()
    assert torch.equal(ops.nchw_to_nhwc_bf16(img), img.permute(0, 2, 3, 1).to(torch.bfloat16).contiguous())
    t3 = ops.nchw_to_nhwc_bf16(img, 3)
    assert t3.shape == (3, 9, 5, 210)
    assert torch.equal(t3[..., 140:].float() + t3[..., 70:140].float() + t3[..., :70].float(), img.permute(0, 2, 3, 1))
    f = torch.randn(4, 7, 7, 512, generator=gen).to(torch.bfloat16).cuda()
    want = f.double().mean(dim=(1, 2))
    got = ops.avgpool_nhwc(f).double()
    assert bool(((got - want).abs() <= 2.0 ** -8 * want.abs() + 1e-6).all())


def _packed_resnet(tmq, seed):
    from tmq_b200 import workloads
    torch.manual_seed(seed)
    model, ctrl = workloads.build_resnet18(101, ctrl=tmq.QuantizationControl())
    gen = torch.Generator().manual_seed(seed + 1)
    with torch.no_grad():
        for node in ctrl._registry.values():
            node.weight.copy_(_ternary(node.weight.shape, gen))
        for m in model.modules():
            if isinstance(m, (nn.BatchNorm2d, nn.BatchNorm1d)):
                # keep activations O(1) through the net: a ternary fan-in sum of unit-variance inputs has variance
                # 0.7 * fan_in, which the running variance reflects
                m.running_mean.normal_(0, 0.1, generator=gen)
                m.weight.uniform_(0.8, 1.2, generator=gen)
                m.bias.normal_(0, 0.2, generator=gen)
        for name, m in model.named_modules():
            if isinstance(m, tmq.Conv2d):
                fan_in = m.weight[0].numel()
                bn = dict(model.named_modules())[name.replace("conv", "bn").replace("downsample.0", "downsample.1")]
                bn.running_var.fill_(0.7 * fan_in * 0.6)
        model.fc.bn.running_var.fill_(0.7 * 512 * 0.3)
    model.cuda().eval()
    weights = {name: m.weight.detach().clone() for name, m in model.named_modules() if isinstance(m, (tmq.Conv2d, tmq.Linear))}
    tmq.compressed_state_dict(model)
    return model, workloads.PackedResNet18(model), weights


def test_packed_resnet18_every_layer_at_the_benchmarked_configuration(tmq, ops):
    """Batch 256 of 224 x 224 images.  Each layer's output is compared, on a spread of images, with fp64 torch applied to
    the very bf16 tensor the layer received: one bf16 ulp of the output plus accumulation slack.  A wrong residual add,
    a wrong fold of BatchNorm or a geometry slip in any single layer fails here however late in the net it sits."""
    model, net, weights = _packed_resnet(tmq, 21)
    gen = torch.Generator(device="cuda").manual_seed(3)
    images = torch.randn(256, 3, 224, 224, generator=gen, device="cuda")
    pick = torch.tensor([0, 1, 100, 127, 128, 254, 255], device="cuda")
    seen = []

    def check(name, layer, x_in, res, y):
        seen.append(name)
        if layer is not None:
            w = ops.expand_ternary(layer.layer.weight.data, list(layer.layer.original_shape)).double()
            if name == "conv1":
                xin = x_in[pick].to(torch.bfloat16).double()                    # the stem rounds the image to bf16 itself
            else:
                xin = x_in[pick].permute(0, 3, 1, 2).double()
            ref = nn.functional.conv2d(xin, w, None, layer.stride, layer.padding, layer.dilation)
            ref = ref * layer.scale.double().view(1, -1, 1, 1) + layer.bias.double().view(1, -1, 1, 1)
            if res is not None:
                ref = ref + res[pick].permute(0, 3, 1, 2).double()
            if layer.relu and name != "conv1":                                   # the stem's ReLU is applied by the pooling
                ref = torch.relu(ref)
            got = y[pick].permute(0, 3, 1, 2).double()
            tol = 2.0 ** -7 * ref.abs() + 1e-4 * ref.abs().max()
            bad = (got - ref).abs() > tol
            assert not bool(bad.any()), (name, int(bad.sum()), float((got - ref).abs().max()), float(ref.abs().max()))
            assert float(ref.abs().max()) > 0.1 and bool(torch.isfinite(got).all()), name
        elif name == "maxpool":
            want = torch.relu(nn.functional.max_pool2d(x_in[pick].permute(0, 3, 1, 2).float(), 3, 2, 1))
            assert torch.equal(y[pick].permute(0, 3, 1, 2).float(), want)
        elif name == "avgpool":
            want = x_in[pick].double().mean(dim=(1, 2))
            assert bool(((y[pick].double() - want).abs() <= 2.0 ** -8 * want.abs() + 1e-6).all())
        elif name == "fc":
            wfc = weights["fc"].double()
            ref = (x_in[pick].double() @ wfc.t()) * net.fc_scale.double() + net.fc_bias.double()
            assert float((y[pick].double() - ref).abs().max()) <= 1e-5 * float(ref.abs().max())

    logits = net(images, trace=check)
    ops.check_gemm_status()
    assert len(seen) == 1 + 1 + 8 * 2 + 3 + 2 and logits.shape == (256, 101)
    # end to end on the sampled images: an fp64 chain that rounds to bf16 wherever the kernels do
    with torch.no_grad():
        def conv(pc, x, res=None, relu=None):
            w = ops.expand_ternary(pc.layer.weight.data, list(pc.layer.original_shape)).double()
            r = nn.functional.conv2d(x, w, None, pc.stride, pc.padding, pc.dilation) * pc.scale.double().view(1, -1, 1, 1) \
                + pc.bias.double().view(1, -1, 1, 1)
            if res is not None:
                r = r + res
            if pc.relu if relu is None else relu:
                r = torch.relu(r)
            return r.to(torch.bfloat16).double()
        x = conv(net.conv1, images[pick].to(torch.bfloat16).double(), relu=False)
        x = torch.relu(nn.functional.max_pool2d(x, 3, 2, 1))
        for c1, c2, down in net.blocks:
            identity = x if down is None else conv(down, x)
            x = conv(c2, conv(c1, x), res=identity)
        pooled = x.mean(dim=(2, 3)).to(torch.bfloat16).double()
        want = (pooled @ weights["fc"].double().t()) * net.fc_scale.double() + net.fc_bias.double()
    assert float((logits[pick].double() - want).abs().max()) <= 0.02 * float(want.abs().max())
    assert int((logits[pick].argmax(1) == want.argmax(1)).sum()) >= len(pick) - 1


def test_api_route_and_packed_pipeline_give_the_same_bits(tmq, ops):
    """tmq.Conv2d.compact_forward and workloads.PackedConv are two callers of one kernel: with an identity BatchNorm
    folded in they must agree bit for bit."""
    from tmq_b200 import workloads
    gen = torch.Generator().manual_seed(17)
    for cin, cout, k, s, p in [(64, 64, 3, 1, 1), (128, 256, 3, 2, 1), (64, 128, 1, 2, 0)]:
        layer, _ = _compact_conv(tmq, cin, cout, k, s, p, 1, gen, bias=False)
        bn = nn.BatchNorm2d(cout).cuda().eval()
        bn.running_var.fill_(1.0 - bn.eps)                                      # scale = gamma / sqrt(var + eps) = 1 exactly
        pc = workloads.PackedConv(layer, bn, relu=False)
        assert torch.equal(pc.scale, torch.ones_like(pc.scale)) and float(pc.bias.abs().max()) == 0.0
        x = torch.randn(4, cin, 14, 14, generator=gen).to(torch.bfloat16).cuda().contiguous(memory_format=torch.channels_last)
        a = layer(x)
        b = pc(x.permute(0, 2, 3, 1))
        assert torch.equal(a.permute(0, 2, 3, 1), b)
    # and a whole compact model through the API: no unfold, finite logits, same top-1 as the packed pipeline mostly
    model, net, _ = _packed_resnet(tmq, 33)
    imgs = torch.randn(8, 3, 224, 224, device="cuda")
    real_unfold = torch.nn.functional.unfold
    torch.nn.functional.unfold = None
    try:
        with torch.no_grad():
            y_api = model.to(torch.bfloat16)(imgs.to(torch.bfloat16))
    finally:
        torch.nn.functional.unfold = real_unfold
    ops.check_gemm_status()
    y_packed = net(imgs)
    assert y_api.shape == (8, 101) and bool(torch.isfinite(y_api.float()).all())
    assert float((y_api.float() - y_packed).abs().max()) <= 0.1 * float(y_packed.abs().max())


def _seeded_fill(model, seed):
    # the same rule as tests/golden/make_golden.py: seeded_fill
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for key, t in model.state_dict().items():
            if not t.is_floating_point() or key.endswith("post_scale"):
                continue
            if key.endswith("running_var"):
                t.copy_(torch.rand(t.shape, generator=g) + 0.5)
            elif key.endswith("running_mean"):
                t.copy_(torch.randn(t.shape, generator=g) * 0.1)
            elif t.dim() >= 2:
                t.copy_(torch.rand(t.shape, generator=g) * 2.4 - 1.2)
            elif "bn" in key.split(".")[-2] and key.endswith("weight"):
                t.copy_(torch.rand(t.shape, generator=g) + 0.5)
            elif key.endswith("weight") and t.dim() == 1:
                t.copy_(torch.rand(t.shape, generator=g) + 0.5)
            else:
                t.copy_(torch.randn(t.shape, generator=g) * 0.1)


def test_resnet18_qat_step_matches_the_reference_cpu_run(tmq):
    """Baseline config 4a at test size against the reference's own CPU execution (fixture made by
    tests/golden/make_golden.py: make_resnet_qat_step): same seeded parameters, same batch, epoch 44 of the default
    50-epoch schedule.  The soft-step and loss kernels are bit-exact; what differs is cuDNN against the CPU convolutions
    (fp32 both, TF32 off), so the bars are fp32 reorder noise through twenty layers."""
    from tmq_b200 import workloads
    G = np.load(os.path.join(GOLDEN, "resnet_qat_step.npz"), allow_pickle=False)
    old = (torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32)
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        torch.manual_seed(0)
        model, ctrl = workloads.build_resnet18(101)
        assert len(ctrl._registry) == int(G["n_registered"])
        _seeded_fill(model, 4242)
        for e in range(1, 45):
            ctrl.step(e)
        assert ctrl.digamma == float(G["digamma"]) and ctrl.qpenalty == float(G["qpenalty"])
        model.cuda().train()
        x, y = torch.from_numpy(G["x"]).cuda(), torch.from_numpy(G["y"]).cuda()
        logits = model(x)
        ce = nn.functional.cross_entropy(logits, y)
        ql = ctrl.quantization_loss()
        (ce + ql).backward()
        want = torch.from_numpy(G["logits"]).cuda()
        err = float((logits - want).abs().max() / want.abs().max())
        assert err <= 2e-3, err
        assert abs(ce.item() - float(G["ce"])) <= 1e-3 * float(G["ce"])
        assert abs(ql.item() - float(G["qloss"])) <= 1e-6 * float(G["qloss"])
        params = dict(model.named_parameters())
        for key in G.files:
            if key.startswith("grad/"):
                g_ref = torch.from_numpy(G[key]).cuda()
                g = params[key[5:]].grad
                e = float((g - g_ref).abs().max() / g_ref.abs().max())
                assert e <= 1e-2, (key, e)
        ctrl.clamp()
        got = params["layer1.0.conv1.weight"].detach().cpu().numpy()
        assert np.array_equal(got.view(np.uint32), G["clamped/layer1.0.conv1.weight"].view(np.uint32))
    finally:
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = old


def test_second_device_gets_its_own_kernel_attributes(ops):
    """The shared-memory opt-in of the tensor-core kernels is per device: a GEMM and a convolution on cuda:1 after
    cuda:0, in one process."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from oracle import ternary as T
    rng = np.random.default_rng(0)
    W = rng.integers(-1, 2, (128, 256)).astype(np.float32)
    P = T.pack(W)
    X = torch.randn(200, 256).to(torch.bfloat16)
    ref = T.gemm_f64_fast(X.float().numpy(), P, 128)
    for dev in ("cuda:0", "cuda:1"):
        wt = ops.prepack(torch.from_numpy(P).to(dev), 128, ops.FMT_BF16)
        y = ops.ternary_gemm(X.to(dev), wt, 128, out_dtype=torch.float32)
        ops.check_gemm_status(dev)
        assert np.abs(y.cpu().numpy() - ref).max() <= 1e-5 * np.abs(ref).max(), dev
        wc = torch.randint(-1, 2, (64, 64, 3, 3)).float()
        rows = ops.compactify_ternary(wc.to(dev))
        xc = torch.randn(2, 64, 9, 9).to(torch.bfloat16)
        yc = ops.ternary_conv2d_nhwc(xc.to(dev).permute(0, 2, 3, 1).contiguous(),
                                     ops.prepack(ops.conv_rows_kkc(rows, 64, 3, 3), 64, ops.FMT_BF16), 64, (3, 3), (1, 1),
                                     (1, 1), (1, 1), out_dtype=torch.float32)
        refc = nn.functional.conv2d(xc.double(), wc.double(), None, 1, 1)
        assert float((yc.permute(0, 3, 1, 2).double().cpu() - refc).abs().max()) <= 1e-5 * float(refc.abs().max())
        ops.check_gemm_status(dev)


def test_graphed_inference_replays_the_pass(tmq, ops):
    """The packed ResNet-18 pass captured into a CUDA graph gives the bits of the launch-by-launch pass, also for a
    second input of the same shape."""
    from tmq_b200 import workloads
    _, net, _ = _packed_resnet(tmq, 21)
    x1 = torch.randn(4, 3, 64, 64, device="cuda")
    x2 = torch.randn(4, 3, 64, 64, device="cuda")
    g = workloads.GraphedInference(net, x1)
    assert torch.equal(g(x1).clone(), net(x1))
    assert torch.equal(g(x2).clone(), net(x2))
    ops.check_gemm_status()
    with pytest.raises(RuntimeError):
        g(torch.randn(2, 3, 64, 64, device="cuda"))


@pytest.mark.parametrize("shape,k,s,p", [((8, 64, 112, 112), 3, 2, 1), ((3, 8, 17, 23), 3, 2, 1), ((2, 4, 9, 9), 2, 2, 0),
                                         ((2, 12, 10, 14), 3, 1, 1), ((1, 4, 5, 5), 5, 3, 2)])
def test_training_maxpool_matches_torch(ops, shape, k, s, p):
    """Forward values and winners, and the gathered backward, against torch's max_pool2d on the same channels-last
    fp32 tensor: inputs with many exact ties (a ReLU's zeros) and a NaN."""
    gen = torch.Generator().manual_seed(sum(shape) + k)
    x = torch.relu(torch.randn(shape, generator=gen)).cuda()             # about half the values are exactly zero: ties
    x[0, 0, 0, 0] = float("nan")
    x = x.contiguous(memory_format=torch.channels_last)
    xa = x.clone().requires_grad_(True)
    xb = x.clone().requires_grad_(True)
    ya = ops.maxpool2d_train(xa, k, s, p)
    yb = torch.nn.functional.max_pool2d(xb, k, s, p)
    assert ya.shape == yb.shape
    assert torch.equal(torch.nan_to_num(ya.detach(), nan=-7.0), torch.nan_to_num(yb.detach(), nan=-7.0))
    g = torch.randn(ya.shape, generator=gen).cuda().contiguous(memory_format=torch.channels_last)
    ya.backward(g)
    yb.backward(g)
    assert xa.grad.shape == xb.grad.shape
    assert float((xa.grad - xb.grad).abs().max()) <= 1e-6 * float(xb.grad.abs().max())
    # anything the kernels do not cover falls back to torch's pooling
    z = torch.randn(2, 3, 8, 8, device="cuda")                           # 3 channels, not channels-last
    assert torch.equal(ops.maxpool2d_train(z, 3, 2, 1), torch.nn.functional.max_pool2d(z, 3, 2, 1))
