"""Convolution (im2col + tcgen05 GEMM), batch norm + residual + ReLU and pooling on NHWC
tensors: the PyTorch reference paths against ``F.conv2d`` / ``F.batch_norm`` / ``F.max_pool2d``
on CPU, the native kernels against those reference paths on a GPU (small and odd shapes), and
a small ResNet trained on both."""
import pytest
import torch
import torch.nn.functional as F


def _nchw(x):
    return x.permute(0, 3, 1, 2)


CONV_CASES = [(2, 9, 9, 16, 24, 3, 1, 1), (2, 10, 9, 16, 8, 3, 2, 1), (2, 20, 20, 3, 16, 7, 2, 3),
              (3, 8, 8, 32, 16, 1, 1, 0), (2, 9, 9, 16, 40, 1, 2, 0)]


def _conv_pair(case, dtype, device):
    from necklace_b200.ops.conv import Conv2d
    N, H, W, Ci, Co, k, s, p = case
    torch.manual_seed(0)
    conv = Conv2d(Ci, Co, k, s, p, dtype=dtype, device=device)
    x = torch.randn(N, H, W, Ci).to(dtype).to(device).requires_grad_(True)
    return conv, x


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv_reference_path_matches_torch(case):
    conv, x = _conv_pair(case, torch.float32, None)
    N, H, W, Ci, Co, k, s, p = case
    y = conv(x)
    ref = F.conv2d(_nchw(x), conv.weight_oihw(), stride=s, padding=p)
    assert torch.allclose(_nchw(y), ref, atol=1e-4)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().clone().requires_grad_(True)
    wr = conv.weight_oihw().detach().clone().requires_grad_(True)
    F.conv2d(_nchw(xr), wr, stride=s, padding=p).backward(_nchw(g))
    assert torch.allclose(x.grad, xr.grad, atol=1e-4)
    gw = conv.weight.grad[:, :k * k * Ci].view(Co, k, k, Ci).permute(0, 3, 1, 2)
    assert torch.allclose(gw, wr.grad, atol=1e-3)


@pytest.mark.parametrize("relu,res", [(False, False), (True, False), (True, True)])
def test_batchnorm_reference_path_matches_torch(relu, res):
    from necklace_b200.ops.conv import BatchNorm2d
    torch.manual_seed(1)
    bn = BatchNorm2d(16, relu=relu, dtype=torch.float32)
    with torch.no_grad():
        bn.weight.copy_(torch.rand(16) + 0.5)
        bn.bias.copy_(torch.randn(16) * 0.1)
    x = torch.randn(3, 5, 7, 16, requires_grad=True)
    r = torch.randn(3, 5, 7, 16, requires_grad=True) if res else None
    y = bn(x, r)
    xr = x.detach().clone().requires_grad_(True)
    rr = r.detach().clone().requires_grad_(True) if res else None
    w, b = bn.weight.detach().clone().requires_grad_(True), bn.bias.detach().clone().requires_grad_(True)
    ref = F.batch_norm(_nchw(xr), None, None, w, b, True, 0.1, 1e-5).permute(0, 2, 3, 1)
    if res:
        ref = ref + rr
    if relu:
        ref = torch.relu(ref)
    assert torch.allclose(y, ref, atol=1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    ref.backward(g)
    assert torch.allclose(x.grad, xr.grad, atol=1e-4)
    assert torch.allclose(bn.weight.grad, w.grad, atol=1e-4)
    assert torch.allclose(bn.bias.grad, b.grad, atol=1e-4)
    if res:
        assert torch.allclose(r.grad, rr.grad, atol=1e-5)


def test_pooling_reference_paths():
    from necklace_b200.ops.conv import global_avg_pool, max_pool_3x3_s2
    x = torch.randn(2, 9, 10, 8, requires_grad=True)
    y = max_pool_3x3_s2(x)
    ref = F.max_pool2d(_nchw(x.detach()), 3, 2, 1)
    assert torch.equal(_nchw(y), ref)
    y.sum().backward()
    assert float(x.grad.sum()) == y.numel()
    z = torch.randn(2, 3, 3, 8, requires_grad=True)
    a = global_avg_pool(z)
    assert torch.allclose(a, z.mean((1, 2)))
    a.sum().backward()
    assert torch.allclose(z.grad, torch.full_like(z, 1 / 9))


# ------------------------------------------------------------------------------- GPU
def _rel(a, b):
    return float((a.float().cpu() - b.float().cpu()).norm() / (b.float().cpu().norm() + 1e-12))


@pytest.mark.gpu
@pytest.mark.parametrize("case", CONV_CASES + [(4, 56, 56, 64, 64, 3, 1, 1)])
def test_conv_gpu_matches_fp32(case):
    from necklace_b200.ops import check_status
    conv, x = _conv_pair(case, torch.bfloat16, "cuda")
    N, H, W, Ci, Co, k, s, p = case
    y = conv(x)
    g = torch.randn_like(y)
    y.backward(g)
    torch.cuda.synchronize()
    check_status()
    xr = x.detach().float().cpu().requires_grad_(True)
    wr = conv.weight_oihw().detach().float().cpu().requires_grad_(True)
    ref = F.conv2d(_nchw(xr), wr, stride=s, padding=p)
    ref.backward(_nchw(g.float().cpu()))
    assert _rel(_nchw(y), ref) < 1e-2
    assert _rel(x.grad, xr.grad) < 1.5e-2
    gw = conv.weight.grad[:, :k * k * Ci].view(Co, k, k, Ci).permute(0, 3, 1, 2)
    assert _rel(gw, wr.grad) < 1.5e-2


@pytest.mark.gpu
@pytest.mark.parametrize("shape,relu,res", [((2, 9, 9, 24), False, False), ((3, 7, 5, 64), True, False),
                                            ((2, 14, 14, 256), True, True), ((1, 3, 3, 8), True, True)])
def test_batchnorm_gpu_matches_fp32(shape, relu, res):
    from necklace_b200.ops import check_status
    from necklace_b200.ops.conv import BatchNorm2d
    torch.manual_seed(2)
    C = shape[-1]
    bn = BatchNorm2d(C, relu=relu, device="cuda")
    ref_bn = BatchNorm2d(C, relu=relu, dtype=torch.float32)
    w0, b0 = (torch.rand(C) + 0.5).bfloat16(), (torch.randn(C) * 0.1).bfloat16()
    with torch.no_grad():
        bn.weight.copy_(w0)
        bn.bias.copy_(b0)
        ref_bn.weight.copy_(w0.float())
        ref_bn.bias.copy_(b0.float())
    x = torch.randn(shape).bfloat16()
    r = torch.randn(shape).bfloat16() if res else None
    g = torch.randn(shape).bfloat16()
    xg = x.cuda().requires_grad_(True)
    rg = r.cuda().requires_grad_(True) if res else None
    y = bn(xg, rg)
    y.backward(g.cuda())
    torch.cuda.synchronize()
    check_status()
    xc = x.float().requires_grad_(True)
    rc = r.float().requires_grad_(True) if res else None
    yc = ref_bn(xc, rc)
    yc.backward(g.float())
    assert _rel(y, yc) < 1e-2
    assert _rel(xg.grad, xc.grad) < 2e-2
    assert _rel(bn.weight.grad, ref_bn.weight.grad) < 2e-2
    assert _rel(bn.bias.grad, ref_bn.bias.grad) < 2e-2
    if res:
        assert _rel(rg.grad, rc.grad) < 1e-2
    assert _rel(bn.running_mean, ref_bn.running_mean) < 1e-2
    assert _rel(bn.running_var, ref_bn.running_var) < 1e-2


@pytest.mark.gpu
def test_pooling_gpu_matches_fp32():
    from necklace_b200.ops.conv import global_avg_pool, max_pool_3x3_s2
    torch.manual_seed(3)
    for shape in [(2, 9, 10, 16), (1, 112, 112, 64), (3, 7, 7, 8)]:
        x = torch.randn(shape).bfloat16()
        g = None
        xg = x.cuda().requires_grad_(True)
        xc = x.float().requires_grad_(True)
        yg, yc = max_pool_3x3_s2(xg), max_pool_3x3_s2(xc)
        assert torch.equal(yg.float().cpu(), yc)
        g = torch.randn_like(yc).bfloat16()
        yg.backward(g.cuda())
        yc.backward(g.float())
        assert _rel(xg.grad, xc.grad) < 1e-2
    x = torch.randn(4, 7, 7, 64).bfloat16()
    xg, xc = x.cuda().requires_grad_(True), x.float().requires_grad_(True)
    ag, ac = global_avg_pool(xg), global_avg_pool(xc)
    assert _rel(ag, ac) < 1e-2
    g = torch.randn(4, 64).bfloat16()
    ag.backward(g.cuda())
    ac.backward(g.float())
    assert _rel(xg.grad, xc.grad) < 1e-2


def _small_resnet(device, dtype_cast):
    from necklace_b200.models.resnet import ResNet
    torch.manual_seed(0)
    net = ResNet(classes=10, layers=(1, 1, 1, 1), width=16)
    return net.to(device) if dtype_cast is None else net.to(dtype_cast).to(device)


def test_small_resnet_trains_on_cpu_reference_paths():
    from necklace_b200.parallel.engine import OptimConfig, TrainEngine
    net = _small_resnet("cpu", torch.float32)
    eng = TrainEngine(net, optim=OptimConfig("sgd", lr=0.05, beta1=0.9))
    g = torch.Generator().manual_seed(1)
    x, y = torch.randn(8, 3, 32, 32, generator=g), torch.randint(0, 10, (8,), generator=g)
    losses = [float(eng.step(x.float(), y)) for _ in range(5)]
    assert losses[-1] < losses[0]


@pytest.mark.gpu
def test_small_resnet_gpu_matches_cpu_fp32():
    """Five SGD-momentum steps of a small ResNet on the native kernels (bf16, fp32 master)
    follow the fp32 CPU run of the same network and data."""
    from necklace_b200.ops import check_status
    from necklace_b200.parallel.engine import OptimConfig, TrainEngine
    g = torch.Generator().manual_seed(1)
    x, y = torch.randn(16, 3, 32, 32, generator=g), torch.randint(0, 10, (16,), generator=g)
    opt = OptimConfig("sgd", lr=0.05, beta1=0.9)
    cpu = TrainEngine(_small_resnet("cpu", torch.float32), optim=opt)
    gpu = TrainEngine(_small_resnet("cuda", None), optim=opt)
    lc = [float(cpu.step(x, y)) for _ in range(5)]
    lg = [float(gpu.step(x.cuda(), y.cuda())) for _ in range(5)]
    torch.cuda.synchronize()
    check_status()
    assert lg[-1] < lg[0]
    assert all(abs(a - b) < 0.08 * max(1.0, abs(a)) for a, b in zip(lc, lg)), (lc, lg)
