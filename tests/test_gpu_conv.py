"""tcgen05 implicit-GEMM convolutions (forward, data gradient, weight gradient) against PyTorch fp32."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

# n, h, w, cin, cout, k, stride
SHAPES = [
    (2, 8, 8, 64, 64, 1, 1),
    (2, 14, 14, 64, 64, 3, 1),
    (3, 10, 12, 128, 256, 3, 1),
    (2, 14, 14, 64, 128, 1, 2),
    (2, 14, 14, 64, 128, 3, 2),
    (4, 7, 7, 128, 128, 3, 1),
    (5, 9, 11, 64, 64, 3, 2),     # odd extents: the parity classes differ in size
    (8, 56, 56, 64, 256, 1, 1),
    (8, 56, 56, 64, 64, 3, 1),
    (4, 28, 28, 256, 512, 1, 2),
    (4, 28, 28, 128, 128, 3, 2),
    (32, 56, 56, 64, 64, 1, 1),   # enough tiles for the weights to stay resident in shared memory
]


def _status():
    from tips_b200.ops import base
    return base.K().tipsk_conv_status()


def _make(n, h, w, cin, cout, k, seed):
    torch.manual_seed(seed)
    dev = torch.device("cuda", 0)
    x = (torch.randn(n, cin, h, w, device=dev) * 0.5).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    wgt = (torch.randn(cout, k, k, cin, device=dev) * (1.0 / (k * cin ** 0.5))).to(torch.bfloat16)
    return x, wgt


@pytest.mark.parametrize("n,h,w,cin,cout,k,stride", SHAPES)
def test_conv_forward(n, h, w, cin, cout, k, stride):
    from tips_b200.ops.conv import conv2d, supported
    x, wgt = _make(n, h, w, cin, cout, k, 1)
    assert supported(x, wgt, stride, k // 2)
    y = conv2d(x, wgt, stride, k // 2)
    assert _status() == 0
    ref = F.conv2d(x.float(), wgt.float().permute(0, 3, 1, 2), stride=stride, padding=k // 2)
    assert y.shape == ref.shape
    scale = max(1.0, float(ref.abs().max()))
    assert (y.float() - ref).abs().max() <= 1.5e-2 * scale


@pytest.mark.parametrize("n,h,w,cin,cout,k,stride", SHAPES)
def test_conv_backward(n, h, w, cin, cout, k, stride):
    from tips_b200.ops.conv import conv2d
    x, wgt = _make(n, h, w, cin, cout, k, 2)
    x.requires_grad_()
    wgt.requires_grad_()
    y = conv2d(x, wgt, stride, k // 2)
    dy = (torch.randn_like(y.float()) * 0.5).to(torch.bfloat16)
    y.backward(dy)
    assert _status() == 0
    xr = x.detach().float().requires_grad_()
    wr = wgt.detach().float().requires_grad_()
    F.conv2d(xr, wr.permute(0, 3, 1, 2), stride=stride, padding=k // 2).backward(dy.float())
    sx = max(1.0, float(xr.grad.abs().max()))
    sw = max(1.0, float(wr.grad.abs().max()))
    assert (x.grad.float() - xr.grad).abs().max() <= 1.5e-2 * sx
    assert (wgt.grad.float() - wr.grad).abs().max() <= 1.5e-2 * sw


def test_conv_output_statistics():
    from tips_b200.ops.conv import conv2d
    x, wgt = _make(4, 14, 14, 64, 128, 3, 3)
    stats = torch.zeros(2, 128, dtype=torch.float32, device=x.device)
    y = conv2d(x, wgt, 1, 1, stats=stats)
    s1, s2 = stats[0], stats[1]
    assert _status() == 0
    yf = y.float()
    ref1 = yf.sum(dim=(0, 2, 3))
    ref2 = (yf * yf).sum(dim=(0, 2, 3))
    assert torch.allclose(s1, ref1, rtol=1e-3, atol=1e-2)
    assert torch.allclose(s2, ref2, rtol=1e-3, atol=1e-2)


@pytest.mark.parametrize("n,h,w", [(2, 32, 32), (3, 30, 46), (4, 224, 224)])
def test_stem_convolution(n, h, w):
    from tips_b200.ops.conv import Conv2d
    dev = torch.device("cuda", 0)
    torch.manual_seed(n)
    conv = Conv2d(3, 64, 7, stride=2, padding=3).to(dev).to(torch.bfloat16)
    x = torch.randn(n, 3, h, w, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    stats = torch.zeros(2, 64, dtype=torch.float32, device=dev)
    y = conv(x, stats=stats)
    dy = (torch.randn_like(y.float()) * 0.1).to(torch.bfloat16)
    y.backward(dy)
    assert _status() == 0
    wr = conv.weight.detach().float().requires_grad_()
    ref = F.conv2d(x.float(), wr.permute(0, 3, 1, 2), stride=2, padding=3)
    ref.backward(dy.float())
    assert y.shape == ref.shape
    assert (y.detach().float() - ref.detach()).abs().max() <= 2e-2 * max(1.0, float(ref.abs().max()))
    assert torch.allclose(stats[0], y.detach().float().sum(dim=(0, 2, 3)), rtol=1e-3, atol=0.1)
    sw = max(1.0, float(wr.grad.abs().max()))
    assert (conv.weight.grad.float() - wr.grad).abs().max() <= 2e-2 * sw


def test_stem_takes_an_fp32_nchw_image():
    """The stem fed an fp32 NCHW batch (layout change and cast inside its padding copy) gives the same output and
    weight gradient as the stem fed the bf16 channels-last copy of that batch."""
    from tips_b200.ops.conv import Conv2d
    dev = torch.device("cuda", 0)
    torch.manual_seed(5)
    conv = Conv2d(3, 64, 7, stride=2, padding=3).to(dev).to(torch.bfloat16)
    raw = torch.randn(3, 3, 62, 94, device=dev)
    x = raw.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    y0 = conv(x)
    dy = (torch.randn_like(y0.float()) * 0.1).to(torch.bfloat16)
    y0.backward(dy)
    g0 = conv.weight.grad.clone()
    conv.weight.grad = None
    y1 = conv(raw)
    y1.backward(dy)
    assert _status() == 0
    assert y1.dtype == torch.bfloat16 and torch.equal(y0, y1)
    # the weight gradient is summed over pixel ranges with fp32 atomics, so its last bits depend on arrival order
    assert torch.allclose(g0.float(), conv.weight.grad.float(), rtol=2e-2, atol=2e-2 * float(g0.float().abs().max()))


def test_conv_module_falls_back_for_other_filters():
    from tips_b200.ops.conv import Conv2d
    dev = torch.device("cuda", 0)
    conv = Conv2d(16, 24, 5, stride=1, padding=2).to(dev).to(torch.bfloat16)
    x = torch.randn(2, 16, 12, 12, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    y = conv(x)
    ref = F.conv2d(x.float(), conv.weight.float().permute(0, 3, 1, 2), stride=1, padding=2)
    assert (y.float() - ref).abs().max().item() <= 3e-2 * max(1.0, float(ref.abs().max()))


def test_resnet_block_matches_library_convolutions():
    """One bottleneck stack with full-width channels: tcgen05 convolutions + fused statistics against the same
    weights run through library convolutions."""
    from tips_b200.models import resnet50 as R
    dev = torch.device("cuda", 0)
    torch.manual_seed(5)
    ours = R.ResNet50(num_classes=16, layers=(1, 1, 1, 1), width=64).to(dev).to(torch.bfloat16).train()
    R._LIBRARY_CONV = True
    try:
        lib = R.ResNet50(num_classes=16, layers=(1, 1, 1, 1), width=64).to(dev).to(torch.bfloat16).train()
    finally:
        R._LIBRARY_CONV = False
    src = dict(ours.named_parameters())
    with torch.no_grad():
        for name, p in lib.named_parameters():
            q = src[name]
            p.copy_(q.permute(0, 3, 1, 2) if (p.dim() == 4 and q.shape != p.shape) or (p.dim() == 4) else q)
        # give the zero-initialised last BN of each block a non-trivial scale
        for m1, m2 in zip(ours.modules(), lib.modules()):
            if isinstance(m1, R.BatchNorm2d):
                m1.weight.fill_(0.5)
                m2.weight.fill_(0.5)
    x = torch.randn(8, 3, 64, 64, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 16, (8,), device=dev)
    l1 = ours.loss(x, y)
    l2 = lib.loss(x, y)
    l1.backward()
    l2.backward()
    assert _status() == 0
    assert abs(float(l1) - float(l2)) <= 5e-2 * max(1.0, abs(float(l2)))
    g1 = dict(ours.named_parameters())
    checked = 0
    for name, p in lib.named_parameters():
        if p.grad is None or p.dim() != 4:
            continue
        ga = g1[name].grad.float().permute(0, 3, 1, 2)
        gb = p.grad.float()
        # bf16 rounding differences compound through the depth of the network: compare directions
        cos = float((ga * gb).sum() / (ga.norm() * gb.norm() + 1e-12))
        assert cos >= 0.97, (name, cos)
        checked += 1
    assert checked >= 10


@pytest.mark.parametrize("k,stride", [(1, 1), (3, 1), (1, 2), (3, 2)])
def test_conv_passthrough_accumulates_the_branch_gradient(k, stride):
    from tips_b200.ops.conv import conv2d_passthrough
    x, wgt = _make(4, 14, 14, 64, 128, k, 7)
    x.requires_grad_()
    wgt.requires_grad_()
    y, alias = conv2d_passthrough(x, wgt, stride, k // 2)
    side = (alias.float() * 0.5).to(torch.bfloat16)   # another consumer of x
    dy = (torch.randn_like(y.float()) * 0.5).to(torch.bfloat16)
    dside = (torch.randn_like(side.float())).to(torch.bfloat16)
    torch.autograd.backward([y, side], [dy, dside])
    assert _status() == 0
    xr = x.detach().float().requires_grad_()
    wr = wgt.detach().float().requires_grad_()
    yr = F.conv2d(xr, wr.permute(0, 3, 1, 2), stride=stride, padding=k // 2)
    torch.autograd.backward([yr, xr * 0.5], [dy.float(), dside.float()])
    sx = max(1.0, float(xr.grad.abs().max()))
    assert (x.grad.float() - xr.grad).abs().max() <= 2e-2 * sx
