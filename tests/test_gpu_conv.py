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
    s1 = torch.zeros(128, dtype=torch.float32, device=x.device)
    s2 = torch.zeros(128, dtype=torch.float32, device=x.device)
    y = conv2d(x, wgt, 1, 1, stats=(s1, s2))
    assert _status() == 0
    yf = y.float()
    ref1 = yf.sum(dim=(0, 2, 3))
    ref2 = (yf * yf).sum(dim=(0, 2, 3))
    assert torch.allclose(s1, ref1, rtol=1e-3, atol=1e-2)
    assert torch.allclose(s2, ref2, rtol=1e-3, atol=1e-2)


def test_conv_module_falls_back_for_the_stem():
    from tips_b200.ops.conv import Conv2d
    dev = torch.device("cuda", 0)
    conv = Conv2d(3, 64, 7, stride=2, padding=3).to(dev).to(torch.bfloat16)
    x = torch.randn(2, 3, 32, 32, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    y = conv(x)
    ref = F.conv2d(x.float(), conv.weight.float().permute(0, 3, 1, 2), stride=2, padding=3)
    assert (y.float() - ref).abs().max() <= 3e-2 * max(1.0, float(ref.abs().max()))
