"""tcgen05 GEMM against a PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 512, 256), (8192, 512, 1680), (300, 1000, 2048),
                                   (1000, 16, 256), (512, 1, 256), (130, 72, 40), (4096, 1024, 4096),
                                   (16384, 4096, 2048), (9400, 1024, 4096)])  # the last two take 256 x 256 tiles
@pytest.mark.parametrize("act", [None, "relu", "gelu"])
def test_gemm_tn(m, n, k, act):
    from tips_b200.ops.linear import gemm_status, gemm_tn
    torch.manual_seed(m + n + k)
    dev = torch.device("cuda", 0)
    a = (torch.randn(m, k, device=dev) * 0.5).to(torch.bfloat16)
    b = (torch.randn(n, k, device=dev) * 0.5).to(torch.bfloat16)
    bias = torch.randn(n, device=dev).to(torch.bfloat16)
    y, pre = gemm_tn(a, b, bias, act, want_pre=True)
    assert gemm_status() == 0
    ref_pre = a.float() @ b.float().t() + bias.float()
    ref = torch.relu(ref_pre) if act == "relu" else torch.nn.functional.gelu(ref_pre) if act == "gelu" else ref_pre
    scale = max(1.0, float(ref_pre.abs().max()))
    assert (pre.float() - ref_pre).abs().max() <= 1e-2 * scale
    assert (y.float() - ref).abs().max() <= 1e-2 * scale


def test_linear_module_grads():
    from tips_b200.ops.linear import Linear
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    lin = Linear(256, 512, act="relu").to(dev).to(torch.bfloat16)
    x = torch.randn(1024, 256, device=dev).to(torch.bfloat16).requires_grad_()
    y = lin(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    w = lin.weight.detach().float().requires_grad_()
    b = lin.bias.detach().float().requires_grad_()
    yr = torch.relu(xr @ w.t() + b)
    yr.backward(dy.float())
    assert torch.allclose(y.float(), yr, atol=0.1, rtol=5e-2)
    assert torch.allclose(x.grad.float(), xr.grad, atol=0.3, rtol=5e-2)
    assert torch.allclose(lin.weight.grad.float(), w.grad, atol=0.6, rtol=5e-2)
    assert torch.allclose(lin.bias.grad.float(), b.grad, atol=0.6, rtol=5e-2)


@pytest.mark.parametrize("m,n,k", [(128, 64, 64), (256, 512, 256), (8192, 1728, 512), (300, 1000, 2048),
                                   (16384, 1024, 4096), (20000, 256, 512), (16384, 4096, 2048), (9400, 1024, 4096)])
def test_gemm_nn(m, n, k):
    from tips_b200.ops.linear import gemm_nn, gemm_status
    torch.manual_seed(m + n + k)
    dev = torch.device("cuda", 0)
    a = (torch.randn(m, k, device=dev) * 0.5).to(torch.bfloat16)
    b = (torch.randn(k, n, device=dev) * 0.5).to(torch.bfloat16)
    y = gemm_nn(a, b)
    assert gemm_status() == 0
    ref = a.float() @ b.float()
    assert (y.float() - ref).abs().max() <= 1e-2 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("m,n,k", [(32768, 2048, 1024), (4096, 512, 256), (1000, 64, 128)])
def test_linear_weight_grad(m, n, k):
    """dW = dz^T x on the split-K MN-major kernel; the first shape takes its 256 x 256 tile."""
    from tips_b200.ops.linear import _weight_grad, gemm_status
    torch.manual_seed(m)
    dev = torch.device("cuda", 0)
    dz = (torch.randn(m, n, device=dev) * 0.25).to(torch.bfloat16)
    x = (torch.randn(m, k, device=dev) * 0.25).to(torch.bfloat16)
    dw = _weight_grad(dz, x)
    assert gemm_status() == 0
    ref = dz.float().t() @ x.float()
    assert (dw.float() - ref).abs().max() <= 1e-2 * max(1.0, float(ref.abs().max()))
