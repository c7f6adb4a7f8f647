"""Linear layers on the tcgen05 GEMM (csrc/kernels/gemm_tcgen05.cu).

``gemm_tn(a, b)`` computes ``a @ b.T`` for bf16 row-major ``a [M,K]`` and ``b [N,K]`` with the bias
and activation fused into the epilogue.  ``Linear`` builds forward and backward from it:

    y  = act(x W^T + b)                      gemm_tn(x, W)
    dz = dy * act'(.) ; db = colsum(dz)      one pass (bias_act_bwd kernel)
    dx = dz W                                gemm_nn(dz, W): W is read in place as an MN-major operand
    dW = dz^T x                              the split-K weight-gradient kernel of conv_tcgen05.cu, which reads dz and x
                                             as they are (both operands MN-major); transposed copies of the
                                             activations only for feature counts that are not multiples of 64

The reference has no GEMM or linear layer; this serves the CTR MLP and the BERT-shaped encoder.
CPU tensors (host-only tests) and shapes the kernel does not take (row strides that are not a
multiple of 16 bytes) use torch.matmul.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import base

_ACT = {None: 0, "none": 0, "relu": 1, "gelu": 2}


def _supported(a: torch.Tensor, b: torch.Tensor) -> bool:
    return (a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2
            and a.stride(1) == 1 and b.stride(1) == 1 and a.stride(0) % 8 == 0 and b.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0)


def gemm_tn(a, b, bias=None, act=None, want_pre=False):
    """act(a @ b.T + bias). Returns y, or (y, pre_activation) when want_pre."""
    code = _ACT[act]
    m, k = a.shape
    n = b.shape[0]
    assert b.shape[1] == k
    if not _supported(a, b):
        pre = a.float() @ b.float().t()
        if bias is not None:
            pre = pre + bias.float()
        y = F.relu(pre) if code == 1 else F.gelu(pre) if code == 2 else pre
        y = y.to(a.dtype)
        return (y, pre.to(a.dtype)) if want_pre else y
    c = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    pre = torch.empty_like(c) if want_pre else None
    bb = None if bias is None else bias.to(torch.bfloat16).contiguous()
    base.check(base.K().tipsk_gemm_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), base.ptr(bb), base.ptr(pre), m, n, k,
                                        a.stride(0), b.stride(0), n, code, base.stream()), "gemm_bf16")
    return (c, pre) if want_pre else c


def gemm_nn(a: torch.Tensor, b: torch.Tensor, into: torch.Tensor | None = None) -> torch.Tensor:
    """a @ b for bf16 row-major a [M,K] and b [K,N]: b is read in place as an MN-major operand.  With `into`
    (a contiguous [M,N] bf16 tensor) the product is added to it by the kernel's reduce-add stores."""
    m, k = a.shape
    n = b.shape[1]
    assert b.shape[0] == k
    if not (_supported(a, b) and n >= 64 and n % 8 == 0):
        c = gemm_tn(a, b.t().contiguous())
        return c if into is None else into.add_(c)
    if into is not None:
        assert into.shape == (m, n) and into.is_contiguous() and into.dtype == torch.bfloat16
        c = into
    else:
        c = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    base.check(base.K().tipsk_gemm_bf16_nn(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, a.stride(0), b.stride(0),
                                           n, 0 if into is None else 1, base.stream()), "gemm_bf16_nn")
    return c


def _weight_grad(dz: torch.Tensor, x2: torch.Tensor) -> torch.Tensor:
    """dz^T @ x2 as [N, K].  A linear layer is a 1x1 convolution over "pixels" = rows, so the convolution's
    weight-gradient kernel applies: it contracts over the rows with both operands read in place."""
    m, n = dz.shape
    k = x2.shape[1]
    if (dz.is_cuda and dz.dtype == torch.bfloat16 and x2.dtype == torch.bfloat16 and n % 64 == 0 and k % 64 == 0
            and m >= 16 and dz.is_contiguous() and x2.is_contiguous()
            and dz.data_ptr() % 16 == 0 and x2.data_ptr() % 16 == 0):
        dw = torch.empty(n, k, dtype=torch.float32, device=dz.device)
        base.check(base.K().tipsk_conv2d_wgrad(x2.data_ptr(), dz.data_ptr(), dw.data_ptr(), 1, 1, m, k, n, 1, 1, 1, 0,
                                               base.stream()), "linear_wgrad")
        return dw
    return gemm_tn(dz.t().contiguous(), x2.t().contiguous())


def gemm_status() -> int:
    """0 when no GEMM launch since the last call reported a bounded-wait timeout (synchronises)."""
    lib = base.K()
    return int(lib.tipsk_gemm_status()) or int(lib.tipsk_conv_status())  # the weight gradient runs on the conv kernels


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, act):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        code = _ACT[act]
        if code == 2:
            y, pre = gemm_tn(x2, weight, bias, act, want_pre=True)
        else:
            y, pre = gemm_tn(x2, weight, bias, act), None
        ctx.save_for_backward(x2, weight, y if code == 1 else pre, bias)
        ctx.act = code
        ctx.in_shape = x.shape
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        return _linear_backward(ctx, dy, None)


def _linear_backward(ctx, dy, d_alias):
    """Gradients of the fused linear layer; `d_alias` (optional) is the gradient of another consumer of x, into
    which dx is accumulated inside the GEMM."""
    x2, weight, saved, bias = ctx.saved_tensors
    n = weight.shape[0]
    dy2 = dy.reshape(-1, n)
    if not dy2.is_contiguous():
        dy2 = dy2.contiguous()
    dbias = None
    vec_ok = (n * dy2.element_size()) % 16 == 0  # the fused kernel works on 16-byte column vectors
    if dy2.is_cuda and vec_ok:
        dz = dy2
        db = torch.empty(n, dtype=torch.float32, device=dy2.device) if bias is not None else None
        if ctx.act != 0 or db is not None:
            if ctx.act != 0:
                dz = torch.empty_like(dy2)
            # ReLU: the mask of y equals the mask of the pre-activation, so y stands in for it.
            base.check(base.K().tipsk_bias_act_bwd(dy2.data_ptr(), base.ptr(saved) if ctx.act != 0 else None, None,
                                                   dz.data_ptr() if ctx.act != 0 else None, base.ptr(db),
                                                   dy2.shape[0], n, ctx.act, base.code(dy2), base.stream()),
                       "bias_act_bwd")
        if db is not None:
            dbias = db.to(bias.dtype)
    else:
        if ctx.act == 1:
            dz = dy2 * (saved > 0).to(dy2.dtype)
        elif ctx.act == 2:
            s = saved.float()
            dz = (dy2.float() * (0.5 * (1 + torch.erf(s / math.sqrt(2))) + s * torch.exp(-0.5 * s * s) / math.sqrt(2 * math.pi))).to(dy2.dtype)
        else:
            dz = dy2
        if bias is not None:
            dbias = dz.float().sum(0).to(bias.dtype)
    dx = dw = None
    if ctx.needs_input_grad[0]:
        into = None
        if d_alias is not None:
            into = d_alias.reshape(-1, x2.shape[1])
            if not (into.is_contiguous() and into.dtype == torch.bfloat16 and into.data_ptr() % 16 == 0):
                into = into.contiguous()
        dx = gemm_nn(dz, weight, into=into).view(ctx.in_shape)
    if ctx.needs_input_grad[1]:
        dw = _weight_grad(dz, x2).to(weight.dtype)
    return dx, dw, dbias, None


class _LinearPassFn(torch.autograd.Function):
    """linear(x) together with an alias of x for the other consumers of x (a residual connection): the backward pass
    adds dx into the gradient of that alias inside the GEMM (reduce-add stores) instead of leaving two tensors for
    autograd to sum.  The alias gradient is modified in place, so it must not be shared with another branch."""

    @staticmethod
    def forward(ctx, x, weight, bias, act):
        y = _LinearFn.forward(ctx, x, weight, bias, act)
        return y, x.detach()

    @staticmethod
    def backward(ctx, dy, d_alias):
        return _linear_backward(ctx, dy, d_alias)


def linear(x, weight, bias=None, act=None):
    """act(x @ weight.T + bias) with the epilogue fused into the GEMM."""
    return _LinearFn.apply(x, weight, bias, act)


def linear_passthrough(x, weight, bias=None, act=None):
    """(linear(x), alias of x): use the alias for the residual branch; see _LinearPassFn."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        return _LinearPassFn.apply(x, weight, bias, act)
    return linear(x, weight, bias, act), x


class Linear(nn.Module):
    def __init__(self, in_features, out_features, bias=True, act=None):
        super().__init__()
        self.in_features, self.out_features, self.act = in_features, out_features, act
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    def forward(self, x, passthrough=False):
        if passthrough:
            return linear_passthrough(x, self.weight, self.bias, self.act)
        return linear(x, self.weight, self.bias, self.act)
