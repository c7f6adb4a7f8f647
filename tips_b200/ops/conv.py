"""Channels-last bf16 convolution backed by the tcgen05 implicit-GEMM kernels (csrc/kernels/conv_tcgen05.cu).

``Conv2d`` keeps its weight as ``[C_out, R, S, C_in]`` (the K-major operand layout of the kernels) and takes
activations that are NCHW tensors in ``channels_last`` memory format, i.e. NHWC in memory.  Forward, data
gradient and weight gradient all run on the tensor cores through TMA-loaded shifted boxes; nothing is
unfolded.  The 7x7 stem on 3-channel images runs on the same kernels through a padded 8-channel copy of the
image.  Shapes the kernels do not cover (CPU tensors, other dtypes, other filter sizes) go through
``torch.nn.functional.conv2d`` on a permuted view of the same weight.

The reference has no convolution of its own: its evaluated model is a TensorFlow ResNet-50 (README.md:12).
"""
from __future__ import annotations

import math
import os

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import base


# TIPS_CONV_DGRAD_TRANSPOSED_COPY=1: give the data gradient a transposed copy of the weights (K-major operand)
# instead of the forward weights themselves; kept for A/B measurements.
_DGRAD_TRANSPOSED_COPY = os.environ.get("TIPS_CONV_DGRAD_TRANSPOSED_COPY", "0") == "1"


def _is_stem(x, weight, stride, padding) -> bool:
    """The 7x7 / stride 2 / pad 3 convolution of a 3-channel image that needs no input gradient."""
    cout, r, s, cin = weight.shape
    return (cin == 3 and r == 7 and s == 7 and stride == 2 and padding == 3 and cout % 64 == 0
            and not x.requires_grad)


def _is_raw_image(x, weight, stride, padding) -> bool:
    """An fp32 NCHW image batch handed straight to the stem: the padding copy changes layout and casts."""
    return (x.dtype == torch.float32 and x.dim() == 4 and x.is_contiguous() and weight.dtype == torch.bfloat16
            and _is_stem(x, weight, stride, padding))


def supported(x: torch.Tensor, weight: torch.Tensor, stride: int, padding: int) -> bool:
    if x.is_cuda and _is_raw_image(x, weight, stride, padding):
        return True
    if not (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 4):
        return False
    if _is_stem(x, weight, stride, padding):
        return True
    cout, r, s, cin = weight.shape
    return bool(base.K().tipsk_conv2d_supported(cin, cout, r, s, stride, padding))


def _nhwc(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous(memory_format=torch.channels_last)


def conv2d_forward(x, weight, stride, padding, stats=None):
    """y = conv(x, weight); `stats` = fp32 [2, C_out] tensor, zeroed by the caller, that receives the per-channel sum
    and sum of squares of the bf16 output from the kernel's epilogue."""
    xc = _nhwc(x)
    n, cin, h, w = xc.shape
    cout, r, s, _ = weight.shape
    ho = (h + 2 * padding - r) // stride + 1
    wo = (w + 2 * padding - s) // stride + 1
    y = torch.empty((n, cout, ho, wo), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
    wc = weight.contiguous()
    base.check(base.K().tipsk_conv2d_fwd(
        xc.data_ptr(), wc.data_ptr(), y.data_ptr(), n, h, w, cin, cout, r, s, stride, padding,
        stats.data_ptr() if stats is not None else None,
        stats.data_ptr() + 4 * cout if stats is not None else None, base.stream()), "conv2d_fwd")
    return xc, y


def conv2d_dgrad(dy, weight, x_shape, stride, padding, into=None):
    """Data gradient; with `into` (a channels-last tensor of x's shape) the gradient is added to it in place by
    the kernel's reduce-add stores and `into` is returned."""
    n, cin, h, w = x_shape
    cout, r, s, _ = weight.shape
    dyc = _nhwc(dy)
    if into is not None:
        assert tuple(into.shape) == tuple(x_shape) and into.is_contiguous(memory_format=torch.channels_last)
        dx = into
    else:
        dx = torch.empty(x_shape, dtype=dy.dtype, device=dy.device, memory_format=torch.channels_last)
    launches = 1 if stride == 1 else (1 if r == 1 else 4)
    if _DGRAD_TRANSPOSED_COPY:
        wt = weight.permute(3, 1, 2, 0).contiguous()  # [C_in, R, S, C_out], K-major for the contraction over C_out
        base.check(base.K().tipsk_conv2d_dgrad(
            dyc.data_ptr(), wt.data_ptr(), dx.data_ptr(), n, h, w, cin, cout, r, s, stride, padding,
            1 if into is not None else 0, base.stream()), "conv2d_dgrad")
    else:
        # the forward weights as they are: the kernel contracts over their rows (MN-major operand)
        base.check(base.K().tipsk_conv2d_dgrad_ohwi(
            dyc.data_ptr(), weight.contiguous().data_ptr(), dx.data_ptr(), n, h, w, cin, cout, r, s, stride, padding,
            1 if into is not None else 0, base.stream()), "conv2d_dgrad")
    base.count_launches(launches - 1)
    return dx


def conv2d_wgrad(x, dy, weight_shape, stride, padding):
    cout, r, s, cin = weight_shape
    xc, dyc = _nhwc(x), _nhwc(dy)
    n, _, h, w = xc.shape
    dw = torch.empty(weight_shape, dtype=torch.float32, device=x.device)
    base.check(base.K().tipsk_conv2d_wgrad(
        xc.data_ptr(), dyc.data_ptr(), dw.data_ptr(), n, h, w, cin, cout, r, s, stride, padding, base.stream()),
        "conv2d_wgrad")
    return dw


class _Conv2dFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, stride, padding, stats):
        xc, y = conv2d_forward(x, weight, stride, padding, stats)
        ctx.save_for_backward(xc, weight)
        ctx.stride, ctx.padding = stride, padding
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, weight = ctx.saved_tensors
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = conv2d_dgrad(dy, weight, tuple(xc.shape), ctx.stride, ctx.padding)
        if ctx.needs_input_grad[1]:
            dw = conv2d_wgrad(xc, dy, tuple(weight.shape), ctx.stride, ctx.padding).to(weight.dtype)
        return dx, dw, None, None, None


class _Conv2dPassFn(torch.autograd.Function):
    """conv(x) together with an alias of x for the other consumers of x (a residual branch).  The backward pass then
    sees the gradient of that alias next to the gradient of the convolution output and adds the data gradient into
    it inside the kernel, instead of producing a second tensor for autograd to sum.  The alias gradient is modified
    in place: it must not be shared with another branch."""

    @staticmethod
    def forward(ctx, x, weight, stride, padding, stats):
        xc, y = conv2d_forward(x, weight, stride, padding, stats)
        ctx.save_for_backward(xc, weight)
        ctx.stride, ctx.padding = stride, padding
        return y, x.detach()

    @staticmethod
    def backward(ctx, dy, d_alias):
        xc, weight = ctx.saved_tensors
        dx = dw = None
        if ctx.needs_input_grad[0]:
            into = None
            if d_alias is not None:
                into = d_alias if d_alias.is_contiguous(memory_format=torch.channels_last) else _nhwc(d_alias)
            dx = conv2d_dgrad(dy, weight, tuple(xc.shape), ctx.stride, ctx.padding, into=into)
        if ctx.needs_input_grad[1]:
            dw = conv2d_wgrad(xc, dy, tuple(weight.shape), ctx.stride, ctx.padding).to(weight.dtype)
        return dx, dw, None, None, None


class _StemFn(torch.autograd.Function):
    """7x7 / stride 2 stem: the image is copied once into a zero-padded 8-channel buffer in which the horizontal
    taps of a filter row are contiguous; forward and weight gradient then run on the same tcgen05 kernels as the
    other convolutions (seven filter-row taps of 64 elements each)."""

    @staticmethod
    def forward(ctx, x, weight, stats):
        import ctypes
        lib = base.K()
        raw = x.dtype == torch.float32
        xc = x if raw else _nhwc(x)
        n, _, h, w = xc.shape
        cout = weight.shape[0]
        g = [ctypes.c_int() for _ in range(4)]
        lib.tipsk_stem_geometry(h, w, *[ctypes.byref(v) for v in g])
        hp, wp, ho, wo = (v.value for v in g)
        xp = torch.empty((n, hp, wp, 8), dtype=weight.dtype, device=x.device)
        if raw:
            base.check(lib.tipsk_stem_pad_nchw_f32(xc.data_ptr(), xp.data_ptr(), n, h, w, base.stream()),
                       "stem_pad_nchw")
        else:
            base.check(lib.tipsk_stem_pad(xc.data_ptr(), xp.data_ptr(), n, h, w, base.stream()), "stem_pad")
        wpad = F.pad(weight, (0, 5, 0, 1)).contiguous()  # [C_out, 7, 8, 8]
        y = torch.empty((n, cout, ho, wo), dtype=weight.dtype, device=x.device, memory_format=torch.channels_last)
        base.check(lib.tipsk_stem_conv_fwd(
            xp.data_ptr(), wpad.data_ptr(), y.data_ptr(), n, h, w, cout,
            stats.data_ptr() if stats is not None else None,
            stats.data_ptr() + 4 * cout if stats is not None else None, base.stream()), "stem_conv_fwd")
        ctx.save_for_backward(xp)
        ctx.geom = (n, h, w, cout)
        ctx.wdtype = weight.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        (xp,) = ctx.saved_tensors
        n, h, w, cout = ctx.geom
        dyc = _nhwc(dy)
        dw = torch.empty((cout, 7, 8, 8), dtype=torch.float32, device=dy.device)
        base.check(base.K().tipsk_stem_conv_wgrad(xp.data_ptr(), dyc.data_ptr(), dw.data_ptr(), n, h, w, cout,
                                                  base.stream()), "stem_conv_wgrad")
        return None, dw[:, :, :7, :3].to(ctx.wdtype), None


def conv2d_passthrough(x, weight, stride=1, padding=0, stats=None):
    """(conv(x), alias of x); see _Conv2dPassFn.  Falls back to the plain pair when the kernels do not apply."""
    if supported(x, weight, stride, padding) and not _is_stem(x, weight, stride, padding):
        return _Conv2dPassFn.apply(x, weight, stride, padding, stats)
    return conv2d(x, weight, stride, padding, stats), x


def conv2d(x, weight, stride=1, padding=0, stats=None):
    """Convolution of a channels-last activation with an ``[C_out, R, S, C_in]`` weight."""
    if supported(x, weight, stride, padding):
        if _is_stem(x, weight, stride, padding):
            return _StemFn.apply(x, weight, stats)
        return _Conv2dFn.apply(x, weight, stride, padding, stats)
    if stats is not None:
        raise ValueError("fused output statistics need a shape the tcgen05 kernels cover")
    return F.conv2d(x, weight.permute(0, 3, 1, 2), stride=stride, padding=padding)


class Conv2d(nn.Module):
    """Bias-free 2-D convolution with an ``[C_out, R, S, C_in]`` weight."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding = kernel_size, stride, padding
        self.weight = nn.Parameter(torch.empty(out_channels, kernel_size, kernel_size, in_channels))
        # He initialisation on the fan-out, the usual choice for ResNets
        std = math.sqrt(2.0 / (out_channels * kernel_size * kernel_size))
        nn.init.normal_(self.weight, 0.0, std)

    def forward(self, x, stats=None):
        return conv2d(x, self.weight, self.stride, self.padding, stats)

    def extra_repr(self):
        return (f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, stride={self.stride}, "
                f"padding={self.padding}, layout=OHWI")
