"""3x3 / stride 2 / pad 1 max pooling on channels-last activations (csrc/kernels/pool.cu).

The forward kernel stores one byte of argmax position per output element, so the backward kernel is a
deterministic gather that never re-reads the input activation.  Other configurations, CPU tensors and other
dtypes use ``torch.nn.functional.max_pool2d``.  The reference has no pooling of its own (its model math is
TensorFlow's); this is the stem pool of the ResNet-50 benchmark model.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import base


class _MaxPoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xc = x.contiguous(memory_format=torch.channels_last)
        n, c, h, w = xc.shape
        ho, wo = (h - 1) // 2 + 1, (w - 1) // 2 + 1
        y = torch.empty((n, c, ho, wo), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
        idx = torch.empty((n, ho, wo, c), dtype=torch.uint8, device=x.device)
        base.check(base.K().tipsk_maxpool3x3s2_fwd(xc.data_ptr(), y.data_ptr(), idx.data_ptr(), n, h, w, c,
                                                   base.code(xc), base.stream()), "maxpool_fwd")
        ctx.save_for_backward(idx)
        ctx.x_shape = (n, c, h, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        n, c, h, w = ctx.x_shape
        dyc = dy.contiguous(memory_format=torch.channels_last)
        dx = torch.empty(ctx.x_shape, dtype=dy.dtype, device=dy.device, memory_format=torch.channels_last)
        base.check(base.K().tipsk_maxpool3x3s2_bwd(dyc.data_ptr(), idx.data_ptr(), dx.data_ptr(), n, h, w, c,
                                                   base.code(dyc), base.stream()), "maxpool_bwd")
        return dx


def max_pool_3x3_s2(x: torch.Tensor) -> torch.Tensor:
    if x.is_cuda and x.dim() == 4 and x.dtype in (torch.bfloat16, torch.float16) and x.shape[1] % 8 == 0:
        return _MaxPoolFn.apply(x)
    return F.max_pool2d(x, 3, stride=2, padding=1)


class MaxPool3x3S2(nn.Module):
    def forward(self, x):
        return max_pool_3x3_s2(x)


class _GlobalAvgPoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xc = x.contiguous(memory_format=torch.channels_last)
        n, c, h, w = xc.shape
        y = torch.empty((n, c), dtype=x.dtype, device=x.device)
        base.check(base.K().tipsk_global_avgpool_fwd(xc.data_ptr(), y.data_ptr(), n, h * w, c, base.code(xc),
                                                     base.stream()), "avgpool_fwd")
        ctx.x_shape = (n, c, h, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        n, c, h, w = ctx.x_shape
        dyc = dy.contiguous()
        dx = torch.empty(ctx.x_shape, dtype=dy.dtype, device=dy.device, memory_format=torch.channels_last)
        base.check(base.K().tipsk_global_avgpool_bwd(dyc.data_ptr(), dx.data_ptr(), n, h * w, c, base.code(dyc),
                                                     base.stream()), "avgpool_bwd")
        return dx


def global_avg_pool(x: torch.Tensor) -> torch.Tensor:
    """[N, C, H, W] (channels-last) -> [N, C]: the mean over the pixels (the pooling in front of a classifier)."""
    es = x.element_size()
    if x.is_cuda and x.dim() == 4 and x.dtype in (torch.bfloat16, torch.float16, torch.float32) and (x.shape[1] * es) % 16 == 0:
        return _GlobalAvgPoolFn.apply(x)
    return x.float().mean(dim=(2, 3)).to(x.dtype)
