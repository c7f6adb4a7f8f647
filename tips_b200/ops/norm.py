"""Normalisation layers backed by the sm_100a kernels in csrc/kernels/norm.cu and
layernorm.cu.

``BatchNorm2d`` works on channels-last activations and can fuse the residual add
and the ReLU that follow it in a ResNet block (forward and backward);
``LayerNorm`` normalises the last dimension.  The reference has no model math
of its own (it trains TensorFlow models); these are the "BN/LN" hot ops of the
flagship models.  On CPU tensors the layers compute the same function with
plain PyTorch so that host-only tests can run; on CUDA tensors the kernels are
mandatory.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import base


class _BatchNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, weight, bias, running_mean, running_var, training, momentum, eps, relu, stats=None):
        # x: NCHW tensor in channels_last memory format, i.e. an [N*H*W, C] matrix.
        assert x.is_cuda
        xc = x.contiguous(memory_format=torch.channels_last) if x.dim() == 4 else x.contiguous()
        c = xc.shape[1]
        m = xc.numel() // c
        y = torch.empty_like(xc)
        res = None
        if residual is not None:
            res = residual.contiguous(memory_format=torch.channels_last) if residual.dim() == 4 else residual.contiguous()
        lib = base.K()
        if training:
            save_mean = torch.empty(c, dtype=torch.float32, device=x.device)
            save_invstd = torch.empty(c, dtype=torch.float32, device=x.device)
            # How the backward pass will know the ReLU mask: without a residual it rebuilds it from x ("recompute");
            # with a residual the forward kernel leaves one bit per element ("bits"); otherwise it reads y.
            mode = "none"
            if relu:
                if residual is None:
                    mode = "recompute"
                elif c % 8 == 0 and xc.dtype != torch.float32:
                    mode = "bits"
                else:
                    mode = "y"
            ws = None
            if stats is None:
                parts = lib.tipsk_bn_partials(m, c)
                ws = torch.empty(parts * 2 * c, dtype=torch.float32, device=x.device)
                base.count_launches(2)
            bits = torch.empty(m * c // 8, dtype=torch.uint8, device=x.device) if mode == "bits" else None
            base.check(lib.tipsk_bn_fwd_train_mask(
                xc.data_ptr(), base.ptr(res), y.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                base.ptr(running_mean), base.ptr(running_var), save_mean.data_ptr(), save_invstd.data_ptr(),
                base.ptr(ws), base.ptr(stats), base.ptr(bits), m, c, eps, momentum, int(relu), base.code(xc),
                base.stream()), "bn_fwd_train")
            ctx.mask_mode = mode
            ctx.save_for_backward(xc, y if mode == "y" else None, weight, save_mean, save_invstd,
                                  bias if mode == "recompute" else None, bits)
        else:
            base.check(lib.tipsk_bn_fwd_eval(
                xc.data_ptr(), base.ptr(res), y.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                running_mean.data_ptr(), running_var.data_ptr(), m, c, eps, int(relu), base.code(xc), base.stream()),
                "bn_fwd_eval")
            ctx.mask_mode = "y" if relu else "none"
            ctx.save_for_backward(xc, y if relu else None, weight,
                                  running_mean.clone(), torch.rsqrt(running_var + eps), None, None)
        ctx.relu = bool(relu)
        ctx.has_res = residual is not None
        ctx.training_mode = bool(training)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, y, weight, save_mean, save_invstd, bias, bits = ctx.saved_tensors
        if not ctx.training_mode:
            raise RuntimeError("backward through batch norm in eval mode is not supported by the fused kernel")
        c = x.shape[1]
        m = x.numel() // c
        dyc = dy.contiguous(memory_format=torch.channels_last) if dy.dim() == 4 else dy.contiguous()
        dx = torch.empty_like(x)
        dres = torch.empty_like(x) if ctx.has_res else None
        dgamma = torch.empty(c, dtype=torch.float32, device=x.device)
        dbeta = torch.empty(c, dtype=torch.float32, device=x.device)
        lib = base.K()
        parts = lib.tipsk_bn_partials(m, c)
        ws = torch.empty(parts * 2 * c, dtype=torch.float32, device=x.device)
        if ctx.mask_mode == "bits":
            base.check(lib.tipsk_bn_bwd_bitmask(
                dyc.data_ptr(), x.data_ptr(), bits.data_ptr(), weight.data_ptr(), save_mean.data_ptr(),
                save_invstd.data_ptr(), dx.data_ptr(), base.ptr(dres), dgamma.data_ptr(), dbeta.data_ptr(),
                ws.data_ptr(), m, c, base.code(x), base.stream()), "bn_bwd_bitmask")
        elif ctx.mask_mode == "recompute":
            base.check(lib.tipsk_bn_bwd_relu_recompute(
                dyc.data_ptr(), x.data_ptr(), weight.data_ptr(), bias.data_ptr(), save_mean.data_ptr(),
                save_invstd.data_ptr(), dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), ws.data_ptr(), m, c,
                base.code(x), base.stream()), "bn_bwd_relu_recompute")
        else:
            base.check(lib.tipsk_bn_bwd(
                dyc.data_ptr(), x.data_ptr(), base.ptr(y), weight.data_ptr(), save_mean.data_ptr(),
                save_invstd.data_ptr(), dx.data_ptr(), base.ptr(dres), dgamma.data_ptr(), dbeta.data_ptr(),
                ws.data_ptr(), m, c, int(ctx.relu), base.code(x), base.stream()), "bn_bwd")
        base.count_launches(2)
        return dx, dres, dgamma.to(weight.dtype), dbeta.to(weight.dtype), None, None, None, None, None, None, None


def batch_norm(x, weight, bias, running_mean, running_var, training=True, momentum=0.1, eps=1e-5, relu=False,
               residual=None, stats=None):
    """y = relu?(BN(x) + residual?) on a channels-last activation.  `stats` (fp32 [2, C]: per-channel sums of x and
    of x^2, e.g. from a convolution epilogue) lets the training forward skip its reduction pass."""
    if x.is_cuda:
        return _BatchNormFn.apply(x, residual, weight, bias, running_mean, running_var, training, momentum, eps, relu,
                                  stats if training else None)
    y = F.batch_norm(x.float(), running_mean, running_var, weight.float(), bias.float(), training, momentum, eps)
    if residual is not None:
        y = y + residual.float()
    if relu:
        y = F.relu(y)
    return y.to(x.dtype)


class BatchNorm2d(nn.Module):
    """Batch norm over NHWC activations with optional fused residual add and ReLU.

    Affine parameters and running statistics are fp32 whatever the activation dtype.
    """

    def __init__(self, num_features, eps=1e-5, momentum=0.1, relu=False):
        super().__init__()
        self.num_features = num_features
        self.eps = eps
        self.momentum = momentum
        self.relu = relu
        self.weight = nn.Parameter(torch.ones(num_features, dtype=torch.float32))
        self.bias = nn.Parameter(torch.zeros(num_features, dtype=torch.float32))
        self.register_buffer("running_mean", torch.zeros(num_features, dtype=torch.float32))
        self.register_buffer("running_var", torch.ones(num_features, dtype=torch.float32))

    def _apply(self, fn, recurse=True):
        # keep the affine parameters and statistics in fp32 under .to(bf16) / .half()
        out = super()._apply(fn, recurse)
        for name in ("weight", "bias"):
            p = getattr(self, name)
            if p.dtype != torch.float32:
                p.data = p.data.float()
        for name in ("running_mean", "running_var"):
            b = getattr(self, name)
            if b.dtype != torch.float32:
                setattr(self, name, b.float())
        return out

    def forward(self, x, residual=None, stats=None):
        return batch_norm(x, self.weight, self.bias, self.running_mean, self.running_var, self.training,
                          self.momentum, self.eps, self.relu, residual, stats)


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, residual=None):
        cols = x.shape[-1]
        xc = x.contiguous()
        rows = xc.numel() // cols
        y = torch.empty_like(xc)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        w = weight.to(xc.dtype)
        b = bias.to(xc.dtype)
        if residual is not None:
            # LN(x + residual) in one pass; the sum is kept for the backward pass, whose dx goes to both inputs
            rc = residual.contiguous()
            summed = torch.empty_like(xc)
            base.check(base.K().tipsk_ln_fwd_residual(
                xc.data_ptr(), rc.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), summed.data_ptr(),
                mean.data_ptr(), rstd.data_ptr(), rows, cols, eps, base.code(xc), base.stream()), "ln_fwd_residual")
            xc = summed
        else:
            base.check(base.K().tipsk_ln_fwd(xc.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), mean.data_ptr(),
                                             rstd.data_ptr(), rows, cols, eps, base.code(xc), base.stream()), "ln_fwd")
        ctx.save_for_backward(xc, w, mean, rstd)
        ctx.wdtype = weight.dtype
        ctx.has_res = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, mean, rstd = ctx.saved_tensors
        cols = x.shape[-1]
        rows = x.numel() // cols
        dyc = dy.contiguous()
        dx = torch.empty_like(x)
        lib = base.K()
        parts = lib.tipsk_ln_bwd_partials(rows, cols)
        pg = torch.empty(parts, cols, dtype=torch.float32, device=x.device)
        pb = torch.empty(parts, cols, dtype=torch.float32, device=x.device)
        base.check(lib.tipsk_ln_bwd(dyc.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                    dx.data_ptr(), pg.data_ptr(), pb.data_ptr(), parts, rows, cols, base.code(x),
                                    base.stream()), "ln_bwd")
        dgamma = torch.empty(cols, dtype=torch.float32, device=x.device)
        dbeta = torch.empty(cols, dtype=torch.float32, device=x.device)
        base.check(lib.tipsk_ln_reduce_partials(pg.data_ptr(), pb.data_ptr(), parts, cols, dgamma.data_ptr(),
                                                dbeta.data_ptr(), 0, base.stream()), "ln_reduce")
        return dx, dgamma.to(ctx.wdtype), dbeta.to(ctx.wdtype), None, (dx if ctx.has_res else None)


def layer_norm(x, weight, bias, eps=1e-5, residual=None):
    """LN(x) or, with `residual`, LN(x + residual) with the add fused into the kernel."""
    if x.is_cuda:
        return _LayerNormFn.apply(x, weight, bias, eps, residual)
    if residual is not None:
        x = x + residual
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), bias.float(), eps).to(x.dtype)


class LayerNorm(nn.Module):
    def __init__(self, normalized_shape, eps=1e-5):
        super().__init__()
        self.normalized_shape = int(normalized_shape)
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(self.normalized_shape))
        self.bias = nn.Parameter(torch.zeros(self.normalized_shape))

    def forward(self, x, residual=None):
        return layer_norm(x, self.weight, self.bias, self.eps, residual)
