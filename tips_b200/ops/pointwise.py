"""Pointwise epilogues and fused losses (csrc/kernels/epilogue.cu):
bias + activation, binary cross-entropy with logits, softmax cross-entropy.
CPU tensors take a plain PyTorch path so that host-only tests can run."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import base

_ACT = {None: 0, "none": 0, "relu": 1, "gelu": 2}


class _BiasActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, act):
        cols = x.shape[-1]
        xc = x.contiguous()
        rows = xc.numel() // cols
        y = torch.empty_like(xc)
        b = None if bias is None else bias.to(xc.dtype).contiguous()
        base.check(base.K().tipsk_bias_act_fwd(xc.data_ptr(), base.ptr(b), y.data_ptr(), rows, cols, act,
                                               base.code(xc), base.stream()), "bias_act_fwd")
        ctx.save_for_backward(xc, b)
        ctx.act = act
        ctx.bias_dtype = None if bias is None else bias.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x, b = ctx.saved_tensors
        cols = x.shape[-1]
        rows = x.numel() // cols
        dyc = dy.contiguous()
        need_dx = ctx.act != 0
        dx = torch.empty_like(x) if need_dx else dyc
        dbias = torch.empty(cols, dtype=torch.float32, device=x.device) if b is not None else None
        base.check(base.K().tipsk_bias_act_bwd(dyc.data_ptr(), x.data_ptr(), base.ptr(b),
                                               dx.data_ptr() if need_dx else None, base.ptr(dbias), rows, cols,
                                               ctx.act, base.code(x), base.stream()), "bias_act_bwd")
        return dx, (None if dbias is None else dbias.to(ctx.bias_dtype)), None


def bias_act(x, bias=None, act="relu"):
    """act(x + bias) with act in {None, "relu", "gelu"}; bias broadcasts over the last dimension."""
    a = _ACT[act]
    if x.is_cuda:
        return _BiasActFn.apply(x, bias, a)
    y = x if bias is None else x + bias
    if a == 1:
        y = F.relu(y)
    elif a == 2:
        y = F.gelu(y)
    return y


class _SigmoidBceFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, reduction_scale):
        z = logits.contiguous()
        t = targets.to(torch.float32).contiguous()
        n = z.numel()
        loss = torch.zeros((), dtype=torch.float32, device=z.device)
        dz = torch.empty_like(z)
        base.check(base.K().tipsk_sigmoid_bce(z.data_ptr(), t.data_ptr(), loss.data_ptr(), dz.data_ptr(), n,
                                              reduction_scale, base.code(z), base.stream()), "sigmoid_bce")
        ctx.save_for_backward(dz)
        return loss * reduction_scale

    @staticmethod
    def backward(ctx, dloss):
        (dz,) = ctx.saved_tensors
        return dz * dloss.to(dz.dtype), None, None


def sigmoid_bce_loss(logits, targets, reduction="mean"):
    """Binary cross-entropy with logits; the gradient is produced in the same pass as the loss."""
    scale = 1.0 / logits.numel() if reduction == "mean" else 1.0
    if logits.is_cuda:
        return _SigmoidBceFn.apply(logits, targets, scale)
    return F.binary_cross_entropy_with_logits(logits.float(), targets.float(), reduction=reduction)


class _DotSigmoidBceFn(torch.autograd.Function):
    """loss = reduction(BCE(x @ w + b, targets)) for a layer with ONE output unit, in two streaming kernels
    (forward keeps d loss / d logit; backward produces dx, dw, db in one pass over x)."""

    @staticmethod
    def forward(ctx, x, weight, bias, targets, scale):
        x2 = x if x.stride(-1) == 1 else x.contiguous()
        rows, k = x2.shape
        w = weight.reshape(-1).contiguous()
        t = targets.to(torch.float32).contiguous()
        loss = torch.empty((), dtype=torch.float32, device=x.device)
        dz = torch.empty(rows, dtype=torch.float32, device=x.device)
        base.check(base.K().tipsk_dot_sigmoid_bce_fwd(x2.data_ptr(), w.data_ptr(), base.ptr(bias), t.data_ptr(),
                                                      loss.data_ptr(), dz.data_ptr(), None, rows, k, x2.stride(0),
                                                      scale, base.code(x2), base.stream()), "dot_sigmoid_bce_fwd")
        ctx.save_for_backward(x2, w, dz)
        ctx.meta = (weight.shape, weight.dtype, None if bias is None else bias.dtype)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        x2, w, dz = ctx.saved_tensors
        wshape, wdtype, bdtype = ctx.meta
        rows, k = x2.shape
        dx = torch.empty(rows, k, dtype=x2.dtype, device=x2.device)
        dw = torch.empty(k, dtype=torch.float32, device=x2.device)
        db = torch.empty(1, dtype=torch.float32, device=x2.device) if bdtype is not None else None
        up = dloss.to(torch.float32).contiguous()
        base.check(base.K().tipsk_dot_sigmoid_bce_bwd(x2.data_ptr(), w.data_ptr(), dz.data_ptr(), up.data_ptr(),
                                                      dx.data_ptr(), dw.data_ptr(), base.ptr(db), rows, k,
                                                      x2.stride(0), base.code(x2), base.stream()),
                   "dot_sigmoid_bce_bwd")
        return dx, dw.view(wshape).to(wdtype), (None if db is None else db.to(bdtype)), None, None


def linear1_sigmoid_bce_loss(x, weight, bias, targets, reduction="mean"):
    """Binary cross-entropy of ``sigmoid(x @ weight.T + bias)`` for a ``[1, K]`` weight: the one-unit output layer
    of a click model and its loss as one op.  Same value and gradients as
    ``sigmoid_bce_loss(linear(x, weight, bias).view(-1), targets)``."""
    assert weight.shape[0] == 1 and x.dim() == 2
    scale = 1.0 / x.shape[0] if reduction == "mean" else 1.0
    es = x.element_size()
    if (x.is_cuda and x.dtype == weight.dtype and x.dtype in (torch.bfloat16, torch.float16, torch.float32)
            and (x.shape[1] * es) % 16 == 0 and (x.stride(0) * es) % 16 == 0 and x.data_ptr() % 16 == 0
            and (bias is None or bias.dtype == x.dtype)):
        return _DotSigmoidBceFn.apply(x, weight, bias, targets, scale)
    z = F.linear(x.float(), weight.float(), None if bias is None else bias.float()).view(-1)
    return F.binary_cross_entropy_with_logits(z, targets.float(), reduction=reduction)


class _EmbedSumFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, tok, pos, typ):
        b, seq = ids.shape
        hidden = tok.shape[1]
        idc = ids.contiguous()
        x = torch.empty(b, seq, hidden, dtype=tok.dtype, device=tok.device)
        base.check(base.K().tipsk_embed_sum_fwd(idc.data_ptr(), tok.data_ptr(), pos.data_ptr(), typ.data_ptr(),
                                                x.data_ptr(), b * seq, seq, hidden, tok.shape[0], base.code(tok),
                                                base.stream()), "embed_sum_fwd")
        ctx.save_for_backward(idc)
        ctx.shapes = (tuple(tok.shape), tuple(pos.shape), tuple(typ.shape), tok.dtype)
        return x

    @staticmethod
    def backward(ctx, dx):
        (idc,) = ctx.saved_tensors
        tshape, pshape, yshape, dtype = ctx.shapes
        b, seq = idc.shape
        g = dx.contiguous()
        dtok = torch.empty(tshape, dtype=dtype, device=g.device)
        dpos = torch.zeros(pshape, dtype=dtype, device=g.device) if pshape[0] != seq else torch.empty(pshape, dtype=dtype, device=g.device)
        dtyp = torch.empty(yshape, dtype=dtype, device=g.device)
        base.check(base.K().tipsk_embed_sum_bwd(idc.data_ptr(), g.data_ptr(), dtok.data_ptr(), dpos.data_ptr(),
                                                dtyp.data_ptr(), b * seq, seq, tshape[1], tshape[0], base.code(g),
                                                base.stream()), "embed_sum_bwd")
        return None, dtok, dpos, dtyp


def embed_sum(ids, tok_weight, pos_weight, type_row):
    """``tok_weight[ids] + pos_weight[:seq] + type_row`` for ids [B, S]: the input embedding of a transformer
    encoder as one gather kernel (and three small kernels in backward); `pos_weight` has at least S rows."""
    hidden = tok_weight.shape[1]
    es = tok_weight.element_size()
    if (ids.is_cuda and tok_weight.is_cuda and tok_weight.dtype == pos_weight.dtype == type_row.dtype
            and tok_weight.dtype in (torch.bfloat16, torch.float16, torch.float32) and (hidden * es) % 16 == 0
            and tok_weight.is_contiguous() and pos_weight.is_contiguous() and type_row.is_contiguous()
            and pos_weight.shape[0] >= ids.shape[1]):
        return _EmbedSumFn.apply(ids, tok_weight, pos_weight, type_row)
    seq = ids.shape[1]
    return tok_weight[ids] + pos_weight[:seq][None] + type_row


class _SoftmaxXentFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, ignore_index):
        cols = logits.shape[-1]
        z = logits.contiguous()
        rows = z.numel() // cols
        lab = labels.contiguous().view(-1)
        acc = torch.zeros(2, dtype=torch.float32, device=z.device)
        dz = torch.empty_like(z)
        base.check(base.K().tipsk_softmax_xent(z.data_ptr(), lab.data_ptr(), acc.data_ptr(),
                                               acc.data_ptr() + 4, dz.data_ptr(), rows, cols, ignore_index, 1.0,
                                               base.code(z), base.stream()), "softmax_xent")
        inv = 1.0 / torch.clamp(acc[1], min=1.0)
        ctx.save_for_backward(dz, inv)
        return acc[0] * inv

    @staticmethod
    def backward(ctx, dloss):
        dz, inv = ctx.saved_tensors
        return dz * (dloss * inv).to(dz.dtype), None, None


def softmax_cross_entropy(logits, labels, ignore_index=-100):
    """Mean softmax cross-entropy over the rows whose label is not `ignore_index`."""
    if logits.is_cuda:
        return _SoftmaxXentFn.apply(logits, labels, ignore_index)
    return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), labels.view(-1), ignore_index=ignore_index)
