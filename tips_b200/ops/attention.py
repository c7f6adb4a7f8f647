"""Self-attention on a packed QKV projection without layout glue.

``packed_attention(qkv, heads)`` takes the output of the fused QKV linear layer, ``[batch, seq, 3 * hidden]``, and
returns ``[batch, seq, hidden]``.  The attention itself is the library's fused scaled-dot-product attention (the
reference has no attention at all; its models are TensorFlow's), but everything around it is done here so that
no tensor is re-laid by generic strided copies: q, k and v are strided views of the packed tensor, the output and
the incoming gradient change layout with one vectorised pass of ``tipsk_copy4d`` each, and the three gradients
are written straight into one packed ``[batch, seq, 3, heads, d]`` buffer (instead of three zero-filled tensors that
autograd then sums).
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import base


def copy4d(src: torch.Tensor, dst: torch.Tensor) -> None:
    """dst[...] = src[...] for 4-D tensors of equal shape whose last axis is contiguous on both sides."""
    assert src.shape == dst.shape and src.dim() == 4 and src.dtype == dst.dtype
    assert src.stride(3) == 1 and dst.stride(3) == 1
    es = src.element_size()
    n0, n1, n2, d = src.shape
    ss = (ctypes.c_int64 * 3)(*(src.stride(i) * es for i in range(3)))
    ds = (ctypes.c_int64 * 3)(*(dst.stride(i) * es for i in range(3)))
    base.check(base.K().tipsk_copy4d(src.data_ptr(), dst.data_ptr(), n0, n1, n2, d * es, ss, ds, base.stream()),
               "copy4d")


def _fast_ok(t: torch.Tensor, d: int) -> bool:
    return t.is_cuda and t.dtype in (torch.bfloat16, torch.float16) and (d * t.element_size()) % 16 == 0


class _PackedAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, heads, causal):
        b, s, three_h = qkv.shape
        h = three_h // 3
        d = h // heads
        packed = qkv.detach().view(b, s, 3, heads, d)
        with torch.enable_grad():
            q, k, v = (packed[:, :, i].transpose(1, 2).requires_grad_() for i in range(3))  # [b, heads, s, d] views
            out = F.scaled_dot_product_attention(q, k, v, is_causal=causal)
        ctx.graph = (q, k, v, out)
        ctx.geom = (b, s, heads, d)
        o = out.detach()
        if o.transpose(1, 2).is_contiguous():  # the library kept the [b, s, heads, d] memory order of the inputs
            return o.transpose(1, 2).reshape(b, s, h)
        y = torch.empty(b, s, heads, d, dtype=o.dtype, device=o.device)
        copy4d(o.transpose(1, 2), y)
        return y.view(b, s, h)

    @staticmethod
    def backward(ctx, dy):
        q, k, v, out = ctx.graph
        b, s, heads, d = ctx.geom
        ctx.graph = None
        dyv = dy.reshape(b, s, heads, d)
        if out.transpose(1, 2).is_contiguous():
            dout = dyv.transpose(1, 2)  # same memory order as `out`
        else:
            dout = torch.empty(b, heads, s, d, dtype=dy.dtype, device=dy.device)
            copy4d(dyv.transpose(1, 2), dout)
        dq, dk, dv = torch.autograd.grad(out, (q, k, v), dout)
        dqkv = torch.empty(b, s, 3, heads, d, dtype=dy.dtype, device=dy.device)
        for i, g in enumerate((dq, dk, dv)):
            copy4d(g.transpose(1, 2), dqkv[:, :, i])  # [b, s, heads, d] view of the gradient -> its packed slot
        return dqkv.view(b, s, 3 * heads * d), None, None


def packed_attention(qkv: torch.Tensor, heads: int, causal: bool = False) -> torch.Tensor:
    """Multi-head self-attention on ``qkv = [batch, seq, 3 * hidden]`` (q, k, v concatenated on the last axis)."""
    b, s, three_h = qkv.shape
    d = three_h // 3 // heads
    if _fast_ok(qkv, d) and qkv.is_contiguous():
        return _PackedAttentionFn.apply(qkv, heads, causal)
    q, k, v = qkv.view(b, s, 3, heads, d).permute(2, 0, 3, 1, 4)
    att = F.scaled_dot_product_attention(q, k, v, is_causal=causal)
    return att.transpose(1, 2).reshape(b, s, three_h // 3)
