"""Gradient compression applied around an allreduce.

API parity with the reference (tips/tensorflow/compression.py:20-75): a
``Compressor`` interface with ``compress(tensor) -> (tensor, ctx)`` and
``decompress(tensor, ctx)``, ``NoneCompressor``, ``FP16Compressor`` and the
``Compression`` namespace.  ``BF16Compressor`` is added because bf16 is the
natural wire type on B200.  The engine reduces 16-bit floats with fp32
accumulation, so a compressed allreduce actually works here (the reference's
engine rejects fp16, tips/core/collective/utils.h:29-46).
"""
from __future__ import annotations

import torch


class Compressor:
    """Interface: compress before the collective, decompress after it."""

    @staticmethod
    def compress(tensor):
        raise NotImplementedError

    @staticmethod
    def decompress(tensor, ctx):
        raise NotImplementedError


class NoneCompressor(Compressor):
    @staticmethod
    def compress(tensor):
        return tensor, None

    @staticmethod
    def decompress(tensor, ctx):
        return tensor


class _CastCompressor(Compressor):
    wire = torch.float16

    @classmethod
    def compress(cls, tensor):
        if tensor.is_floating_point() and tensor.dtype != cls.wire:
            return tensor.to(cls.wire), tensor.dtype
        return tensor, None

    @classmethod
    def decompress(cls, tensor, ctx):
        return tensor.to(ctx) if ctx is not None else tensor


class FP16Compressor(_CastCompressor):
    wire = torch.float16


class BF16Compressor(_CastCompressor):
    wire = torch.bfloat16


class Compression:
    none = NoneCompressor
    fp16 = FP16Compressor
    bf16 = BF16Compressor
