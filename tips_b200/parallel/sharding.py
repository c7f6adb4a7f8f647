"""Which part of a flat bucket each rank owns when the optimizer step runs inside the allreduce kernel.

The fused kernel (csrc/kernels/comm.cu, ``AllreduceUpdateKernel``) cuts a bucket into 16-byte vectors and the
vectors into tiles of ``subtile * nranks``; rank r owns sub-tile r of every tile and keeps the fp32 master
weights and optimizer state of those vectors only, packed densely in tile order.  ``ShardLayout`` is the same
arithmetic on the host: it cuts a full flat tensor into a rank's share and reassembles the shares, which is what
checkpoints and state broadcasts need (they always see full-size tensors, whatever the number of ranks).

The reference keeps optimizer state inside TensorFlow and replicates it on every rank
(tips/tensorflow/__init__.py:252-456); a sharded state has no counterpart there.
"""
from __future__ import annotations

import torch


class ShardLayout:
    def __init__(self, numel: int, elem_size: int, nranks: int, subtile: int):
        if 16 % elem_size:
            raise ValueError("element size must divide 16 bytes")
        self.per_vec = 16 // elem_size
        if numel % self.per_vec:
            raise ValueError("the bucket must be a whole number of 16-byte vectors")
        self.numel = numel
        self.nranks = nranks
        self.subtile = subtile
        nvec = numel // self.per_vec
        tile = subtile * nranks
        self.ntiles = (nvec + tile - 1) // tile
        self.shard_numel = self.ntiles * subtile * self.per_vec
        self.padded_numel = self.shard_numel * nranks

    def take(self, full: torch.Tensor, rank: int) -> torch.Tensor:
        """The share of `full` ([numel]) that `rank` owns, as a new [shard_numel] tensor (zero padded)."""
        if full.numel() != self.numel:
            raise ValueError(f"expected {self.numel} elements, got {full.numel()}")
        pad = full.new_zeros(self.padded_numel)
        pad[:self.numel] = full.reshape(-1)
        return pad.view(self.ntiles, self.nranks, self.subtile * self.per_vec)[:, rank].reshape(-1).clone()

    def assemble(self, shards: torch.Tensor) -> torch.Tensor:
        """Inverse of `take`: `shards` is [nranks, shard_numel] (or flat, rank-major); returns [numel]."""
        s = shards.reshape(self.nranks, self.ntiles, self.subtile * self.per_vec)
        return s.permute(1, 0, 2).reshape(-1)[:self.numel].clone()
