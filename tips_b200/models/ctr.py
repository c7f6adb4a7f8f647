"""CTR model trained in parameter-server mode: sparse fields looked up in sharded
embedding tables (pull), concatenated with dense features, an MLP with a sigmoid
output, binary cross-entropy; the embedding gradients are pushed back and applied
on the owning rank by the server-side optimizer, the MLP is data-parallel.

This is the workload the reference's parameter server targets (PsClient pull /
push of sparse rows with a server-side update rule, tips/core/ps/ps_client.h:78-130,
sparse_access_method.h:41-61); the reference ships no model for it.
"""
from __future__ import annotations

import torch
import torch.nn as nn

import tips_b200 as tips
from ..ops.linear import Linear
from ..ops.optim import FusedAdam
from ..ops.pointwise import linear1_sigmoid_bce_loss, sigmoid_bce_loss
from ..ps.gpu import ShardedEmbedding, embedding_lookup


def synthetic_ctr_batch(batch: int, fields: int, rows: int, dense_features: int, seed: int, alpha: float = 1.05):
    """ids [B, F] ~ bounded Zipf(alpha) over [0, rows), dense ~ N(0,1), labels ~ Bernoulli(0.25)."""
    g = torch.Generator().manual_seed(seed)
    u = torch.rand(batch, fields, generator=g, dtype=torch.float64)
    e = 1.0 - alpha
    x = ((float(rows) ** e - 1.0) * u + 1.0) ** (1.0 / e)  # inverse CDF of p(x) ~ x^-alpha on [1, rows]
    ids = (x.floor().to(torch.int64) - 1).clamp_(0, rows - 1)
    dense = torch.randn(batch, dense_features, generator=g).to(torch.bfloat16)
    labels = (torch.rand(batch, generator=g) < 0.25).to(torch.float32)
    return ids, dense, labels


class CtrMLP(nn.Module):
    def __init__(self, in_features: int, hidden=(512, 256)):
        super().__init__()
        dims = [in_features] + list(hidden)
        self.layers = nn.ModuleList([Linear(dims[i], dims[i + 1], act="relu") for i in range(len(hidden))])
        self.out = Linear(dims[-1], 1)

    def hidden(self, x):
        for layer in self.layers:
            x = layer(x)
        return x

    def forward(self, x):
        return self.out(self.hidden(x))

    def loss(self, x, labels):
        """Mean binary cross-entropy; the one-unit output layer and the loss run as one streaming op."""
        return linear1_sigmoid_bce_loss(self.hidden(x), self.out.weight, self.out.bias, labels)


class CtrTrainer:
    """Owns the tables, the MLP and both optimizers; `train_step` is one synchronous PS step.

    With ``graph=True`` the whole step (pull, MLP forward/backward on the tcgen05 GEMM, push with the
    server-side Adagrad, the in-place NVLink allreduce of the MLP gradients and the fused Adam update) is
    captured once in a CUDA graph and replayed, which removes the per-launch host cost of a step that is
    otherwise launch-bound.  Every rank replays the same graph, so the collective kernels meet in the same
    order without any negotiation.
    """

    def __init__(self, num_fields=26, rows_per_table=10_000_000, dim=64, dense_features=13, hidden=(512, 256),
                 table_lr=0.05, mlp_lr=1e-3, device=None, expected_batch=8192, seed=0, graph=False, sync_ps=True,
                 overlap_push=True):
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.fields, self.dim, self.dense = num_fields, dim, dense_features
        self.emb_cols = num_fields * dim
        # padded to a multiple of 64 columns (zero-filled): the weight-gradient kernel contracts 64-channel boxes
        self.in_features = (self.emb_cols + dense_features + 63) // 64 * 64
        self.tables = ShardedEmbedding(num_fields, rows_per_table, dim, optimizer="adagrad", lr=table_lr,
                                       init_scale=0.05, seed=seed, expected_batch=expected_batch, device=self.device,
                                       sync=sync_ps)
        # the push of the embedding gradients runs beside the allreduce and the update of the MLP
        self.tables.push_stream = torch.cuda.Stream(device=self.device) if overlap_push else None
        torch.manual_seed(seed + 17)
        self.mlp = CtrMLP(self.in_features, hidden).to(self.device).to(torch.bfloat16)
        self.world = tips.size() if tips.is_initialized() else 1
        self.graph = bool(graph)
        self._x = None
        self._g = None
        self._static = None
        self._calls = 0
        if self.graph:
            self.opt = FusedAdam(self.mlp.parameters(), lr=mlp_lr, weight_decay=0.0, capturable=True)
            st = tips.runtime.device_state() if tips.is_initialized() else None
            self.opt.build(st)
            self._dev_state = st
        else:
            opt = FusedAdam(self.mlp.parameters(), lr=mlp_lr, weight_decay=0.0)
            self.opt = tips.DistributedOptimizer(opt) if tips.is_initialized() else opt
        if tips.is_initialized() and tips.size() > 1:
            tips.broadcast_parameters(self.mlp.state_dict(), root_rank=0, optimizer=None if self.graph else self.opt)
            if self.graph:  # the flat master copies follow the broadcast parameters
                for fs in self.opt.build():
                    if fs.low:
                        fs.master.copy_(fs.flat_param)

    def _input_buffer(self, batch):
        if self._x is None or self._x.shape[0] != batch:
            self._x = torch.zeros(batch, self.in_features, dtype=torch.bfloat16, device=self.device)
        return self._x

    def _features(self, ids, dense):
        x = self._input_buffer(ids.shape[0]).detach()
        x[:, self.emb_cols:self.emb_cols + self.dense] = dense
        return embedding_lookup(self.tables, ids, x, col0=0, grad_scale=1.0 / self.world)

    def forward(self, ids, dense):
        """Click logits [B]."""
        return self.mlp(self._features(ids, dense)).view(-1)

    def _allreduce_inline(self):
        """Graph mode: pack every bucket and average it over the ranks in place, on the current stream."""
        from ..ops import base
        for fs in self.opt.build():
            b = fs.bucket
            b.pack()
            if self.world > 1:
                nbytes = b.numel * b.grad.element_size()
                base.check(base.K().tipsk_allreduce(None, None, b.win_off, nbytes, base.code(b.grad), 0, 1.0,
                                                    1.0 / self.world, 3, base.comm_stream()), "allreduce")
            fs.grads_packed = True

    def _step_impl(self, ids, dense, labels):
        loss = self.mlp.loss(self._features(ids, dense), labels)
        loss.backward()
        if self.graph:
            self._allreduce_inline()
        self.opt.step()
        self.tables.join_push()
        return loss.detach()

    def train_step(self, ids, dense, labels):
        if not self.graph:
            return self._step_impl(ids, dense, labels)
        if self._static is None:
            self._static = [torch.empty_like(ids), torch.empty_like(dense), torch.empty_like(labels)]
        for dst, src in zip(self._static, (ids, dense, labels)):
            dst.copy_(src, non_blocking=True)
        if self._g is None:
            self._calls += 1
            if self._calls <= 3:  # eager warm-up: lazy initialisation, kernel attributes, optimizer state
                return self._step_impl(*self._static)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._loss_static = self._step_impl(*self._static)
            self._g = g
        self._g.replay()
        return self._loss_static

    def close(self):
        """Release the tables and the captured graph."""
        self._g = None
        self._loss_static = None
        self.tables.close()

    def check(self):
        from ..ops.linear import gemm_status
        self.tables.check()
        if gemm_status() != 0:
            raise RuntimeError("a GEMM launch reported a bounded-wait timeout")
        st = tips.runtime.device_state() if tips.is_initialized() else None
        if st is not None and st.window is not None:
            st.check_status()


def smoke_step(device):
    """Tiny PS step used by the smoke test: 4 fields x 1000 rows x dim 16."""
    t = CtrTrainer(num_fields=4, rows_per_table=1000, dim=16, dense_features=5, hidden=(64, 32), device=device,
                   expected_batch=256)
    ids, dense, labels = synthetic_ctr_batch(256, 4, 1000, 5, seed=1)
    l0 = t.train_step(ids.to(device), dense.to(device), labels.to(device)).item()
    l1 = t.train_step(ids.to(device), dense.to(device), labels.to(device)).item()
    t.check()
    assert l0 == l0 and l1 == l1
    return l0, l1
