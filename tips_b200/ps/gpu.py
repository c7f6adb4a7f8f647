"""GPU-resident sharded parameter-server tables.

The reference's parameter server keeps rows in host hash maps on server ranks and
moves them through an RPC (tips/core/ps/sparse_table.h:38-185, ps_server.h:147-265,
ps_client.h:78-130).  Here every rank is a server and a worker at once: a table's
row ``id`` lives at local row ``id // N`` of a slab in peer-mapped device memory on
the rank given by a rotated round-robin rule (``place``; csrc/kernels/ps_placement.h),
``pull`` is a lookup kernel that reads rows straight from the owner's HBM over NVLink,
and ``push`` sums the duplicate ids of the batch locally, stores one row per distinct
id into the owner's inbox, and the owner applies the server-side optimizer once per
touched row (csrc/kernels/ps.cu).

Rows exist from the start (a dense slab initialised to zero or to a seeded uniform),
which is what the reference's lazy zero-initialisation on first pull amounts to
(tips/core/ps/sparse_access_method.h:23-27); arbitrary 64-bit keys are served by the
host tables in tips_b200.ps.host.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..ops import base
from ..utils.trace import nvtx_range

_RULES = {"sgd": 0, "adagrad": 1, "literal_reference": 2}
_active = None


def _world():
    """(rank, size, emulated, device_state) of the GPU data plane."""
    from .. import runtime
    st = runtime.device_state()
    if st is None:
        from ..parallel import device as _device
        try:
            st = _device.state()
        except RuntimeError:
            st = None
    if st is None:
        return 0, 1, 0, None
    return (0 if st.emulated else st.rank), st.size, st.emulated, st


class ShardedEmbedding:
    """`num_fields` tables of [rows_per_table, dim] fp32, row-sharded over the ranks."""

    def __init__(self, num_fields: int, rows_per_table: int, dim: int, optimizer: str = "adagrad", lr: float = 0.01,
                 eps: float = 1e-8, init_scale: float = 0.0, seed: int = 0, slots: Optional[int] = None,
                 expected_batch: int = 8192, device=None, sync: bool = True, servers=None):
        """`servers`: the ranks that hold shards (default: every rank).  Every rank of the job may pull and push (a
        worker); only the listed ranks serve rows: the reference's split into PS_SERVER and PS_WORKER node sets, where
        a rank may be either or both (tips/core/ps/route.h:22-134).  On this transport every rank still maps a
        window of the slab's size, because the peer-mapped allocation is symmetric; only the servers' windows hold rows.

        `sync=True`: a push is the exact synchronous update (gradients of all ranks summed per row, then the
        optimizer applied once), with cross-rank fences around it.  `sync=False`: the reference's consistency model:
        pushes are applied to the owner's rows as they arrive (atomics, no fences), pulls may read rows mid-update."""
        if optimizer not in _RULES:
            raise ValueError(f"optimizer must be one of {sorted(_RULES)}")
        if dim % 4:
            raise ValueError("dim must be a multiple of 4")
        self.num_fields, self.rows, self.dim = num_fields, rows_per_table, dim
        self.rule, self.lr, self.eps = _RULES[optimizer], lr, eps
        self.sync = bool(sync)
        self.push_stream = None    # set by a trainer: embedding_lookup's backward then pushes on that stream
        self.push_inflight = None
        if not self.sync and self.rule not in (0, 1):
            raise ValueError("asynchronous pushes support the sgd and adagrad rules")
        self.rank, self.size, self.emulated, st = _world()
        self.device = device or (st.device if st is not None else torch.device("cuda", torch.cuda.current_device()))
        self.servers = sorted(set(range(self.size) if servers is None else servers))
        if not self.servers or self.servers[0] < 0 or self.servers[-1] >= self.size:
            raise ValueError("servers must be ranks of the job")
        self.nservers = len(self.servers)
        n = self.nservers   # rows are placed among the servers
        self.rows_per_shard = (rows_per_table + n - 1) // n
        field_bytes = self.rows_per_shard * dim * 4
        self.has_state = self.rule == 1
        self.field_off = [f * field_bytes for f in range(num_fields)]
        self.state_off = [(num_fields + f) * field_bytes if self.has_state else 0 for f in range(num_fields)]
        slab_bytes = field_bytes * num_fields * (2 if self.has_state else 1)
        # bf16 copy of the rows, kept current by the owner's apply pass and read by bf16 pulls: only where rows
        # cross NVLink (several ranks) and only with synchronous pushes (asynchronous ones update rows in place)
        from ..config import get_config
        self.shadow_base = slab_bytes if (self.size > 1 and self.sync and get_config().ps_bf16_shadow) else 0
        if self.shadow_base:
            slab_bytes += (field_bytes // 2) * num_fields
        if slots is None:
            slots = 1
            while slots < 2 * expected_batch * num_fields:
                slots *= 2
        self.slots = slots
        # rows one sender may send to one owner in a push: the worst case (every distinct row of a batch has the
        # same owner), so a skewed batch can never overflow an inbox
        self.inbox_cap = (expected_batch * num_fields + 1) // 2 * 2
        self.item_cap = expected_batch * num_fields   # items (sample, field) of a batch that an indexed pull can hold
        lib = base.K()
        self._alloc_bytes = (slab_bytes, int(lib.tipsk_ps_acc_bytes(slots, dim)),
                             int(lib.tipsk_ps_inbox_bytes(self.size, self.inbox_cap, dim)) if self.size > 1 else 0,
                             int(lib.tipsk_ps_ctl_bytes()))
        self._allocate(st)
        local = range(self.size) if self.emulated else [self.rank]
        for r in local:
            if r not in self.servers:
                continue
            slab = self.slabs[r] if self.emulated else self.slabs[0]
            for f in range(num_fields):
                w = slab[self.field_off[f]:self.field_off[f] + field_bytes].view(torch.float32)
                base.check(lib.tipsk_table_init(w.data_ptr(), self.rows_per_shard, dim, f, self.servers.index(r), n,
                                                rows_per_table, seed, float(init_scale), base.stream()), "table_init")
            if self.has_state:
                slab[num_fields * field_bytes:2 * num_fields * field_bytes].zero_()
        self.refresh_shadow()
        torch.cuda.synchronize()
        self._sync_ranks()
        self._configure()

    # ------------------------------------------------------------------ set-up
    def _allocate(self, st):
        """Table slab and inbox in peer-mapped memory; accumulation table, touched list and control words local."""
        n = self.size
        slab_bytes, acc_bytes, inbox_bytes, ctl_bytes = self._alloc_bytes
        nlocal = n if self.emulated else 1
        dev = self.device
        self.accs = [torch.zeros(acc_bytes, dtype=torch.uint8, device=dev) for _ in range(nlocal)]
        self.ulists = [torch.zeros(2 * self.slots, dtype=torch.int32, device=dev) for _ in range(nlocal)]
        self.ctls = [torch.zeros(ctl_bytes, dtype=torch.uint8, device=dev) for _ in range(nlocal)]
        self.item_slots = [torch.zeros(self.item_cap, dtype=torch.int32, device=dev) for _ in range(nlocal)]
        self.caches = [torch.empty(self.slots * self.dim * 4, dtype=torch.uint8, device=dev) for _ in range(nlocal)]
        if self.emulated or n == 1:
            self.slabs = [torch.empty(slab_bytes, dtype=torch.uint8, device=dev) for _ in range(nlocal)]
            self.inboxes = [torch.zeros(max(inbox_bytes, 16), dtype=torch.uint8, device=dev) for _ in range(nlocal)]
            self._slab_ptrs = [t.data_ptr() for t in self.slabs]
            self._inbox_ptrs = [t.data_ptr() for t in self.inboxes]
            return
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        group = dist.group.WORLD
        slab = symm_mem.empty(slab_bytes, dtype=torch.uint8, device=dev)
        h1 = symm_mem.rendezvous(slab, group.group_name)
        inbox = symm_mem.empty(inbox_bytes, dtype=torch.uint8, device=dev)
        h2 = symm_mem.rendezvous(inbox, group.group_name)
        inbox.zero_()
        self._handles = (h1, h2)
        self.slabs, self.inboxes = [slab], [inbox]
        self._slab_ptrs = [int(p) for p in h1.buffer_ptrs]
        self._inbox_ptrs = [int(p) for p in h2.buffer_ptrs]

    def _sync_ranks(self):
        if self.size > 1 and not self.emulated:
            from .. import runtime
            torch.cuda.synchronize()
            runtime.barrier()

    def _configure(self):
        global _active
        lib = base.K()
        n = self.size
        srv = (ctypes.c_int32 * self.nservers)(*self.servers)
        base.check(lib.tipsk_ps_configure(base.ptr_array([self._slab_ptrs[r] for r in self.servers]),
                                          base.ptr_array([self._inbox_ptrs[r] for r in self.servers]),
                                          base.ptr_array(self.accs), base.ptr_array(self.ulists),
                                          base.ptr_array(self.ctls), base.ptr_array(self.item_slots),
                                          base.ptr_array(self.caches), n, len(self.accs), srv, self.nservers,
                                          base.u64_array(self.field_off), base.u64_array(self.state_off),
                                          base.i64_array([self.rows_per_shard] * self.num_fields), self.num_fields,
                                          self.dim, self.slots, self.inbox_cap, self.item_cap, self.shadow_base),
                   "ps_configure")
        from ..config import get_config
        lib.tipsk_ps_wire_follows_grads(0 if get_config().ps_wire_dtype == "fp32" else 1)
        _active = self

    def _activate(self):
        if self.slabs is None:
            raise RuntimeError("this table was closed")
        if _active is not self:
            self._configure()

    def close(self):
        """Release the device memory of the tables (the kernel library keeps no pointer to it afterwards)."""
        global _active
        if _active is self:
            _active = None
        torch.cuda.synchronize()
        self._sync_ranks()
        self.slabs = self.inboxes = self.accs = self.ulists = self.ctls = self.item_slots = self.caches = None
        self._handles = None
        self._slab_ptrs = self._inbox_ptrs = []

    # ------------------------------------------------------------------ data path
    def _per_rank(self, tensors):
        """Per-local-rank pointer array: a list of tensors when emulated, one tensor otherwise."""
        if self.emulated:
            assert isinstance(tensors, (list, tuple)) and len(tensors) == self.size
            return base.ptr_array(list(tensors)), tensors[0]
        return base.ptr_array([tensors]), tensors

    def pull(self, ids, out=None, out_col0: int = 0, dtype=torch.bfloat16, fence: bool = True, index: bool = False):
        """Gather rows: ids [B, F] int64 -> out[:, out_col0 + f*dim : ...] (a new [B, F*dim] tensor if out is None).

        `index=True` resolves the batch into its distinct rows first and fetches each of them once (about half of a
        Zipf batch is duplicates); the index stays in place for a following ``push(ids, ..., reuse_index=True)`` of
        the same, unmodified ids, which then skips the hashing.  Any other pull or push drops it."""
        self._activate()
        ids_arr, ids0 = self._per_rank(ids)
        b = ids0.shape[0]
        if index and b * self.num_fields > self.item_cap:
            index = False  # a batch larger than announced: plain pull
        if out is None:
            mk = lambda: torch.empty(b, self.num_fields * self.dim, dtype=dtype, device=self.device)
            out = [mk() for _ in range(self.size)] if self.emulated else mk()
        out_arr, out0 = self._per_rank(out)
        with nvtx_range("tips.ps.pull"):
            base.check(base.K().tipsk_ps_pull(ids_arr, out_arr, b, out0.stride(0), out_col0, base.code(out0),
                                              int(fence and self.sync), int(index and self.sync), base.stream()),
                       "ps_pull")
        self._indexed = bool(index and self.sync)
        return out

    def push(self, ids, grads, grad_col0: int = 0, grad_scale: float = 1.0, lr: Optional[float] = None,
             reuse_index: bool = False):
        """Scatter-reduce the row gradients to their owners and apply the optimizer there."""
        self._activate()
        ids_arr, ids0 = self._per_rank(ids)
        g_arr, g0 = self._per_rank(grads)
        args = (ids_arr, g_arr, ids0.shape[0], g0.stride(0), grad_col0, base.code(g0), float(grad_scale), self.rule,
                float(self.lr if lr is None else lr), float(self.eps))
        with nvtx_range("tips.ps.push"):
            if self.sync:
                reuse = bool(reuse_index and getattr(self, "_indexed", False))
                base.check(base.K().tipsk_ps_push(*args, int(reuse), base.stream()), "ps_push")
                self._indexed = False
            else:
                base.check(base.K().tipsk_ps_push_async(*args, base.stream()), "ps_push")
        base.count_launches(1)

    def join_push(self):
        """Make the current stream wait for a push that embedding_lookup's backward put on `push_stream`."""
        if self.push_stream is not None and self.push_inflight is not None:
            torch.cuda.current_stream().wait_stream(self.push_stream)
            self.push_inflight = None

    def check(self):
        """Raise if a push overflowed the accumulation table or an id was out of range. Synchronises."""
        self._activate()
        err = ctypes.c_int32(0)
        touched = ctypes.c_uint64(0)
        base.check(base.K().tipsk_ps_status(ctypes.byref(err), ctypes.byref(touched)), "ps_status")
        if err.value == 1:
            raise RuntimeError("parameter-server push: accumulation table full; raise `slots`")
        if err.value == 2:
            raise RuntimeError("parameter-server: an id was negative or beyond the table")
        if err.value == 3:
            raise RuntimeError("parameter-server push: an owner's inbox is full; raise `expected_batch`")
        return int(touched.value)

    def traffic(self):
        """(distinct rows of the pushed batches, those that crossed NVLink to their owner, rows that indexed pulls
        read over NVLink) since the last call.  Synchronises."""
        self._activate()
        out = (ctypes.c_uint64 * 3)()
        base.check(base.K().tipsk_ps_traffic(out), "ps_traffic")
        return int(out[0]), int(out[1]), int(out[2])

    # ------------------------------------------------------------------ host views / checkpoint
    def local_shard(self, field: int, rank: Optional[int] = None, state: bool = False) -> torch.Tensor:
        """[rows_per_shard, dim] fp32 view of this rank's shard of `field` (or its Adagrad state)."""
        slab = self.slabs[rank if self.emulated else 0]
        off = (self.state_off if state else self.field_off)[field]
        nbytes = self.rows_per_shard * self.dim * 4
        return slab[off:off + nbytes].view(torch.float32).view(self.rows_per_shard, self.dim)

    def refresh_shadow(self) -> None:
        """Rebuild the bf16 copy of the rows from the fp32 rows (after rows were written from outside the push
        path: initialisation, a loaded dump, a direct edit of `local_shard`)."""
        if not self.shadow_base:
            return
        half = self.rows_per_shard * self.dim * 2
        for r in self._ranks_here():
            slab = self.slabs[r if self.emulated else 0]
            for f in range(self.num_fields):
                dst = slab[self.shadow_base + f * half:self.shadow_base + (f + 1) * half].view(torch.bfloat16)
                dst.copy_(self.local_shard(f, r).reshape(-1))

    def place(self, ids: torch.Tensor, field: int, world: Optional[int] = None):
        """(index of the owning server, local row) of the rows `ids` of `field`: the rule of
        csrc/kernels/ps_placement.h among `world` servers (default: this table's)."""
        n = self.nservers if world is None else world
        lrow = ids // n
        rot = ((((lrow & 0xFFFFFFFF) * 0x9E3779B1) & 0xFFFFFFFF) >> 16) + field
        return (ids % n + rot) % n, lrow

    def global_ids(self, field: int, rank: int, world: Optional[int] = None, rows_per_shard: Optional[int] = None,
                   device=None) -> torch.Tensor:
        """Global row id held at every local row of the shard of `field` on server number `rank` (ids >= rows are
        padding)."""
        n = self.nservers if world is None else world
        lrow = torch.arange(self.rows_per_shard if rows_per_shard is None else rows_per_shard, dtype=torch.int64,
                            device=device)
        rot = ((((lrow & 0xFFFFFFFF) * 0x9E3779B1) & 0xFFFFFFFF) >> 16) + field
        return lrow * n + (rank + n - rot % n) % n

    def dense_table(self, field: int, state: bool = False) -> torch.Tensor:
        """The whole [rows, dim] table of `field` (or its Adagrad state) assembled from the shards this process
        can see: all of them when the ranks are emulated or there is one rank (tests, small tables)."""
        assert self.emulated or self.size == 1
        out = torch.zeros(self.rows_per_shard * self.nservers, self.dim, device=self.device)
        for j, r in enumerate(self.servers):
            out[self.global_ids(field, j, device=self.device)] = self.local_shard(field, r, state=state)
        return out[:self.rows].clone()

    # ------------------------------------------------------------------ dumps
    # The reference can only dump a sparse table as text, one line per key ("<key>\tVec:\t<e> <e> ... \n",
    # tips/core/ps/sparse_table.h:86-93,147-152) and has no loader.  Here every rank writes the shards it owns
    # in a binary file (header + raw fp32 rows and optimizer state, staged through pinned host memory) that can
    # be read back under a different number of ranks, and small tables can also be written in that text format.

    def _ranks_here(self):
        """World ranks whose shards this process holds (servers only)."""
        here = range(self.size) if self.emulated else [self.rank]
        return [r for r in here if r in self.servers]

    def save(self, prefix: str) -> list:
        """Write `<prefix>.rank<r>.bin` for the shard(s) held by this process; returns the paths."""
        import json
        import numpy as np
        torch.cuda.synchronize()
        paths = []
        for r in self._ranks_here():
            path = f"{prefix}.rank{r}.bin"
            header = {"format": "tips_b200.ps.v2", "rank": self.servers.index(r), "world": self.nservers,
                      "fields": self.num_fields,
                      "rows": self.rows, "rows_per_shard": self.rows_per_shard, "dim": self.dim,
                      "state": bool(self.has_state)}
            with open(path, "wb") as f:
                hb = json.dumps(header).encode()
                f.write(np.array([len(hb)], dtype=np.uint64).tobytes())
                f.write(hb)
                for state in ([False, True] if self.has_state else [False]):
                    for fld in range(self.num_fields):
                        shard = self.local_shard(fld, r, state=state)
                        for lo in range(0, self.rows_per_shard, 1 << 20):  # at most 1M rows on the host at a time
                            f.write(shard[lo:lo + (1 << 20)].cpu().numpy().tobytes())
            paths.append(path)
        self._sync_ranks()
        return paths

    def load(self, prefix: str) -> None:
        """Read every `<prefix>.rank*.bin` written by `save` (by any number of ranks) and keep the rows this
        process owns under the current sharding (`place`)."""
        import glob
        import json
        import numpy as np
        files = sorted(glob.glob(f"{prefix}.rank*.bin"))
        if not files:
            raise FileNotFoundError(f"no table dump matches {prefix}.rank*.bin")
        seen_world = None
        for path in files:
            with open(path, "rb") as f:
                hlen = int(np.frombuffer(f.read(8), dtype=np.uint64)[0])
                h = json.loads(f.read(hlen))
                if (h["fields"], h["rows"], h["dim"]) != (self.num_fields, self.rows, self.dim):
                    raise ValueError(f"{path}: table geometry differs from this table")
                seen_world = h["world"]
                old_n, old_r, old_rows = h["world"], h["rank"], h["rows_per_shard"]
                for state in ([False, True] if h["state"] else [False]):
                    for fld in range(self.num_fields):
                        for lo in range(0, old_rows, 1 << 20):
                            cnt = min(1 << 20, old_rows - lo)
                            buf = np.frombuffer(f.read(cnt * self.dim * 4), dtype=np.float32).reshape(cnt, self.dim)
                            if state and not self.has_state:
                                continue
                            ids = self.global_ids(fld, old_r, world=old_n, rows_per_shard=old_rows)[lo:lo + cnt]
                            valid = ids < self.rows
                            owner, lrow = self.place(ids, fld)
                            for r in self._ranks_here():
                                mine = valid & (owner == self.servers.index(r))
                                if not bool(mine.any()):
                                    continue
                                rows = torch.from_numpy(buf.copy())[mine].to(self.device)
                                dst = self.local_shard(fld, r, state=state)
                                dst[lrow[mine].to(self.device)] = rows
        if seen_world is None:
            raise ValueError("empty dump")
        self.refresh_shadow()
        torch.cuda.synchronize()
        self._sync_ranks()

    def save_text(self, path: str, field: int) -> None:
        """The rows of `field` held by this process in the reference's text format (small tables, tests)."""
        torch.cuda.synchronize()
        with open(path, "w") as f:
            for r in self._ranks_here():
                shard = self.local_shard(field, r).cpu()
                keys = self.global_ids(field, self.servers.index(r)).tolist()
                for lrow in range(self.rows_per_shard):
                    if keys[lrow] >= self.rows:
                        continue
                    f.write(f"{keys[lrow]}\tVec:\t" + "".join(f"{float(v):g} " for v in shard[lrow]) + "\n")


class _LookupFn(torch.autograd.Function):
    """pull in forward; push (scatter-reduce + server-side optimizer) in backward."""

    @staticmethod
    def forward(ctx, table, ids, anchor, out, col0, grad_scale):
        # the backward pass pushes the gradients of these very ids: with several ranks the batch is resolved into its
        # distinct rows once, for the pull (each row crosses NVLink once) and for the push (no second hashing);
        # with one rank the plain lookup is as fast and needs no extra pass
        table.pull(ids, out=out, out_col0=col0, index=table.size > 1)
        ctx.table, ctx.ids, ctx.col0, ctx.grad_scale = table, ids, col0, grad_scale
        ctx.ids_version = ids._version
        ctx.mark_dirty(out)
        return out

    @staticmethod
    def backward(ctx, dout):
        g = dout if dout.stride(1) == 1 else dout.contiguous()
        table = ctx.table
        reuse = ctx.ids._version == ctx.ids_version
        side = getattr(table, "push_stream", None)
        if side is None:
            table.push(ctx.ids, g, grad_col0=ctx.col0, grad_scale=ctx.grad_scale, reuse_index=reuse)
        else:
            # the push runs beside what follows on this stream (gradient allreduce and update of the dense part);
            # the owner of `push_stream` joins it before the next pull and keeps `g` alive until then
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                table.push(ctx.ids, g, grad_col0=ctx.col0, grad_scale=ctx.grad_scale, reuse_index=reuse)
            table.push_inflight = g
        return None, None, None, None, None, None


def embedding_lookup(table: ShardedEmbedding, ids: torch.Tensor, out: torch.Tensor, col0: int = 0,
                     grad_scale: float = 1.0) -> torch.Tensor:
    """Differentiable pull into `out` (a [B, ld] buffer); the backward pass pushes the gradient."""
    anchor = torch.zeros((), device=out.device, requires_grad=True)
    return _LookupFn.apply(table, ids, anchor, out, col0, grad_scale)


class ShardedDense:
    """A dense parameter-server table on the GPUs: a vector of `size` elements whose fp32 master copy and optimizer
    state are sharded over the ranks (every rank serves 1/N of the vector), updated by the server-side rule when
    gradients are pushed, with the current values readable on every rank.

    The reference declares a range-partitioned dense table with a pull access method
    (tips/core/ps/dense_table.h:49-131, dense_access_method.h:10-25) and stops there; the host version of this
    table is ``tips_b200.ps.host.HostDenseTable``.  On the GPUs a push is ONE kernel (csrc/kernels/comm.cu,
    ``AllreduceUpdateKernel``): every rank reduces the share of the pushed gradients that it serves straight out
    of the peers' memory (NVLS ``multimem.ld_reduce`` or peer loads), applies SGD-momentum or Adam(W) to its share
    of the master weights, and stores the new values into every rank's copy, so a pull is a local read.  With one
    rank the same rule runs as the plain fused optimizer kernel.

    ``push`` is a collective: every rank calls it with its own gradient, in the same order."""

    def __init__(self, size: int, dtype=torch.bfloat16, optimizer: str = "sgd", lr: float = 0.01, momentum: float = 0.0,
                 betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0, device=None, average: bool = True):
        from .. import runtime
        from ..ops.optim import FusedAdam, FusedSGD
        if optimizer not in ("sgd", "adam", "adamw"):
            raise ValueError("optimizer must be sgd, adam or adamw")
        st = runtime.device_state() if runtime.is_initialized() else None
        self.world = runtime.size() if runtime.is_initialized() else 1
        self.device = device or (st.device if st is not None else torch.device("cuda", torch.cuda.current_device()))
        self.size, self.average = int(size), bool(average)
        self.param = torch.nn.Parameter(torch.zeros(self.size, dtype=dtype, device=self.device))
        if optimizer == "sgd":
            self.opt = FusedSGD([self.param], lr=lr, momentum=momentum, weight_decay=weight_decay,
                                bucket_bytes=1 << 62)
        else:
            from ..ops.optim import FusedAdamW
            cls = FusedAdamW if optimizer == "adamw" else FusedAdam
            self.opt = cls([self.param], lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, bucket_bytes=1 << 62)
        use_window = st is not None and st.window is not None and self.world > 1
        self._fs = self.opt.build(st if use_window else None)[0]
        self.sharded = bool(use_window and self.opt.shard_for_fused_update(st))
        if self.world > 1 and not self.sharded:
            raise RuntimeError("a dense table over several ranks needs the symmetric window of the GPU data plane")

    def pull(self, begin: int = 0, end: Optional[int] = None) -> torch.Tensor:
        """Current values of elements [begin, end): this rank's copy, which the last push brought up to date."""
        return self.param.detach()[begin:self.size if end is None else end]

    def assign(self, values: torch.Tensor) -> None:
        """Overwrite the whole vector (initial values, a restored checkpoint); every rank passes the same values."""
        with torch.no_grad():
            self.param.copy_(values.to(self.param.dtype).reshape(-1))
        self._fs.refresh_master_from_params()

    def push(self, grad: torch.Tensor, lr: Optional[float] = None) -> None:
        """Hand in this rank's gradient of the whole vector; the gradients of all ranks are summed (averaged with
        ``average=True``) and every rank's shard is updated by the table's rule."""
        if lr is not None:
            self.opt.param_groups[0]["lr"] = lr
        fs, b = self._fs, self._fs.bucket
        self.param.grad = grad.reshape(-1)
        b.pack()
        fs.grads_packed = True
        post = 1.0 / self.world if self.average else 1.0
        if self.sharded:
            self.opt.push_update_hyper(fs)
            base.check(base.K().tipsk_allreduce_update(b.win_off, post, 3, base.comm_stream()), "dense_push")
        elif post != 1.0:
            b.grad.mul_(post)
        self.opt.step()

    def state(self) -> dict:
        """Full-size master weights and optimizer state (a collective when the table is sharded)."""
        fs = self._fs
        return {"master": fs.full_master().cpu(), "steps": fs.steps,
                "state": {k: fs.full(v).cpu() for k, v in fs.state.items() if k != "step_dev"}}

    def load_state(self, saved: dict) -> None:
        """Inverse of `state`, under any number of ranks: every rank cuts its own share out."""
        fs = self._fs
        fs.steps = int(saved["steps"])
        fs.load_master(saved["master"].to(self.device))
        for k, v in saved["state"].items():
            fs.load_state(k, v.to(self.device))


class HashedEmbedding:
    """A sparse table keyed by ARBITRARY 64-bit ids whose rows come into existence (as zeros) the first time they
    are pulled: the reference's sparse-table semantics (tips/core/ps/access_method.h:90-99,
    sparse_access_method.h:23-27, sparse_table.h:164-165) on the GPUs.

    Every rank owns an open-addressing table of `capacity_per_rank` slots in peer-mapped memory; the owner of a key
    is a hash of it.  ``pull`` finds or claims the slot on the owner (system-scope CAS over NVLink, bounded probing)
    and reads the row; ``push`` applies SGD or Adagrad to the owner's row with vector atomics as gradients arrive,
    the reference's consistency model (servers apply pushes in arrival order, ps_server.h:248-264), and reports how
    many pushed rows had never been pulled.  ``ShardedEmbedding`` is the table for dense id ranges with the exact
    synchronous update; the host tables in ``tips_b200.ps.host`` serve the same keys from CPU memory."""

    def __init__(self, dim: int, capacity_per_rank: int, optimizer: str = "sgd", lr: float = 0.01, eps: float = 1e-8,
                 device=None):
        if optimizer not in ("sgd", "adagrad"):
            raise ValueError("optimizer must be sgd or adagrad")
        if dim % 4:
            raise ValueError("dim must be a multiple of 4")
        self.rank, self.size, self.emulated, st = _world()
        self.device = device or (st.device if st is not None else torch.device("cuda", torch.cuda.current_device()))
        self.dim, self.lr, self.eps = dim, lr, eps
        self.rule = 1 if optimizer == "adagrad" else 0
        cap = 2
        while cap < capacity_per_rank:
            cap *= 2
        self.cap = cap
        sizes = [cap * 8, cap * dim * 4, cap * dim * 4 if self.rule == 1 else 0]
        nlocal = self.size if self.emulated else 1
        if self.emulated or self.size == 1:
            bufs = [[torch.zeros(max(sz, 16), dtype=torch.uint8, device=self.device) for _ in range(nlocal)] for sz in sizes]
            ptrs = [[t.data_ptr() for t in group] for group in bufs]
        else:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem
            bufs, ptrs, self._handles = [], [], []
            for sz in sizes:
                t = symm_mem.empty(max(sz, 16), dtype=torch.uint8, device=self.device)
                h = symm_mem.rendezvous(t, dist.group.WORLD.group_name)
                t.zero_()
                bufs.append([t])
                ptrs.append([int(p) for p in h.buffer_ptrs])
                self._handles.append(h)
        self._bufs = bufs
        self._keys, self._rows = ptrs[0], ptrs[1]
        self._state = ptrs[2] if self.rule == 1 else None
        self._error = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._missing = torch.zeros(1, dtype=torch.int64, device=self.device)
        torch.cuda.synchronize()
        if self.size > 1 and not self.emulated:
            from .. import runtime
            runtime.barrier()

    def _per_rank(self, tensors):
        if self.emulated:
            assert isinstance(tensors, (list, tuple)) and len(tensors) == self.size
            return base.ptr_array(list(tensors)), tensors[0], len(tensors)
        return base.ptr_array([tensors]), tensors, 1

    def pull(self, keys, dtype=torch.float32, fence: bool = False):
        """keys [B] int64 (any bit pattern except -1) -> [B, dim]; unknown keys become zero rows on their owner."""
        k_arr, k0, nlocal = self._per_rank(keys)
        mk = lambda: torch.empty(k0.numel(), self.dim, dtype=dtype, device=self.device)
        out = [mk() for _ in range(self.size)] if self.emulated else mk()
        o_arr, o0, _ = self._per_rank(out)
        if fence:
            base.check(base.K().tipsk_comm_fence(2, base.stream()), "fence")
        base.check(base.K().tipsk_hash_pull(base.ptr_array(self._keys), base.ptr_array(self._rows), self.size, self.cap,
                                            self.dim, k_arr, o_arr, nlocal, k0.numel(), o0.stride(0), base.code(o0),
                                            self._error.data_ptr(), base.stream()), "hash_pull")
        return out

    def push(self, keys, grads, grad_scale: float = 1.0, lr: Optional[float] = None) -> None:
        k_arr, k0, nlocal = self._per_rank(keys)
        g_arr, g0, _ = self._per_rank(grads)
        base.check(base.K().tipsk_hash_push(base.ptr_array(self._keys), base.ptr_array(self._rows),
                                            base.ptr_array(self._state) if self._state else None, self.size, self.cap,
                                            self.dim, k_arr, g_arr, nlocal, k0.numel(), g0.stride(0), base.code(g0),
                                            float(grad_scale), self.rule, float(self.lr if lr is None else lr),
                                            float(self.eps), self._error.data_ptr(), self._missing.data_ptr(),
                                            base.stream()), "hash_push")

    def check(self) -> int:
        """Raise if a table filled up; returns (and clears) the number of pushed rows that had never been pulled."""
        err, missing = int(self._error.item()), int(self._missing.item())
        self._error.zero_()
        self._missing.zero_()
        if err == 1:
            raise RuntimeError("hashed table: an owner's table is full; raise capacity_per_rank")
        if err == 2:
            raise RuntimeError("hashed table: the key 2**64 - 1 cannot be stored")
        return missing

    def local_size(self, rank: Optional[int] = None) -> int:
        """Rows that exist on this rank (emulated: on `rank`)."""
        keys = self._bufs[0][rank if self.emulated else 0]
        return int((keys.view(torch.int64) != 0).sum().item())
