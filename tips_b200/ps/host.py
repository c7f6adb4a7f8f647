"""Host parameter server: sparse tables of arbitrary 64-bit keys served by CPU shard threads.

Python binding of the native host PS (csrc/ps): the counterpart of the reference's
PsServer / PsClient / SparseTable / Route, which the reference never exposed to
Python (they are driven only from C++ tests, tips/core/ps/ps_server_test.cc:55-131,
ps_client_test.cc:11-85).  Rows are created on first pull and zero-initialised; a
push applies the server-side update rule on the row's owning shard thread.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_double, c_int, c_int64, c_uint64, c_void_p
from typing import Optional, Sequence

import numpy as np

from .. import _lib
from ..runtime import TipsError, _require_init, barrier

_RULES = {"sgd": 0, "adagrad": 1, "literal_reference": 2}
_NP2CODE = {np.dtype(np.float32): 0, np.dtype(np.float64): 1, np.dtype(np.int32): 2, np.dtype(np.int64): 3}
_declared = False


def _lib_ps():
    global _declared
    lib = _lib.core()
    if not _declared:
        lib.tips_ps_last_error.restype = c_char_p
        lib.tips_ps_table_create.restype = c_int64
        lib.tips_ps_table_create.argtypes = [c_char_p, POINTER(c_int), c_int, c_int, c_int, c_double, c_double]
        lib.tips_ps_table_destroy.argtypes = [c_int64]
        lib.tips_ps_pull.argtypes = [c_int64, POINTER(c_uint64), c_int64, c_int, c_int, c_void_p, c_int]
        lib.tips_ps_push.restype = c_int64
        lib.tips_ps_push.argtypes = [c_int64, POINTER(c_uint64), c_int64, c_int, c_int, c_void_p, c_int]
        lib.tips_ps_pull_async.restype = c_int64
        lib.tips_ps_pull_async.argtypes = [c_int64, POINTER(c_uint64), c_int64, c_int, c_int, c_void_p]
        lib.tips_ps_push_async.restype = c_int64
        lib.tips_ps_push_async.argtypes = [c_int64, POINTER(c_uint64), c_int64, c_int, c_int, c_void_p]
        lib.tips_ps_wait.restype = c_int64
        lib.tips_ps_wait.argtypes = [c_int64, c_int]
        lib.tips_ps_cancel.argtypes = [c_int64]
        lib.tips_ps_table_size.restype = c_int64
        lib.tips_ps_table_size.argtypes = [c_int64]
        lib.tips_ps_table_server_of.argtypes = [c_int64, c_uint64]
        lib.tips_ps_table_save.argtypes = [c_int64, c_char_p, c_int]
        lib.tips_ps_table_load.argtypes = [c_int64, c_char_p, c_int, c_int]
        lib.tips_ps_server_counters.argtypes = [c_int64, POINTER(c_uint64), POINTER(c_uint64)]
        lib.tips_ps_dense_create.restype = c_int64
        lib.tips_ps_dense_create.argtypes = [c_char_p, POINTER(c_int), c_int, c_int, c_int64, c_int, c_double, c_double]
        lib.tips_ps_dense_destroy.argtypes = [c_int64]
        lib.tips_ps_dense_pull.argtypes = [c_int64, c_int64, c_int64, c_void_p, c_int]
        lib.tips_ps_dense_push.argtypes = [c_int64, c_int64, c_int64, c_void_p, c_int, c_int]
        lib.tips_ps_dense_local.argtypes = [c_int64, POINTER(c_int64), POINTER(c_double)]
        lib.tips_ps_dense_save.argtypes = [c_int64, c_char_p]
        lib.tips_ps_dense_load.argtypes = [c_int64, c_char_p]
        lib.tips_ps_dense_counters.argtypes = [c_int64, POINTER(c_uint64), POINTER(c_uint64)]
        _declared = True
    return lib


class Route:
    """Which ranks are parameter servers and which are workers (a rank may be both)."""

    def __init__(self, servers: Optional[Sequence[int]] = None, workers: Optional[Sequence[int]] = None):
        _require_init()
        n = _lib.core().tips_size()
        self.servers = sorted(set(range(n) if servers is None else servers))
        self.workers = sorted(set(range(n) if workers is None else workers))
        me = _lib.core().tips_rank()
        self.is_server = me in self.servers
        self.is_worker = me in self.workers


class PsCall:
    """A pull or push in flight (``HostSparseTable.pull_async`` / ``push_async``).  ``wait()`` returns the pulled rows
    or, for a push, the number of rows that did not exist; ``done()`` polls.  The reference's client is asynchronous
    in the same way, with a completion callback per request (tips/core/ps/ps_client.h:78-176)."""

    def __init__(self, handle: int, out, default_timeout_ms: int):
        self._handle = handle
        self._out = out               # pull: the array the answers are written into; kept alive until the call ends
        self._timeout_ms = default_timeout_ms
        self._result = None

    def _finish(self, rc: int):
        self._handle = 0
        if rc < 0:
            raise TipsError("ps call: " + _lib_ps().tips_ps_last_error().decode(), int(-rc))
        self._result = self._out if self._out is not None else int(rc)
        return self._result

    def done(self) -> bool:
        if not self._handle:
            return True
        rc = _lib_ps().tips_ps_wait(self._handle, 0)
        if rc == -5:                  # still running
            return False
        self._finish(rc)
        return True

    def wait(self, timeout_s: Optional[float] = None):
        if not self._handle:
            return self._result
        ms = self._timeout_ms if timeout_s is None else int(timeout_s * 1000)
        rc = _lib_ps().tips_ps_wait(self._handle, ms)
        if rc == -5:
            raise TipsError("ps call timed out (it is still running; wait again or cancel())", 5)
        return self._finish(rc)

    def cancel(self) -> None:
        if self._handle:
            _lib_ps().tips_ps_cancel(self._handle)
            self._handle = 0

    def __del__(self):
        try:
            self.cancel()
        except Exception:
            pass


class HostSparseTable:
    """A sparse table [key -> row of `dim` elements] sharded over the server ranks by a hash of the key."""

    def __init__(self, name: str, dim: int, route: Optional[Route] = None, optimizer: str = "sgd", lr: float = 0.01,
                 eps: float = 1e-8, dtype=np.float32, local_shards: int = 1, timeout_s: float = 60.0):
        _require_init()
        if optimizer not in _RULES:
            raise ValueError(f"optimizer must be one of {sorted(_RULES)}")
        self.route = route or Route()
        self.name, self.dim = name, int(dim)
        self.dtype = np.dtype(dtype)
        self.timeout_ms = int(timeout_s * 1000)
        lib = _lib_ps()
        servers = (c_int * len(self.route.servers))(*self.route.servers)
        self._id = lib.tips_ps_table_create(name.encode(), servers, len(self.route.servers), local_shards,
                                            _RULES[optimizer], lr, eps)
        if self._id < 0:
            raise TipsError("ps table create: " + lib.tips_ps_last_error().decode(), int(-self._id))
        barrier()  # every rank has registered the services

    def _keys(self, keys):
        k = np.ascontiguousarray(np.asarray(keys, dtype=np.uint64).reshape(-1))
        return k, k.ctypes.data_as(POINTER(c_uint64))

    def pull(self, keys) -> np.ndarray:
        """Rows of `keys` as an [n, dim] array; unknown keys are created as zeros on their server."""
        lib = _lib_ps()
        k, kp = self._keys(keys)
        out = np.empty((k.size, self.dim), dtype=self.dtype)
        rc = lib.tips_ps_pull(self._id, kp, k.size, _NP2CODE[self.dtype], self.dim, out.ctypes.data, self.timeout_ms)
        if rc < 0:
            raise TipsError("ps pull: " + lib.tips_ps_last_error().decode(), -rc)
        return out

    def push(self, keys, grads) -> int:
        """Send one gradient row per key; returns how many rows did not exist on their server."""
        lib = _lib_ps()
        k, kp = self._keys(keys)
        g = np.ascontiguousarray(np.asarray(grads, dtype=self.dtype).reshape(k.size, self.dim))
        rc = lib.tips_ps_push(self._id, kp, k.size, _NP2CODE[self.dtype], self.dim, g.ctypes.data, self.timeout_ms)
        if rc < 0:
            raise TipsError("ps push: " + lib.tips_ps_last_error().decode(), int(-rc))
        return int(rc)

    def pull_async(self, keys) -> PsCall:
        """Start a pull and return at once; ``.wait()`` gives the [n, dim] rows.  Lets the rows of the next batch
        travel while the current one is being computed."""
        lib = _lib_ps()
        k, kp = self._keys(keys)
        out = np.empty((k.size, self.dim), dtype=self.dtype)
        h = lib.tips_ps_pull_async(self._id, kp, k.size, _NP2CODE[self.dtype], self.dim, out.ctypes.data)
        if h <= 0:
            raise TipsError("ps pull: " + lib.tips_ps_last_error().decode(), int(-h))
        return PsCall(h, out, self.timeout_ms)

    def push_async(self, keys, grads) -> PsCall:
        """Start a push and return at once (the gradients are copied into the requests before this returns);
        ``.wait()`` gives the number of rows that did not exist on their server."""
        lib = _lib_ps()
        k, kp = self._keys(keys)
        g = np.ascontiguousarray(np.asarray(grads, dtype=self.dtype).reshape(k.size, self.dim))
        h = lib.tips_ps_push_async(self._id, kp, k.size, _NP2CODE[self.dtype], self.dim, g.ctypes.data)
        if h <= 0:
            raise TipsError("ps push: " + lib.tips_ps_last_error().decode(), int(-h))
        return PsCall(h, None, self.timeout_ms)

    def local_size(self) -> int:
        return int(_lib_ps().tips_ps_table_size(self._id))

    def server_of(self, key: int) -> int:
        return int(_lib_ps().tips_ps_table_server_of(self._id, int(key)))

    def save(self, path: str, binary: bool = False) -> None:
        """Dump this rank's shards: text ("<key>\\tVec:\\t<e> <e> ... " per line) or binary."""
        lib = _lib_ps()
        if lib.tips_ps_table_save(self._id, path.encode(), int(binary)) != 0:
            raise TipsError("ps save: " + lib.tips_ps_last_error().decode())

    def load(self, path: str, binary: bool = False) -> None:
        """Load rows from a dump; only rows owned by this rank under the current sharding are kept,
        so a dump written with one number of servers can be read with another."""
        lib = _lib_ps()
        if lib.tips_ps_table_load(self._id, path.encode(), int(binary), _NP2CODE[self.dtype]) != 0:
            raise TipsError("ps load: " + lib.tips_ps_last_error().decode())

    def counters(self):
        a, b = c_uint64(0), c_uint64(0)
        _lib_ps().tips_ps_server_counters(self._id, ctypes.byref(a), ctypes.byref(b))
        return {"rows_pulled": a.value, "rows_pushed": b.value}

    def close(self):
        if self._id > 0:
            barrier()
            _lib_ps().tips_ps_table_destroy(self._id)
            self._id = -1


class HostDenseTable:
    """A dense fp32 vector of `size` elements, range-partitioned over the server ranks' shards; pulled and pushed
    by index range, the update rule applied by the owning shard's thread (csrc/ps/dense_server.h).

    The reference declares this table (range partition, Lookup, ForEach, Load/Save and a pull access method,
    tips/core/ps/dense_table.h:49-131, dense_access_method.h:10-25) but neither builds nor serves it."""

    def __init__(self, name: str, size: int, route: Optional[Route] = None, optimizer: str = "sgd", lr: float = 0.01,
                 eps: float = 1e-8, local_shards: int = 1, timeout_s: float = 60.0):
        _require_init()
        if optimizer not in _RULES:
            raise ValueError(f"optimizer must be one of {sorted(_RULES)}")
        self.route = route or Route()
        self.name, self.size = name, int(size)
        self.timeout_ms = int(timeout_s * 1000)
        lib = _lib_ps()
        servers = (c_int * len(self.route.servers))(*self.route.servers)
        self._id = lib.tips_ps_dense_create(name.encode(), servers, len(self.route.servers), local_shards, self.size,
                                            _RULES[optimizer], lr, eps)
        if self._id < 0:
            raise TipsError("dense ps table create: " + lib.tips_ps_last_error().decode(), int(-self._id))
        barrier()

    def _range(self, begin, end):
        end = self.size if end is None else end
        if not 0 <= begin <= end <= self.size:
            raise ValueError(f"range [{begin}, {end}) is outside the table of {self.size} elements")
        return begin, end

    def pull(self, begin: int = 0, end: Optional[int] = None) -> np.ndarray:
        lib = _lib_ps()
        begin, end = self._range(begin, end)
        out = np.empty(end - begin, dtype=np.float32)
        rc = lib.tips_ps_dense_pull(self._id, begin, end, out.ctypes.data, self.timeout_ms)
        if rc < 0:
            raise TipsError("dense pull: " + lib.tips_ps_last_error().decode(), -rc)
        return out

    def _push(self, values, begin, op):
        lib = _lib_ps()
        v = np.ascontiguousarray(np.asarray(values, dtype=np.float32).reshape(-1))
        begin, end = self._range(begin, begin + v.size)
        rc = lib.tips_ps_dense_push(self._id, begin, end, v.ctypes.data, op, self.timeout_ms)
        if rc < 0:
            raise TipsError("dense push: " + lib.tips_ps_last_error().decode(), -rc)

    def push(self, grads, begin: int = 0) -> None:
        """Send the gradient of elements [begin, begin + len(grads)); the owning shards apply the update rule."""
        self._push(grads, begin, 0)

    def assign(self, values, begin: int = 0) -> None:
        """Overwrite elements [begin, begin + len(values)) (initial values, checkpoint restore)."""
        self._push(values, begin, 1)

    def local_count_and_sum(self):
        """(number of elements stored on this rank, their sum), computed shard-parallel on the server threads."""
        n, s = c_int64(0), c_double(0)
        _lib_ps().tips_ps_dense_local(self._id, ctypes.byref(n), ctypes.byref(s))
        return int(n.value), float(s.value)

    def save(self, path: str) -> None:
        lib = _lib_ps()
        if lib.tips_ps_dense_save(self._id, path.encode()) != 0:
            raise TipsError("dense save: " + lib.tips_ps_last_error().decode())

    def load(self, path: str) -> None:
        """Read a dump written by any rank under any sharding; elements this rank owns now are kept."""
        lib = _lib_ps()
        if lib.tips_ps_dense_load(self._id, path.encode()) != 0:
            raise TipsError("dense load: " + lib.tips_ps_last_error().decode())

    def counters(self):
        a, b = c_uint64(0), c_uint64(0)
        _lib_ps().tips_ps_dense_counters(self._id, ctypes.byref(a), ctypes.byref(b))
        return {"elements_pulled": a.value, "elements_pushed": b.value}

    def close(self):
        if self._id > 0:
            barrier()
            _lib_ps().tips_ps_dense_destroy(self._id)
            self._id = -1


# --------------------------------------------------------------------------------------------------------------
# The sparse table as a layer of a torch model on CPU ranks: pull in forward, push in backward.

def field_keys(ids, num_fields: int):
    """64-bit table keys of a [batch, num_fields] matrix of per-field ids: the field number in the top 24 bits."""
    import torch
    if ids.dim() != 2 or ids.shape[1] != num_fields:
        raise ValueError(f"ids must be [batch, {num_fields}]")
    return (torch.arange(num_fields, dtype=torch.int64).unsqueeze(0) << 40) | ids.to(torch.int64)


class _HostLookupFn:
    """Built lazily so that importing this module does not import torch."""
    fn = None

    @classmethod
    def get(cls):
        if cls.fn is not None:
            return cls.fn
        import torch

        class Fn(torch.autograd.Function):
            @staticmethod
            def forward(ctx, table, ids, anchor, grad_scale, prefetched):
                keys = field_keys(ids, table.num_fields).reshape(-1)
                unique, inverse = torch.unique(keys, return_inverse=True)
                k = unique.numpy().astype(np.uint64)
                rows = prefetched.wait() if prefetched is not None else table.table.pull(k)
                ctx.table, ctx.k, ctx.inverse, ctx.scale = table, k, inverse, grad_scale
                ctx.shape = (ids.shape[0], table.num_fields * table.dim)
                return torch.from_numpy(rows)[inverse].reshape(ctx.shape)

            @staticmethod
            def backward(ctx, grad):
                t = ctx.table
                g = grad.reshape(-1, t.dim).to(torch.float32)
                summed = torch.zeros(ctx.k.size, t.dim, dtype=torch.float32)
                summed.index_add_(0, ctx.inverse, g)              # one gradient row per distinct key
                if ctx.scale != 1.0:
                    summed *= ctx.scale
                if t.sync:
                    barrier()      # every rank has read its rows for this step before any rank changes one
                call = t.table.push_async(ctx.k, summed.numpy())   # travels while the rest of backward runs
                t._pending.append(call)
                t._pushed = True
                return None, None, None, None, None

        cls.fn = Fn
        return Fn


class HostEmbedding:
    """`num_fields` embedding tables of width `dim` served by the host parameter server, used as a layer:
    ``layer(ids)`` pulls the rows of a [batch, num_fields] id matrix (every distinct key once) and returns
    [batch, num_fields * dim]; the backward pass sums the gradient rows per distinct key and pushes them, and the
    servers apply the update rule (SGD / Adagrad).  Rows are created on first pull, any 63-bit id is valid.
    Ranks are not synchronised with one another: a pull sees whatever pushes have reached the servers by then (the
    reference's consistency model); ``sync=True`` makes the steps bulk-synchronous (a barrier before and after the
    pushes of a step), which is what the GPU tables do by default.
    ``wait()`` after ``loss.backward()`` (or before the next pull of the same keys) makes sure the pushes have been
    applied; ``prefetch(ids)`` starts the pull of a later batch (it reads the rows as they are when the request
    arrives, i.e. possibly before the pushes of the step in between: the reference's asynchronous consistency).

    This is the reference's parameter-server mode (tips/core/ps/ps_client.h pull / push around a training step,
    with the server-side rule of tips/core/ps/sparse_access_method.h) bound to a framework, which the reference never
    did; the GPU counterpart is ``tips_b200.ps.gpu.ShardedEmbedding`` / ``embedding_lookup``."""

    def __init__(self, name: str, num_fields: int, dim: int, route: Optional[Route] = None, optimizer: str = "adagrad",
                 lr: float = 0.05, eps: float = 1e-8, local_shards: int = 2, average_over_ranks: bool = True,
                 sync: bool = False):
        self.num_fields, self.dim = int(num_fields), int(dim)
        # sync: bulk-synchronous steps like the GPU tables' default: a barrier before the pushes of a step and one
        # after them (in wait()), so that every rank computes on the same rows; every rank must then run every step
        self.sync = bool(sync)
        self._pushed = False
        self.table = HostSparseTable(name, dim, route, optimizer, lr, eps, np.float32, local_shards)
        # every rank pushes its own gradient: with data-parallel averaging each contributes 1 / size of the step
        self.grad_scale = 1.0 / _lib.core().tips_size() if average_over_ranks else 1.0
        self._pending = []
        self._prefetched = {}

    def prefetch(self, ids) -> None:
        import torch
        keys = torch.unique(field_keys(ids, self.num_fields).reshape(-1)).numpy().astype(np.uint64)
        self._prefetched[ids.data_ptr()] = (ids, self.table.pull_async(keys))

    def __call__(self, ids):
        import torch
        self.wait()                                            # rows pushed by the last step are in before we read
        hit = self._prefetched.pop(ids.data_ptr(), None)
        anchor = torch.zeros((), requires_grad=True)           # makes the output part of the graph
        return _HostLookupFn.get().apply(self, ids, anchor, self.grad_scale, hit[1] if hit else None)

    def wait(self) -> int:
        """Wait for the pushes in flight; returns how many pushed rows did not exist (0 in normal use)."""
        missing = 0
        while self._pending:
            missing += self._pending.pop().wait()
        if self.sync and self._pushed:
            self._pushed = False
            barrier()              # every rank's pushes of this step have been applied
        return missing

    def save(self, path: str, binary: bool = True) -> None:
        """Checkpoint: every server rank writes the rows it serves to ``path.rank<r>`` (after the pushes in flight)."""
        self.wait()
        barrier()
        self.table.save(f"{path}.rank{_lib.core().tips_rank()}", binary=binary)
        barrier()

    def load(self, path: str, nfiles: int, binary: bool = True) -> None:
        """Restore from the files of a checkpoint written by `nfiles` ranks; each rank keeps the rows it serves under
        the current routing, so the number of ranks may differ from the one that wrote the checkpoint."""
        import os
        for r in range(nfiles):
            f = f"{path}.rank{r}"
            if os.path.exists(f):
                self.table.load(f, binary=binary)
        barrier()

    def close(self) -> None:
        self.wait()
        for _, call in self._prefetched.values():
            call.cancel()
        self._prefetched.clear()
        self.table.close()

