"""GPU data plane set-up: device binding, the symmetric memory window, the
communication context of the kernels and the device executor of the engine.

The reference has no device data plane (every op sets ``on_gpu = false``,
tips/tensorflow/ops.cc:97,172,241).  Here each process owns one GPU; the ranks
allocate one identically sized window with ``torch.distributed._symmetric_memory``
(CUDA VMM allocation + handle exchange + NVLS multicast binding), every process
maps every peer's window, and the kernels in csrc/kernels/comm.cu address peer
memory directly.  Window layout:

    [ 64 KiB signal flags | staging area | heap for gradient buckets ]

torch.distributed (NCCL) is used for that rendezvous and as the library floor
(``backend="nccl"``); it is never on the default data path.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .. import _lib
from ..config import get_config

_state = None


class DeviceState:
    def __init__(self):
        self.backend = "fused"
        self.device = None
        self.rank = 0
        self.size = 1
        self.emulated = 0
        self.window = None          # uint8 tensor (this rank's window), or list of tensors when emulated
        self.windows = None
        self.window_bytes = 0
        self.staging_bytes = 0
        self.heap_off = 0
        self.heap_end = 0
        self.peer_ptrs = []
        self.multicast_ptr = 0
        self._events = []
        self.pg_ready = False

    # -- symmetric heap -------------------------------------------------------
    def alloc_symmetric(self, nbytes: int, dtype=torch.uint8):
        """Carve `nbytes` out of the window heap (same offset on every rank as long as every
        rank makes the same allocations in the same order). Returns (tensor, byte offset)."""
        align = 256
        off = (self.heap_off + align - 1) // align * align
        if off + nbytes > self.heap_end:
            raise MemoryError(f"symmetric heap exhausted: need {nbytes} bytes at {off}, heap ends at {self.heap_end}; "
                              f"raise TIPS_SYMM_HEAP_BYTES")
        self.heap_off = off + nbytes
        win = self.window if not self.emulated else self.windows[0]
        t = win[off:off + nbytes]
        if dtype != torch.uint8:
            t = t.view(dtype)
        return t, off

    def in_window(self, t: torch.Tensor) -> bool:
        if self.window is None:
            return False
        base = self.window.data_ptr()
        return base <= t.data_ptr() < base + self.window_bytes

    # -- events -----------------------------------------------------------------
    def events_for_op(self):
        lib = _lib.kernels()
        return lib.tipsk_event_create(), lib.tipsk_event_create()

    def recycle_event(self, ev):
        _lib.kernels().tipsk_event_recycle(ev)

    def metrics(self):
        lib = _lib.kernels()
        from ..ops import base
        return {"comm_kernel_launches": int(lib.tipsk_comm_launches()), "kernel_wrapper_calls": base.launches(),
                "uses_multimem": bool(lib.tipsk_comm_uses_multimem())}

    def check_status(self, clear=True):
        """Raise if a kernel reported a bounded-wait timeout."""
        lib = _lib.kernels()
        out = (ctypes.c_int32 * 7)()
        slots = self.emulated if self.emulated else 1
        for s in range(slots):
            code = lib.tipsk_comm_status(s, out, 1 if clear else 0)
            if code != 0:
                from ..runtime import TipsError
                raise TipsError(
                    f"device collective timed out: rank {out[6]} waited for rank {out[1]} in phase {out[2]} "
                    f"(block {out[3]}, epoch {out[4]}, channel {out[5]})", 5)


def state() -> DeviceState:
    if _state is None:
        raise RuntimeError("the GPU data plane is not set up; call tips_b200.init() on a CUDA machine")
    return _state


def record_event(ev, stream):
    rc = _lib.kernels().tipsk_event_record(ev, stream)
    if rc:
        raise RuntimeError("cudaEventRecord failed")


def stream_wait_event(stream, ev):
    rc = _lib.kernels().tipsk_stream_wait_event(stream, ev)
    if rc:
        raise RuntimeError("cudaStreamWaitEvent failed")


def _ptr_array(ptrs):
    arr = (ctypes.c_void_p * len(ptrs))()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


def setup(emulate_ranks: int = 0) -> DeviceState:
    """Bind the device and build the communication context.

    emulate_ranks > 0 builds that many rank windows on the current device (single process,
    single GPU) so that the multi-rank kernels can be exercised without a second GPU.
    """
    global _state
    from .. import runtime
    cfg = get_config()
    core = _lib.core()
    lib = _lib.kernels()
    st = DeviceState()
    st.backend = cfg.backend
    initialised = bool(core.tips_is_initialized())
    st.rank = core.tips_rank() if initialised else 0
    st.size = core.tips_size() if initialised else 1
    local_rank = core.tips_local_rank() if initialised else 0
    ndev = torch.cuda.device_count()
    dev_index = local_rank % max(ndev, 1)
    torch.cuda.set_device(dev_index)
    st.device = torch.device("cuda", dev_index)

    heap_bytes = int(os.environ.get("TIPS_SYMM_HEAP_BYTES", 2 << 30))
    staging = int(cfg.symm_window_bytes)
    signal = int(lib.tipsk_comm_staging_offset())

    if emulate_ranks and emulate_ranks > 1:
        st.emulated = emulate_ranks
        st.size = emulate_ranks
        heap_bytes = int(os.environ.get("TIPS_SYMM_HEAP_BYTES", 64 << 20))
        total = signal + staging + heap_bytes
        st.windows = [torch.zeros(total, dtype=torch.uint8, device=st.device) for _ in range(emulate_ranks)]
        st.window = st.windows[0]
        st.peer_ptrs = [w.data_ptr() for w in st.windows]
        st.window_bytes = total
    elif st.size > 1:
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29400")
            dist.init_process_group("nccl", rank=st.rank, world_size=st.size, device_id=st.device)
            st.owns_pg = True
        st.pg_ready = True
        total = signal + staging + heap_bytes
        group = dist.group.WORLD
        win = symm_mem.empty(total, dtype=torch.uint8, device=st.device)
        hdl = symm_mem.rendezvous(win, group.group_name)
        st.window = win
        st.window_bytes = total
        st.peer_ptrs = [int(p) for p in hdl.buffer_ptrs]
        try:
            st.multicast_ptr = int(hdl.multicast_ptr or 0)
        except Exception:
            st.multicast_ptr = 0
        win.zero_()
        torch.cuda.synchronize()
        dist.barrier(device_ids=[dev_index])
        st._symm_handle = hdl
    else:
        st.window = None
        st.window_bytes = 0

    st.staging_bytes = staging
    st.heap_off = signal + staging
    st.heap_end = st.window_bytes
    if st.window is not None:
        use_mm = 1 if (cfg.use_multimem and st.multicast_ptr and os.environ.get("TIPS_DISABLE_MULTIMEM", "0") != "1") else 0
        rc = lib.tipsk_comm_init(st.rank if not st.emulated else 0, st.size, _ptr_array(st.peer_ptrs),
                                 ctypes.c_void_p(st.multicast_ptr or None), st.window_bytes, staging,
                                 int(cfg.device_wait_budget_ms), int(cfg.comm_blocks),
                                 int(cfg.one_shot_threshold_bytes), use_mm, 1 if st.emulated else 0)
        if rc:
            raise RuntimeError("tipsk_comm_init: " + lib.tipsk_last_error().decode())
        lib.tipsk_executor_configure(dev_index, ctypes.c_void_p(st.peer_ptrs[st.rank if not st.emulated else 0]),
                                     st.window_bytes)
    if initialised and not st.emulated:
        core.tips_set_device_executor(lib.tipsk_device_executor_ptr())
        if st.size > 1:
            runtime.barrier()
    _state = st
    return st


def teardown(st: DeviceState) -> None:
    global _state
    try:
        torch.cuda.synchronize()
        lib = _lib.kernels()
        lib.tipsk_comm_shutdown()
        if st.pg_ready:
            import torch.distributed as dist
            if dist.is_initialized():
                try:
                    dist.barrier()
                    if getattr(st, "owns_pg", False):
                        dist.destroy_process_group()
                except Exception:
                    pass
    finally:
        _state = None


# ------------------------------------------------------------------ sub-groups


class DeviceGroup:
    """Device collectives (allreduce, allgatherv, broadcast) among a subset of the ranks, run by the same kernels
    as the collectives of all ranks over peer loads and stores.

    A group owns a slice of every rank's window: barrier flags plus a staging area, at the same offset everywhere,
    so its barriers and epochs are independent of the other groups' and of the job-wide collectives, and two
    disjoint groups run at the same time.  EVERY rank of the job constructs the group, in the same order relative
    to other symmetric allocations (the reservation must land at the same offset on all ranks); only members may
    call the collectives, in the same order on every member.  The calls are queued on the current CUDA stream.

    The reference has one communicator for the whole job (tips/core/mpi_context.h:20-53: the global communicator
    and a per-node one); sub-groups are what its parameter-server mode builds on top, with workers and servers as
    separate rank sets (tips/core/ps/route.h:58-114).

    With the ranks emulated on one GPU the tensor arguments are lists with one tensor per member, in member order.
    """

    _standalone_ids = 1 << 40

    def __init__(self, members, group_id: int | None = None, stage_bytes: int | None = None):
        st = state()
        lib = _lib.kernels()
        self.members = sorted(int(m) for m in members)
        if len(set(self.members)) != len(self.members) or not self.members or self.members[0] < 0 \
                or self.members[-1] >= st.size:
            raise ValueError(f"bad group members {members} for a job of {st.size} ranks")
        if st.window is None:
            raise RuntimeError("device groups need more than one rank")
        if group_id is None:
            DeviceGroup._standalone_ids += 1
            group_id = DeviceGroup._standalone_ids
        self.id = int(group_id)
        self.stage_bytes = int(stage_bytes if stage_bytes is not None else get_config().group_stage_bytes) // 4096 * 4096
        # the window is zeroed when it is created and symmetric allocations are never handed out twice,
        # so the flags of the new area start at zero on every rank
        _, self.area_off = st.alloc_symmetric(int(lib.tipsk_comm_flag_bytes()) + self.stage_bytes)
        arr = (ctypes.c_int32 * len(self.members))(*self.members)
        if lib.tipsk_comm_group_create(self.id, arr, len(self.members), self.area_off, self.stage_bytes):
            raise RuntimeError("device group: " + lib.tipsk_last_error().decode())
        self._st = st

    @property
    def size(self) -> int:
        return len(self.members)

    @property
    def rank(self) -> int:
        """Group rank of this process (-1: not a member); 0 when the ranks are emulated."""
        if self._st.emulated:
            return 0
        return self.members.index(self._st.rank) if self._st.rank in self.members else -1

    def _rows(self, x):
        rows = list(x) if isinstance(x, (list, tuple)) else [x]
        want = self.size if self._st.emulated else 1
        if len(rows) != want:
            raise ValueError(f"expected {want} tensor(s), got {len(rows)}")
        if self.rank < 0:
            raise RuntimeError("this rank is not a member of the group")
        for t in rows:
            if not (t.is_cuda and t.is_contiguous()):
                raise ValueError("device group collectives take contiguous CUDA tensors")
        return rows

    def _check(self, rc, what):
        if rc:
            raise RuntimeError(f"group {what}: " + _lib.kernels().tipsk_last_error().decode())

    def allreduce_(self, tensors, op_code: int = 0, prescale: float = 1.0, postscale: float = 1.0):
        """In-place reduction over the members (op_code: 0 sum, 1 max, 2 min, 3 product)."""
        from ..ops import base
        rows = self._rows(tensors)
        nbytes = rows[0].numel() * rows[0].element_size()
        ptrs = _ptr_array([t.data_ptr() for t in rows])
        self._check(_lib.kernels().tipsk_group_allreduce(self.id, ptrs, ptrs, nbytes, base.code(rows[0]), op_code,
                                                        prescale, postscale, base.comm_stream()), "allreduce")
        return tensors

    def allgatherv(self, tensors, first_dims):
        """Concatenation along dim 0 of every member's tensor; `first_dims` lists every member's dim 0."""
        from ..ops import base
        rows = self._rows(tensors)
        inner = rows[0].shape[1:]
        row_bytes = rows[0].element_size()
        for d in inner:
            row_bytes *= d
        sizes = (ctypes.c_uint64 * self.size)(*[int(d) * row_bytes for d in first_dims])
        outs = [torch.empty((int(sum(first_dims)),) + tuple(inner), dtype=t.dtype, device=t.device) for t in rows]
        self._check(_lib.kernels().tipsk_group_allgatherv(self.id, _ptr_array([t.data_ptr() for t in rows]),
                                                         _ptr_array([o.data_ptr() for o in outs]), sizes,
                                                         base.comm_stream()), "allgatherv")
        return outs if isinstance(tensors, (list, tuple)) else outs[0]

    def broadcast_(self, tensors, root: int = 0):
        """In-place broadcast from group rank `root`."""
        from ..ops import base
        rows = self._rows(tensors)
        nbytes = rows[0].numel() * rows[0].element_size()
        ptrs = _ptr_array([t.data_ptr() for t in rows])
        self._check(_lib.kernels().tipsk_group_broadcast(self.id, ptrs, ptrs, nbytes, int(root), base.comm_stream()),
                    "broadcast")
        return tensors

    def close(self):
        _lib.kernels().tipsk_comm_group_destroy(self.id)


# ------------------------------------------------------------------ NCCL floor


def _done(h, out, post=None):
    h.output = out
    h.post = post
    return h


def nccl_allreduce(h, tensor, wire, ctx, compression, reduce_code, prescale, postscale, inplace):
    import torch.distributed as dist
    ops = {0: dist.ReduceOp.SUM, 1: dist.ReduceOp.MAX, 2: dist.ReduceOp.MIN, 3: dist.ReduceOp.PRODUCT}
    buf = wire if (inplace and wire is tensor) else wire.clone()
    if prescale != 1.0:
        buf.mul_(prescale)
    dist.all_reduce(buf, op=ops[reduce_code])
    if postscale != 1.0:
        buf.mul_(postscale)
    out = compression.decompress(buf, ctx)
    if inplace and out is not tensor:
        tensor.copy_(out)
        out = tensor
    return _done(h, out)


def nccl_allgather(h, src):
    import torch.distributed as dist
    n = dist.get_world_size()
    sizes = [torch.zeros(1, dtype=torch.int64, device=src.device) for _ in range(n)]
    dist.all_gather(sizes, torch.tensor([src.shape[0]], dtype=torch.int64, device=src.device))
    sizes = [int(s.item()) for s in sizes]
    outs = [torch.empty((s,) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device) for s in sizes]
    dist.all_gather(outs, src)
    return _done(h, torch.cat(outs, dim=0))


def nccl_broadcast(h, tensor, src, root, inplace):
    import torch.distributed as dist
    buf = src if inplace and src is tensor else src.clone()
    dist.broadcast(buf, src=root)
    if inplace and buf is not tensor:
        tensor.copy_(buf)
        buf = tensor
    return _done(h, buf)
