"""Run-time configuration.

The reference is configured by a handful of environment variables (``GLOG_v``,
``HOROVOD_ELASTIC``), RpcServer constructor arguments and Python keyword
arguments (tips/core/common/naive_rpc.h:100-101,158-160;
tips/tensorflow/__init__.py:65-68).  Here every knob lives in one dataclass
whose fields can be overridden with ``TIPS_<FIELD>`` environment variables.
"""
from __future__ import annotations

import dataclasses
import os


@dataclasses.dataclass
class Config:
    # Collective engine
    fusion_threshold_bytes: int = 64 << 20   # size of one gradient bucket / host fusion buffer
    fusion_slice_bytes: int = 0              # >0: a bucket is reduced in slices of about this size as backward
                                             # completes them; 0: the whole bucket at once (faster on ResNet-50 on
                                             # NVSwitch, where the 51 MB allreduce costs 0.2 ms and a collective that
                                             # shares the SMs with backward slows backward by as much)
    cycle_time_ms: int = 0                   # extra batching delay of the coordinator loop
    stall_warn_s: float = 60.0               # warn when a tensor waits this long for some ranks
    stall_abort_s: float = 0.0               # >0: fail the tensor instead of waiting forever
    # Device data plane
    backend: str = "fused"                   # fused = own sm_100a kernels; nccl = library floor
    wire_dtype: str = "auto"                 # auto = gradient dtype; bf16/fp16 = compress on the wire
    one_shot_threshold_bytes: int = 512 << 10
    device_wait_budget_ms: int = 20000       # bound of every in-kernel wait on a peer
    comm_blocks: int = 64                    # grid of the communication kernels (SM budget)
    use_multimem: bool = True                # NVLS multimem instructions when a multicast mapping exists
    symm_window_bytes: int = 256 << 20       # staging window for tensors outside symmetric memory
    group_stage_bytes: int = 32 << 20        # staging area of every sub-group of ranks with device collectives
    static_schedule: bool = True             # freeze the bucket order after the first negotiated step
    fused_update: bool = False               # fused optimizers step inside the gradient allreduce, state sharded
    device_status_check: str = "step"        # step: every synchronize() reads the kernels' status block (no device
                                             # wait) and raises if a bounded wait ran out; sync: waits for the
                                             # collective first, so the failing step itself raises; off
    collective_timeout_s: float = 0.0        # >0: DistributedOptimizer.synchronize() gives up on a bucket after this long
    numa_bind: bool = False                  # init() limits the process to the CPUs of its GPU's NUMA node
    # Parameter server
    ps_wire_dtype: str = "grad"              # grad: rows of a push cross NVLink in the dtype of the pushed gradients
                                             # (a rank's per-row sum is rounded to bf16 once when they are bf16);
                                             # fp32: always fp32
    ps_bf16_shadow: bool = True              # tables over several ranks keep a bf16 copy of their rows that bf16
                                             # pulls read (half the bytes over NVLink, a quarter more table memory)
    # Observability
    log_level: str = "WARNING"
    timeline_path: str = ""

    @classmethod
    def from_env(cls) -> "Config":
        cfg = cls()
        for f in dataclasses.fields(cls):
            raw = os.environ.get("TIPS_" + f.name.upper())
            if raw is None:
                continue
            if f.type in ("int", int):
                setattr(cfg, f.name, int(raw))
            elif f.type in ("float", float):
                setattr(cfg, f.name, float(raw))
            elif f.type in ("bool", bool):
                setattr(cfg, f.name, raw.lower() in ("1", "true", "yes", "on"))
            else:
                setattr(cfg, f.name, raw)
        return cfg


_config = Config.from_env()


def get_config() -> Config:
    return _config


def set_config(**kwargs) -> Config:
    for k, v in kwargs.items():
        if not hasattr(_config, k):
            raise AttributeError(f"unknown tips config field {k!r}")
        setattr(_config, k, v)
    return _config
