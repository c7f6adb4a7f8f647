"""Configuration from the environment, the engine's Chrome-trace timeline, counters and the NVTX switch."""
import json
import os

import torch

from mp_util import run_ranks


def test_config_from_env(monkeypatch):
    from tips_b200.config import Config, get_config, set_config
    monkeypatch.setenv("TIPS_FUSION_THRESHOLD_BYTES", "12345")
    monkeypatch.setenv("TIPS_STALL_WARN_S", "2.5")
    monkeypatch.setenv("TIPS_STATIC_SCHEDULE", "off")
    monkeypatch.setenv("TIPS_USE_MULTIMEM", "Yes")
    monkeypatch.setenv("TIPS_BACKEND", "nccl")
    monkeypatch.setenv("TIPS_NOT_A_FIELD", "ignored")
    cfg = Config.from_env()
    assert cfg.fusion_threshold_bytes == 12345 and isinstance(cfg.fusion_threshold_bytes, int)
    assert cfg.stall_warn_s == 2.5 and cfg.static_schedule is False and cfg.use_multimem is True
    assert cfg.backend == "nccl" and not hasattr(cfg, "not_a_field")
    defaults = Config()
    assert defaults.fusion_threshold_bytes == 64 << 20 and defaults.static_schedule is True
    before = get_config().cycle_time_ms
    try:
        assert set_config(cycle_time_ms=3).cycle_time_ms == 3
        try:
            set_config(no_such_field=1)
            raise AssertionError("an unknown field must be refused")
        except AttributeError:
            pass
    finally:
        set_config(cycle_time_ms=before)


def test_nvtx_ranges_are_free_without_cuda():
    from tips_b200.utils import trace
    was = trace.enabled()
    try:
        for on in (False, True):
            trace.enable(on)
            assert trace.enabled() is on
            with trace.nvtx_range("pack bucket 0"):       # no CUDA here: a null context either way
                pass
    finally:
        trace.enable(was)


def _timeline(rank, size, folder):
    import tips_b200 as tips
    assert tips.get_config().timeline_path            # set through the environment before init
    for i in range(3):
        out = tips.allreduce(torch.full((64,), float(rank)), op=tips.Sum, name=f"grad.{i}")
        assert float(out[0]) == sum(range(size))
    tips.allgather(torch.ones(rank + 1, 2), name="rows")
    tips.broadcast(torch.ones(5), root_rank=1, name="weights")
    m = tips.metrics()
    assert m["ops_enqueued"] == 5 and m["ops_completed"] == 5 and m["ops_failed"] == 0
    assert m["allreduce_bytes"] == 3 * 64 * 4 and m["negotiation_requests"] >= 5
    tips.shutdown()
    path = os.path.join(folder, f"timeline.json.rank{rank}")
    events = json.load(open(path))
    events = events["traceEvents"] if isinstance(events, dict) else events
    names = {e["name"] for e in events}
    phases = {e["cat"] for e in events}
    assert {"grad.0", "grad.1", "grad.2", "rows", "weights"} <= names, names
    assert {"NEGOTIATE", "EXECUTE"} <= phases, phases
    for e in events:
        assert e["ph"] == "X" and e["dur"] >= 0 and e["pid"] == rank and e["ts"] > 0


def test_timeline_and_counters(tmp_path):
    run_ranks(_timeline, 2, str(tmp_path), env={"TIPS_TIMELINE_PATH": os.path.join(str(tmp_path), "timeline.json")})


def _prometheus(rank, size):
    import urllib.request
    import tips_b200 as tips
    from tips_b200.utils import metrics_export
    from mp_util import free_port
    tips.allreduce(torch.ones(8), op=tips.Sum, name="m.0")
    tips.allgather(torch.ones(rank + 1), name="m.1")
    text = metrics_export.render()
    assert f'tips_ops_completed{{rank="{rank}"}} 2.0' in text and "tips_allreduce_bytes" in text
    if rank == 0:
        port = metrics_export.start_metrics_server(free_port(), addr="127.0.0.1", per_rank_port=False)
        tips.allreduce(torch.ones(8), op=tips.Sum, name="m.2")
        body = urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=10).read().decode()
        assert 'tips_ops_completed{rank="0"} 3.0' in body      # read at scrape time
    else:
        tips.allreduce(torch.ones(8), op=tips.Sum, name="m.2")
    tips.barrier()


def test_prometheus_endpoint():
    run_ranks(_prometheus, 2)
