"""The runtime's counters as a Prometheus endpoint.

``start_metrics_server(port)`` serves ``tips.metrics()`` (collectives enqueued / completed / failed, bytes per
collective kind, negotiation requests, frozen executions, stall warnings, RPC messages, kernel launches) at
``http://<host>:<port>/metrics``; the values are read when the endpoint is scraped, so the training loop pays
nothing.  Needs the ``prometheus_client`` package; every rank serves its own counters (port + local rank by
default), labelled with its rank.  The reference has no metrics beyond log lines (tips/core/common/logging.h).
"""
from __future__ import annotations

from typing import Optional


class _Collector:
    def __init__(self, prefix: str):
        self.prefix = prefix

    def collect(self):
        from prometheus_client.core import GaugeMetricFamily
        from .. import runtime
        if not runtime.is_initialized():
            return
        rank = str(runtime.rank())
        for name, value in sorted(runtime.metrics().items()):
            if isinstance(value, bool):
                value = int(value)
            if not isinstance(value, (int, float)):
                continue
            g = GaugeMetricFamily(f"{self.prefix}_{name}", f"tips runtime counter {name}", labels=["rank"])
            g.add_metric([rank], float(value))
            yield g


_registered = None


def start_metrics_server(port: int = 9400, addr: str = "0.0.0.0", per_rank_port: bool = True, prefix: str = "tips",
                         registry=None) -> int:
    """Start the HTTP endpoint in a daemon thread; returns the port it listens on."""
    global _registered
    import prometheus_client
    from .. import runtime
    registry = registry or prometheus_client.REGISTRY
    if _registered is None:
        _registered = _Collector(prefix)
        registry.register(_registered)
    if per_rank_port and runtime.is_initialized():
        port += runtime.local_rank()
    prometheus_client.start_http_server(port, addr=addr, registry=registry)
    return port


def render(prefix: str = "tips") -> str:
    """The same text a scrape would return, without a server (for logs and tests)."""
    import prometheus_client
    registry = prometheus_client.CollectorRegistry()
    registry.register(_Collector(prefix))
    return prometheus_client.generate_latest(registry).decode()
