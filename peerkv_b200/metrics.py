"""Counters and gauges of the path, under the reference's metric names
(PeerKV umallm/observability/metrics.py:31-46) plus the per-call counters of the
attention path itself.  With `prometheus_client` installed these are real Prometheus
metrics; without it they are plain in-process counters with the same interface, so the
values can always be read back (`snapshot()`), in tests too.
"""
from __future__ import annotations

import threading
from typing import Dict, Tuple

try:  # pragma: no cover - exercised only where prometheus_client is installed
    import prometheus_client as _prom
except Exception:  # pragma: no cover
    _prom = None

_lock = threading.Lock()
_values: Dict[Tuple[str, Tuple[Tuple[str, str], ...]], float] = {}


class _Child:
    def __init__(self, name, labels, prom_child):
        self._key = (name, tuple(sorted(labels.items())))
        self._prom = prom_child

    def inc(self, v: float = 1.0):
        with _lock:
            _values[self._key] = _values.get(self._key, 0.0) + v
        if self._prom is not None:
            self._prom.inc(v)

    def set(self, v: float):
        with _lock:
            _values[self._key] = float(v)
        if self._prom is not None:
            self._prom.set(v)

    def get(self) -> float:
        with _lock:
            return _values.get(self._key, 0.0)


class _Metric:
    def __init__(self, kind: str, name: str, doc: str, labelnames=()):
        self.name, self.labelnames = name, tuple(labelnames)
        self._prom = None
        if _prom is not None:
            try:
                cls = _prom.Counter if kind == "counter" else _prom.Gauge
                self._prom = cls(name, doc, list(labelnames))
            except ValueError:          # registered already (module imported twice)
                self._prom = None
        self._bare = None if labelnames else _Child(name, {}, self._prom)

    def labels(self, **kw) -> _Child:
        pc = self._prom.labels(**kw) if self._prom is not None else None
        return _Child(self.name, {k: str(v) for k, v in kw.items()}, pc)

    def inc(self, v: float = 1.0):
        self._bare.inc(v)

    def set(self, v: float):
        self._bare.set(v)

    def get(self) -> float:
        return self._bare.get()


def Counter(name, doc, labelnames=()):
    return _Metric("counter", name, doc, labelnames)


def Gauge(name, doc, labelnames=()):
    return _Metric("gauge", name, doc, labelnames)


# selector / do-no-harm (the reference's names)
SELECTED_POINT = Counter("peerkv_selected_point_total", "corner chosen", ["point"])
DO_NO_HARM_VIOL = Counter("peerkv_do_no_harm_violations_total", "invariant breaches", ["rule"])
ADMISSIBLE_POINTS = Gauge("peerkv_admissible_points", "size of admissible set (last request)")
PEER_BUSY = Gauge("peerkv_peer_compute_busy", "1 if a peer GPU is computing", ["peer"])
LINK_EFF_GBPS = Gauge("peerkv_link_eff_gbps", "measured one-way effective bandwidth", ["fabric"])
XFER_BYTES = Counter("peerkv_xfer_bytes_total", "bytes that crossed between GPUs", ["dir"])

# the attention path itself
ATTN_CALLS = Counter("peerkv_attn_calls_total", "decode-attention calls", ["path"])        # single | sharded | fallback
KV_BYTES_READ = Counter("peerkv_kv_bytes_read_total", "KV bytes the kernels were asked to read", ["gpu"])
KV_APPEND_TOKENS = Counter("peerkv_kv_append_tokens_total", "new tokens routed to the GPU that owns their block")
DEVICE_STATUS = Counter("peerkv_device_status_total", "non-zero device status words read back", ["bit"])


def snapshot() -> dict:
    """All values recorded so far: {metric{label=value,...}: number}."""
    with _lock:
        items = list(_values.items())
    out = {}
    for (name, labels), v in items:
        key = name + ("{" + ",".join(f"{k}={val}" for k, val in labels) + "}" if labels else "")
        out[key] = v
    return out


def reset():
    """Clears the in-process values (tests)."""
    with _lock:
        _values.clear()
