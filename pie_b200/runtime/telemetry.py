"""Telemetry: spans, counters and gauges of the engine, exported as Prometheus text and as
OTLP-shaped JSON lines (a file or stderr; there is no collector dependency). Probes are cheap
named timers around the hot host path (`probe("fold")`), aggregated per name.
Counterpart of runtime/src/telemetry.rs:1-45 and runtime/src/probe/{mod,fire,driver_cuda}.rs.
"""
from __future__ import annotations

import json
import os
import threading
import time
from collections import defaultdict
from contextlib import contextmanager
from typing import Dict, Optional


class _Stat:
    __slots__ = ("count", "total", "max")

    def __init__(self):
        self.count, self.total, self.max = 0, 0.0, 0.0

    def add(self, v: float) -> None:
        self.count += 1
        self.total += v
        if v > self.max:
            self.max = v


class Telemetry:
    def __init__(self, service: str = "pie_b200", enabled: bool = True, export_path: Optional[str] = None):
        self.service, self.enabled = service, enabled
        self.counters: Dict[str, float] = defaultdict(float)
        self.gauges: Dict[str, float] = {}
        self.probes: Dict[str, _Stat] = defaultdict(_Stat)
        self._lock = threading.Lock()
        self._out = open(export_path, "a") if export_path else None
        self._span_seq = 0

    # ---- metrics
    def incr(self, name: str, value: float = 1.0) -> None:
        if self.enabled:
            with self._lock:
                self.counters[name] += value

    def gauge(self, name: str, value: float) -> None:
        if self.enabled:
            self.gauges[name] = value

    @contextmanager
    def probe(self, name: str):
        if not self.enabled:
            yield
            return
        t0 = time.perf_counter()
        try:
            yield
        finally:
            dt = time.perf_counter() - t0
            with self._lock:
                self.probes[name].add(dt)

    def record_probe_us(self, name: str, micros: float) -> None:
        """Timings measured elsewhere (the driver's per-fire probe fields)."""
        if self.enabled:
            with self._lock:
                self.probes[name].add(micros * 1e-6)

    # ---- spans
    @contextmanager
    def span(self, name: str, **attrs):
        if not self.enabled or self._out is None:
            yield
            return
        with self._lock:
            self._span_seq += 1
            sid = self._span_seq
        start = time.time_ns()
        err = None
        try:
            yield
        except BaseException as e:  # noqa: BLE001
            err = repr(e)
            raise
        finally:
            rec = {"resource": {"service.name": self.service}, "name": name, "spanId": f"{sid:016x}",
                   "startTimeUnixNano": start, "endTimeUnixNano": time.time_ns(),
                   "attributes": attrs, "status": {"code": "ERROR", "message": err} if err else {"code": "OK"}}
            with self._lock:
                self._out.write(json.dumps(rec) + "\n")
                self._out.flush()

    # ---- export
    def prometheus(self) -> str:
        p = self.service
        lines = []
        with self._lock:
            for k, v in sorted(self.counters.items()):
                lines += [f"# TYPE {p}_{k}_total counter", f"{p}_{k}_total {v:g}"]
            for k, v in sorted(self.gauges.items()):
                lines += [f"# TYPE {p}_{k} gauge", f"{p}_{k} {v:g}"]
            for k, s in sorted(self.probes.items()):
                lines += [f"# TYPE {p}_probe_{k}_seconds summary", f"{p}_probe_{k}_seconds_count {s.count}",
                          f"{p}_probe_{k}_seconds_sum {s.total:.9f}", f"{p}_probe_{k}_seconds_max {s.max:.9f}"]
        return "\n".join(lines) + "\n"

    def snapshot(self) -> dict:
        with self._lock:
            return {"counters": dict(self.counters), "gauges": dict(self.gauges),
                    "probes": {k: {"count": s.count, "mean_us": (s.total / s.count * 1e6 if s.count else 0.0),
                                   "max_us": s.max * 1e6} for k, s in self.probes.items()}}

    def close(self) -> None:
        if self._out:
            self._out.close()
            self._out = None


_GLOBAL = Telemetry(enabled=os.environ.get("PIE_TELEMETRY", "0") == "1",
                    export_path=os.environ.get("PIE_TELEMETRY_FILE") or None)


def get() -> Telemetry:
    return _GLOBAL


def configure(enabled: bool, export_path: Optional[str] = None, service: str = "pie_b200") -> Telemetry:
    global _GLOBAL
    _GLOBAL.close()
    _GLOBAL = Telemetry(service, enabled, export_path)
    return _GLOBAL
