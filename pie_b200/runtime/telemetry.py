"""Telemetry: spans, counters and gauges of the engine, exported as Prometheus text and as
OTLP: spans go to a JSON-lines file and / or, batched on a background thread, to a collector's
OTLP/HTTP endpoint (`<endpoint>/v1/traces`, JSON encoding; a collector that is down costs a dropped
batch, never a stalled engine). Probes are cheap named timers around the hot host path
(`probe("fold")`), aggregated per name; the scheduler records its per-fire tree through them.
Counterpart of runtime/src/telemetry.rs:1-45 and runtime/src/probe/{mod,fire,driver_cuda}.rs.
"""
from __future__ import annotations

import json
import os
import queue
import threading
import time
import urllib.request
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
    def __init__(self, service: str = "pie_b200", enabled: bool = True, export_path: Optional[str] = None,
                 endpoint: Optional[str] = None, flush_interval_s: float = 1.0):
        self.service, self.enabled = service, enabled
        self.endpoint = endpoint.rstrip("/") if endpoint else None
        self.dropped_batches = 0
        self._trace_id = os.urandom(16).hex()
        self._q: "queue.Queue" = queue.Queue(maxsize=8192)
        self._flush_s = flush_interval_s
        self._exporter = None
        if enabled and self.endpoint:
            self._exporter = threading.Thread(target=self._export_loop, name="pie-otlp", daemon=True)
            self._exporter.start()
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
        if not self.enabled or (self._out is None and self._exporter is None):
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
            if self._out is not None:
                with self._lock:                 # an open file: writing raises no audit event
                    self._out.write(json.dumps(rec) + "\n")
                    self._out.flush()
            if self._exporter is not None:
                try:
                    self._q.put_nowait(rec)
                except queue.Full:
                    self.dropped_batches += 1

    def _otlp_payload(self, recs) -> bytes:
        def attr(k, v):
            if isinstance(v, bool):
                return {"key": k, "value": {"boolValue": v}}
            if isinstance(v, int):
                return {"key": k, "value": {"intValue": str(v)}}
            if isinstance(v, float):
                return {"key": k, "value": {"doubleValue": v}}
            return {"key": k, "value": {"stringValue": str(v)}}
        spans = [{"traceId": self._trace_id, "spanId": r["spanId"], "name": r["name"], "kind": 1,
                  "startTimeUnixNano": str(r["startTimeUnixNano"]), "endTimeUnixNano": str(r["endTimeUnixNano"]),
                  "attributes": [attr(k, v) for k, v in r["attributes"].items()],
                  "status": {"code": 2, "message": r["status"].get("message", "")} if r["status"]["code"] == "ERROR" else {"code": 1}}
                 for r in recs]
        return json.dumps({"resourceSpans": [{"resource": {"attributes": [attr("service.name", self.service)]},
                                              "scopeSpans": [{"scope": {"name": "pie_b200"}, "spans": spans}]}]}).encode()

    def _export_loop(self) -> None:
        while True:
            recs = []
            try:
                first = self._q.get(timeout=self._flush_s)
                if first is None:
                    return
                recs.append(first)
                while len(recs) < 512:
                    nxt = self._q.get_nowait()
                    if nxt is None:
                        self._post(recs)
                        return
                    recs.append(nxt)
            except queue.Empty:
                pass
            if recs:
                self._post(recs)

    def _post(self, recs) -> None:
        try:
            req = urllib.request.Request(self.endpoint + "/v1/traces", data=self._otlp_payload(recs),
                                         headers={"Content-Type": "application/json"}, method="POST")
            urllib.request.urlopen(req, timeout=2.0).read()
        except Exception:  # noqa: BLE001 - an unreachable collector must not disturb serving
            self.dropped_batches += 1

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
        if self._exporter is not None:
            self._q.put(None)
            self._exporter.join(timeout=5.0)
            self._exporter = None
        if self._out:
            self._out.close()
            self._out = None


_GLOBAL = Telemetry(enabled=os.environ.get("PIE_TELEMETRY", "0") == "1",
                    export_path=os.environ.get("PIE_TELEMETRY_FILE") or None,
                    endpoint=os.environ.get("PIE_TELEMETRY_ENDPOINT") or None)


def get() -> Telemetry:
    return _GLOBAL


def configure(enabled: bool, export_path: Optional[str] = None, service: str = "pie_b200",
              endpoint: Optional[str] = None) -> Telemetry:
    global _GLOBAL
    _GLOBAL.close()
    _GLOBAL = Telemetry(service, enabled, export_path, endpoint)
    return _GLOBAL
