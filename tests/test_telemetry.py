"""Telemetry: the scheduler's per-fire probe tree (runtime/src/probe/fire.rs) and the OTLP/HTTP span
exporter (runtime/src/telemetry.rs) against a local collector stand-in."""
import http.server
import json
import threading
import time

import pytest

from pie_b200.runtime import telemetry


def test_fire_probe_tree_is_recorded_and_children_sum_to_total():
    from test_runtime_cpu import CounterBehavior, MockDriver, engine_with
    tel = telemetry.configure(True)
    try:
        eng = engine_with(MockDriver(CounterBehavior(), total_pages=64))
        for prompt in ([1, 2, 3, 4], [1, 2, 3]):
            eng.run("text-completion-bench", {"prompt_tokens": prompt, "max_tokens": 6, "per_step": True}, 30)
        eng.shutdown()
        snap = tel.snapshot()["probes"]
    finally:
        telemetry.configure(False)
    for k in ("fire_inter_fire", "fire_post_dispatch_to_fire", "fire_accumulate_loop", "fire_execute_batch_build",
              "fire_execute_driver_fire", "fire_execute_response_dispatch", "fire_execute_total",
              "fire_post_dispatch_hooks", "driver_forward", "driver_total"):
        assert k in snap and snap[k]["count"] >= 1, k
    n = snap["fire_execute_total"]["count"]
    total = snap["fire_execute_total"]["mean_us"] * n
    parts = sum(snap[f"fire_execute_{c}"]["mean_us"] * snap[f"fire_execute_{c}"]["count"]
                for c in ("batch_build", "driver_fire", "response_dispatch"))
    assert parts == pytest.approx(total, rel=0.02, abs=50.0 * n)
    assert "pie_b200_probe_fire_execute_total_seconds_count" in telemetry.Telemetry.prometheus(tel)


class _Collector(http.server.BaseHTTPRequestHandler):
    got = []

    def log_message(self, *a):
        pass

    def do_POST(self):
        body = self.rfile.read(int(self.headers["Content-Length"]))
        _Collector.got.append((self.path, self.headers["Content-Type"], json.loads(body)))
        self.send_response(200)
        self.send_header("Content-Length", "2")
        self.end_headers()
        self.wfile.write(b"{}")


def test_spans_reach_an_otlp_http_collector_and_a_dead_collector_only_drops():
    _Collector.got.clear()
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), _Collector)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    tel = telemetry.Telemetry("svc", True, None, f"http://127.0.0.1:{srv.server_address[1]}", flush_interval_s=0.05)
    with tel.span("launch", inferlet="demo", tokens=7, ratio=0.5, ok=True):
        pass
    with pytest.raises(ValueError):
        with tel.span("fails"):
            raise ValueError("boom")
    tel.close()
    srv.shutdown()
    assert _Collector.got and all(p == "/v1/traces" and ct == "application/json" for p, ct, _ in _Collector.got)
    spans = [s for _, _, b in _Collector.got for rs in b["resourceSpans"] for ss in rs["scopeSpans"] for s in ss["spans"]]
    res = _Collector.got[0][2]["resourceSpans"][0]["resource"]["attributes"]
    assert {"key": "service.name", "value": {"stringValue": "svc"}} in res
    by = {s["name"]: s for s in spans}
    assert set(by) == {"launch", "fails"} and len(by["launch"]["traceId"]) == 32 and len(by["launch"]["spanId"]) == 16
    attrs = {a["key"]: a["value"] for a in by["launch"]["attributes"]}
    assert attrs == {"inferlet": {"stringValue": "demo"}, "tokens": {"intValue": "7"}, "ratio": {"doubleValue": 0.5},
                     "ok": {"boolValue": True}}
    assert by["fails"]["status"]["code"] == 2 and "boom" in by["fails"]["status"]["message"]
    assert int(by["launch"]["endTimeUnixNano"]) >= int(by["launch"]["startTimeUnixNano"])

    dead = telemetry.Telemetry("svc", True, None, "http://127.0.0.1:9", flush_interval_s=0.05)
    t0 = time.perf_counter()
    with dead.span("x"):
        pass
    assert time.perf_counter() - t0 < 0.5            # the span itself never waits for the collector
    dead.close()
    assert dead.dropped_batches == 1


def test_nvtx_ranges_wrap_the_driver_phases_and_cost_nothing_when_off():
    import numpy as np
    from pie_b200.driver import nvtx
    from pie_b200.driver.executor import TorchDriver
    from pie_b200.driver.schema import ForwardRequest, SamplerSpec
    from pie_b200.models.config import preset
    events = []
    drv = TorchDriver(preset("tiny-llama", num_hidden_layers=1), device="cpu", num_pages=8)
    i32 = lambda *a: np.asarray(a, dtype=np.int32)
    req = lambda: ForwardRequest(tokens=i32(1, 2, 3), positions=i32(0, 1, 2), qo_indptr=i32(0, 3), kv_page_indices=i32(0),
                                 kv_page_indptr=i32(0, 1), kv_last_page_lens=i32(3), slot_req=i32(0), slot_row=i32(2),
                                 slot_samplers=[SamplerSpec()])
    drv.fire_batch(req())
    assert events == []
    assert nvtx.enable((lambda name: events.append(("push", name)), lambda: events.append(("pop",))))
    try:
        drv.fire_batch(req())
    finally:
        nvtx.disable()
    names = [e[1] for e in events if e[0] == "push"]
    assert names == ["pie.fire", "forward.general", "respond"]
    assert sum(e[0] == "pop" for e in events) == 3 and events[-1] == ("pop",)


def test_monitor_renders_status_processes_and_fire_tree_locally_and_over_the_client(tmp_path):
    import io
    import json
    from test_runtime_cpu import CounterBehavior, MockDriver, engine_with
    from pie_b200.client.client import PieClient
    from pie_b200.server import cli
    from pie_b200.server.auth import Authenticator
    from pie_b200.server.monitor import render, run_monitor
    from pie_b200.server.server import PieServer
    tel = telemetry.configure(True)
    eng = engine_with(MockDriver(CounterBehavior(), total_pages=64))
    srv = PieServer(eng, "127.0.0.1", 0, Authenticator(False), str(tmp_path / "programs"))
    port = srv.start()
    try:
        eng.run("text-completion-bench", {"prompt_tokens": [1, 2, 3], "max_tokens": 5, "per_step": True}, 30)
        st = eng.model_status()
        assert "fire_execute_total" in st["fire"] and st["process_table"] == []
        text = render(st, {})
        assert "per-fire probes" in text and "fire_execute_driver_fire" in text and "batch size" in text and "[mock] kv 0/64" in text
        buf = io.StringIO()
        run_monitor(eng, period=0.01, out=buf, iterations=2, clear=False)
        assert buf.getvalue().count("pie_b200 ") == 2
        c = PieClient(f"ws://127.0.0.1:{port}")
        remote = io.StringIO()
        run_monitor(c.model_status, period=0.01, out=remote, iterations=1, clear=False)
        c.close()
        assert "[mock] kv" in remote.getvalue() and "per-fire probes" in remote.getvalue()
        assert cli.main(["monitor", "--uri", f"ws://127.0.0.1:{port}", "--iterations", "1", "--period", "0.01"]) == 0
        json.dumps(st)                                   # the status stays JSON-serialisable for the query
    finally:
        srv.stop()
        eng.shutdown()
        telemetry.configure(False)
