"""`pie serve --monitor` and `pie monitor [--uri ws://host:port]`: a terminal dashboard of the engine, refreshed
once per second. Per model: KV pages, contexts, batch rate and latency with sparklines, the batch-size histogram,
staged-pass and chain counters, market price, evictions / deferrals / replays; the busiest live processes; and,
when telemetry is on, the scheduler's per-fire probe tree (`fire_*`, `driver_*`). The same renderer serves an
engine in this process and a remote one through the client's `model_status` query.
Counterpart of server/src/cli/monitor/* (TUI over the status query).
"""
from __future__ import annotations

import sys
import time
from typing import Callable

BARS = " ▁▂▃▄▅▆▇█"
FIRE_ORDER = ["fire_inter_fire", "fire_post_dispatch_to_fire", "fire_accumulate_loop", "fire_execute_total",
              "fire_execute_batch_build", "fire_execute_driver_fire", "fire_execute_response_dispatch",
              "fire_post_dispatch_hooks", "driver_build", "driver_h2d", "driver_forward", "driver_sample", "driver_d2h",
              "driver_total"]


def spark(values, width=40):
    vals = list(values)[-width:]
    hi = max(vals) if vals and max(vals) > 0 else 1.0
    return "".join(BARS[min(8, int(8 * v / hi))] for v in vals)


def hist_bar(hist, width=24) -> str:
    """Batch-size histogram (powers of two: 1, 2-3, 4-7, ... 128+) as one row of bars."""
    total = max(1, sum(hist))
    return " ".join(f"{1 << i}{'+' if i == len(hist) - 1 else ''}:{BARS[min(8, int(round(8 * h / total)))]}"
                    for i, h in enumerate(hist))


def render(status: dict, history: dict) -> str:
    lines = [f"pie_b200 {status['version']}  up {status['uptime_s']:.0f}s  processes {status['processes']}"]
    for name, m in status["models"].items():
        h = history.setdefault(name, {"lat": [], "tok": [], "last_tokens": m["total_tokens"]})
        h["lat"].append(m["last_batch_latency_us"] / 1e3)
        h["tok"].append(m["total_tokens"] - h["last_tokens"])
        h["last_tokens"] = m["total_tokens"]
        del h["lat"][:-120], h["tok"][:-120]
        used, total = m["kv_pages_used"], max(1, m["kv_pages_total"])
        lines += [f"[{name}] kv {used}/{total} ({100 * used / total:.1f}%)  contexts {m['contexts']}  "
                  f"snapshots {m.get('snapshots', 0)}  batches {m['total_batches']} (failed {m.get('failed_batches', 0)}, "
                  f"chunked requests {m.get('chunked_requests', 0)})  avg {m['avg_batch_latency_us'] / 1e3:.2f} ms",
                  f"  tokens/s  {spark(h['tok'])} {h['tok'][-1]}",
                  f"  batch ms  {spark(h['lat'])} {h['lat'][-1]:.2f}",
                  f"  batch size  {hist_bar(m.get('batch_size_hist', [0] * 8))}",
                  f"  staged hits {m['bypass_hits']}  chain submits {m['chain_submits']}  drops {m['chain_drops']}  "
                  f"price {m['market_price']:.2f}  waiting {m.get('market_waiting', 0)}",
                  f"  evictions {m['ctx_evictions']}  suspended {m.get('ctx_suspended', 0)}  restored {m.get('ctx_restored', 0)}  "
                  f"replayed tokens {m.get('ctx_replayed_tokens', 0)}  deferred {m.get('ctx_deferred', 0)}  "
                  f"gate holds {m.get('ctx_gate_holds', 0)}  dedup pages {m.get('ctx_dedup_pages', 0)}"]
    procs = status.get("process_table") or []
    if procs:
        lines.append("processes (busiest first)")
        lines += [f"  {p['id'][:8]}  {p['program'][:28]:28s} {p['user'][:12]:12s} {p['age_s']:8.1f}s  {p['tokens']:8d} tok"
                  for p in procs]
    fire = status.get("fire") or {}
    if fire:
        lines.append("per-fire probes                         count    mean us     max us")
        for k in FIRE_ORDER + sorted(set(fire) - set(FIRE_ORDER)):
            if k in fire:
                v = fire[k]
                pad = "  " if k.startswith("fire_execute_") and k != "fire_execute_total" else ""
                lines.append(f"  {pad + k:36s} {v['count']:7d} {v['mean_us']:10.1f} {v['max_us']:10.1f}")
    return "\n".join(lines)


def run_monitor(source, period: float = 1.0, out=None, iterations: int = -1, clear: bool = True) -> None:
    """`source`: an Engine, or any callable returning the status dictionary (a client's `model_status`)."""
    out = out or sys.stdout
    fetch: Callable[[], dict] = source if callable(source) else source.model_status
    history: dict = {}
    n = 0
    while iterations < 0 or n < iterations:
        try:
            text = render(fetch(), history)
        except Exception as e:  # noqa: BLE001 - keep the dashboard alive across a hiccup of the source
            text = f"status unavailable: {e}"
        out.write(("\x1b[2J\x1b[H" if clear else "") + text + "\n")
        out.flush()
        n += 1
        if iterations < 0 or n < iterations:
            time.sleep(period)
