"""`pie serve --monitor`: a terminal view of model_status refreshed once per second (KV pages,
batches, latency, speculation hits, market). Counterpart of server/src/cli/monitor/* (TUI)."""
from __future__ import annotations

import sys
import time

BARS = " ▁▂▃▄▅▆▇█"


def spark(values, width=40):
    vals = list(values)[-width:]
    hi = max(vals) if vals and max(vals) > 0 else 1.0
    return "".join(BARS[min(8, int(8 * v / hi))] for v in vals)


def render(status: dict, history: dict) -> str:
    lines = [f"pie_b200 {status['version']}  up {status['uptime_s']:.0f}s  processes {status['processes']}"]
    for name, m in status["models"].items():
        h = history.setdefault(name, {"lat": [], "tok": [], "last_tokens": m["total_tokens"]})
        h["lat"].append(m["last_batch_latency_us"] / 1e3)
        h["tok"].append(m["total_tokens"] - h["last_tokens"])
        h["last_tokens"] = m["total_tokens"]
        used, total = m["kv_pages_used"], max(1, m["kv_pages_total"])
        lines += [f"[{name}] kv {used}/{total} ({100 * used / total:.1f}%)  contexts {m['contexts']}  "
                  f"batches {m['total_batches']}  avg {m['avg_batch_latency_us'] / 1e3:.2f} ms",
                  f"  tokens/s  {spark(h['tok'])} {h['tok'][-1]}",
                  f"  batch ms  {spark(h['lat'])} {h['lat'][-1]:.2f}",
                  f"  staged hits {m['bypass_hits']}  chain submits {m['chain_submits']}  drops {m['chain_drops']}  "
                  f"price {m['market_price']:.2f}  evictions {m['ctx_evictions']}"]
    return "\n".join(lines)


def run_monitor(engine, period: float = 1.0, out=sys.stdout, iterations: int = -1) -> None:
    history: dict = {}
    n = 0
    while iterations < 0 or n < iterations:
        text = render(engine.model_status(), history)
        out.write("\x1b[2J\x1b[H" + text + "\n")
        out.flush()
        n += 1
        time.sleep(period)
