"""wit-microbench: cost of the host API calls an inferlet makes, measured from inside one
(context create / fork / release, empty forward, messaging push+pull, model lookup).
Counterpart of inferlets/wit-microbench (benches/run_microbench.py)."""
import json
import time

from pie_b200.sdk import Context, Model, messaging, runtime

NAME = "wit-microbench"


async def main(args):
    n = int((args or {}).get("iters", 200))
    model = Model.load(runtime.models()[0])
    out = {}

    def timed(name, fn):
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        out[name + "_us"] = (time.perf_counter() - t0) / n * 1e6

    timed("model_load", lambda: Model.load(runtime.models()[0]))
    timed("context_create_release", lambda: Context(model).release())
    base = Context(model)
    timed("context_fork_release", lambda: base.fork().release())
    t0 = time.perf_counter()
    for _ in range(n):
        await base.forward().execute()
    out["empty_forward_us"] = (time.perf_counter() - t0) / n * 1e6
    t0 = time.perf_counter()
    for i in range(n):
        messaging.push("wit-microbench", "x")
        await messaging.pull("wit-microbench")
    out["push_pull_us"] = (time.perf_counter() - t0) / n * 1e6
    base.release()
    return json.dumps(out)
