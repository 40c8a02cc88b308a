"""launch-stress: corner cases of `runtime.launch`, run as caller or callee by `role`. Scenarios of
the caller: many children at once, a child that fails, a child that is cancelled, nested launches,
a child that outlives a short wait. Counterpart of inferlets/launch-stress/src/lib.rs."""
import asyncio
import json

from pie_b200.sdk import runtime

NAME = "launch-stress"


async def callee(d):
    kind = d.get("directive", "echo")
    if kind == "fail":
        raise RuntimeError("callee asked to fail")
    if kind == "sleep":
        await asyncio.sleep(float(d.get("seconds", 0.2)))
        return "slept"
    if kind == "nest":
        depth = int(d.get("depth", 1))
        if depth <= 0:
            return "leaf"
        child = runtime.launch(NAME, {"role": "callee", "directive": "nest", "depth": depth - 1})
        return "nest(" + await child.wait() + ")"
    return "echo:" + str(d.get("value", ""))


async def main(args):
    args = args or {}
    if args.get("role") == "callee":
        return await callee(args)
    scenario, out = args.get("scenario", "fanout"), {}
    if scenario == "fanout":
        n = int(args.get("n", 16))
        kids = [runtime.launch(NAME, {"role": "callee", "value": i}) for i in range(n)]
        res = await asyncio.gather(*[k.wait() for k in kids])
        out = {"results": list(res), "distinct_pids": len({k.pid for k in kids})}
    elif scenario == "failure":
        kid = runtime.launch(NAME, {"role": "callee", "directive": "fail"})
        try:
            await kid.wait()
            out = {"error": None}
        except Exception as e:  # noqa: BLE001
            out = {"error": str(e)}
    elif scenario == "cancel":
        kid = runtime.launch(NAME, {"role": "callee", "directive": "sleep", "seconds": 30})
        await asyncio.sleep(0.05)
        kid.cancel()
        try:
            await asyncio.wait_for(kid.wait(), 5)
            out = {"cancelled": False}
        except Exception:  # noqa: BLE001
            out = {"cancelled": True}
    elif scenario == "nested":
        kid = runtime.launch(NAME, {"role": "callee", "directive": "nest", "depth": int(args.get("depth", 3))})
        out = {"result": await kid.wait()}
    elif scenario == "unknown-program":
        try:
            runtime.launch("no-such-program", {})
            out = {"error": None}
        except Exception as e:  # noqa: BLE001
            out = {"error": str(e)}
    return json.dumps({"scenario": scenario, **out})
