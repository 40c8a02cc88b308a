"""agent-swarm: a coordinator launches worker inferlets, hands each a task over a push/pull queue
and collects their answers from a results topic. Counterpart of inferlets/agent-swarm/src/lib.rs
(runtime.launch + messaging)."""
import asyncio
import json

from pie_b200.sdk import messaging, runtime

NAME = "agent-swarm"


async def main(args):
    args = args or {}
    role = args.get("role", "coordinator")
    swarm = args.get("swarm", runtime.instance_id())
    if role == "worker":
        task = json.loads(await messaging.pull(f"{swarm}/tasks"))
        answer = {"worker": args.get("index"), "task": task["id"], "result": str(task["text"])[::-1]}
        messaging.push(f"{swarm}/results", json.dumps(answer))
        return "done"
    tasks = args.get("tasks", ["alpha", "beta", "gamma"])
    workers = [runtime.launch(NAME, {"role": "worker", "swarm": swarm, "index": i}) for i in range(len(tasks))]
    for i, t in enumerate(tasks):
        messaging.push(f"{swarm}/tasks", json.dumps({"id": i, "text": t}))
    results = [json.loads(await messaging.pull(f"{swarm}/results")) for _ in tasks]
    await asyncio.gather(*[w.wait() for w in workers])
    return json.dumps({"results": sorted(results, key=lambda r: r["task"])})
