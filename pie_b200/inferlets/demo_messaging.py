"""demo-messaging: push/pull queue and broadcast/subscribe between the roles of one program.
role=producer pushes `count` messages to `topic`; role=consumer pulls them; role=both does both
inside one process. Counterpart of inferlets/demo-messaging/src/lib.rs."""
import json

from pie_b200.sdk import messaging

NAME = "demo-messaging"


async def main(args):
    args = args or {}
    topic, count, role = args.get("topic", "demo"), int(args.get("count", 3)), args.get("role", "both")
    got = []
    if role in ("producer", "both"):
        for i in range(count):
            messaging.push(topic, f"msg-{i}")
    if role in ("consumer", "both"):
        for _ in range(count):
            got.append(await messaging.pull(topic))
    return json.dumps({"received": got})
