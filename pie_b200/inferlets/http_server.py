"""http-server: request handler of a daemon (`launch_daemon`): every HTTP request launches this
program with {method, path, headers, body}; the returned JSON sets status, headers and body.
`POST /complete` with {"prompt": ...} generates a completion; anything else gets a small index.
Counterpart of inferlets/http-server/src/lib.rs (wasi:http incoming-handler)."""
import json

from ._common import load_model, make_sampler, prompt_context

NAME = "http-server"


async def main(req):
    req = req or {}
    method, path = req.get("method", "GET"), req.get("path", "/")
    if method == "POST" and path.startswith("/complete"):
        try:
            body = json.loads(req.get("body") or "{}")
        except json.JSONDecodeError:
            return json.dumps({"status": 400, "headers": {}, "body": "bad json"})
        model = load_model(body)
        ctx = prompt_context(model, body)
        text = await ctx.generate(make_sampler(body), max_tokens=int(body.get("max_tokens", 16))).collect_text()
        ctx.release()
        return json.dumps({"status": 200, "headers": {"content-type": "application/json"},
                           "body": json.dumps({"completion": text})})
    return json.dumps({"status": 200, "headers": {"content-type": "text/plain"},
                       "body": 'POST /complete {"prompt": ...}\n'})
