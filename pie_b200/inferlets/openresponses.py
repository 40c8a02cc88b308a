"""openresponses: request handler of a daemon that speaks the OpenResponses shape.
`POST /responses` with {"model", "input": [{"type":"message","role","content"}...] | "text",
"max_output_tokens", "temperature", "top_p", "stream"} answers with a `response` object whose
`output` holds one assistant message; with "stream": true the body is a server-sent-event
transcript (response.created, response.output_text.delta ..., response.completed).
Counterpart of inferlets/openresponses/src/{lib,handler,streaming,types}.rs."""
import json
import time
import uuid

from pie_b200.sdk import Context

from ._common import load_model, make_sampler

NAME = "openresponses"


def _messages(inp):
    if isinstance(inp, str):
        return [("user", inp)]
    out = []
    for item in inp or []:
        if item.get("type", "message") != "message":
            continue
        content = item.get("content", "")
        if isinstance(content, list):
            content = "".join(p.get("text", "") for p in content if p.get("type") in ("input_text", "output_text", "text"))
        out.append((item.get("role", "user"), content))
    return out


async def main(req):
    req = req or {}
    if req.get("method", "POST") != "POST" or not req.get("path", "/responses").startswith("/responses"):
        return json.dumps({"status": 404, "headers": {}, "body": json.dumps({"error": {"message": "POST /responses"}})})
    try:
        body = json.loads(req.get("body") or "{}")
    except ValueError:
        return json.dumps({"status": 400, "headers": {}, "body": json.dumps({"error": {"message": "invalid JSON"}})})
    msgs = _messages(body.get("input"))
    if not msgs:
        return json.dumps({"status": 400, "headers": {}, "body": json.dumps({"error": {"message": "input is required"}})})
    model = load_model({} if body.get("model") in (None, "auto") else {"model": body["model"]})
    ctx = Context(model)
    if body.get("instructions"):
        ctx.system(body["instructions"])
    for role, text in msgs:
        {"system": ctx.system, "assistant": ctx.assistant}.get(role, ctx.user)(text)
    ctx.cue()
    n_in = len(ctx.buffer)
    args = {k: body[k] for k in ("temperature", "top_p") if k in body}
    tokens = await ctx.generate(make_sampler(args), max_tokens=int(body.get("max_output_tokens", 32))).collect_tokens()
    ctx.release()
    tok = model.tokenizer()
    text = tok.decode(tokens)
    rid, mid = "resp_" + uuid.uuid4().hex[:24], "msg_" + uuid.uuid4().hex[:24]
    resp = {"id": rid, "object": "response", "created_at": int(time.time()), "status": "completed", "model": model.name,
            "output": [{"type": "message", "id": mid, "role": "assistant", "status": "completed",
                        "content": [{"type": "output_text", "text": text, "annotations": []}]}],
            "usage": {"input_tokens": n_in, "output_tokens": len(tokens), "total_tokens": n_in + len(tokens)}}
    if not body.get("stream"):
        return json.dumps({"status": 200, "headers": {"content-type": "application/json"}, "body": json.dumps(resp)})
    events = [("response.created", {"response": dict(resp, status="in_progress", output=[])})]
    for i, t in enumerate(tokens):
        events.append(("response.output_text.delta", {"item_id": mid, "output_index": 0, "content_index": 0,
                                                      "delta": tok.decode([t]), "sequence_number": i + 1}))
    events.append(("response.completed", {"response": resp}))
    sse = "".join(f"event: {name}\ndata: {json.dumps(dict(data, type=name))}\n\n" for name, data in events)
    return json.dumps({"status": 200, "headers": {"content-type": "text/event-stream"}, "body": sse})
