"""async-lm: asynchronous function calling (AsyncLM, arXiv:2412.07017). The model dispatches tool
calls without blocking, keeps generating, and the results are injected into the live context when
they arrive. Token protocol (text markers): `[CALL] id [HEAD] code [END]` dispatches, `[TRAP][END]`
waits for every outstanding call, `[INTR] id [HEAD] value [END]` is written by the runtime only.
The inferlet scans the generated text with a small state machine, runs each call as a concurrent
task, and appends `[INTR]` frames between decode steps. Tools here are local functions (this build
has no outbound network by default). Counterpart of inferlets/async-lm/src/lib.rs."""
import asyncio
import json
import re

from ._common import load_model, make_sampler, prompt_context

NAME = "async-lm"

CALL = re.compile(r"\[CALL\]\s*(\w+)\s*\[HEAD\]\s*(.*?)\s*\[END\]", re.S)
TRAP = "[TRAP][END]"


async def run_tool(code: str, latency: float) -> str:
    await asyncio.sleep(latency)
    name, _, arg = code.partition("(")
    arg = arg.rstrip(")").strip("\"' ")
    tools = {"time": lambda a: "12:00", "weather": lambda a: f"sunny in {a or 'here'}",
             "upper": lambda a: a.upper(), "len": lambda a: str(len(a))}
    fn = tools.get(name.strip())
    return fn(arg) if fn else f"unknown tool {name.strip()}"


async def main(args):
    args = args or {}
    model = load_model(args)
    tok = model.tokenizer()
    ctx = prompt_context(model, args, "Use tools when needed.")
    max_tokens, chunk = int(args.get("max_tokens", 48)), int(args.get("chunk", 8))
    latency = float(args.get("tool_latency_s", 0.01))
    scripted = list(args.get("scripted_calls", []))      # text the test injects as if the model had written it
    text, seen_to, pending, injected, produced, traps = "", 0, {}, [], 0, 0
    sampler = make_sampler(args)
    while produced < max_tokens:
        toks = await ctx.generate(sampler, max_tokens=min(chunk, max_tokens - produced)).stop([]).collect_tokens()
        produced += len(toks)
        text += tok.decode(toks)
        if scripted:                                      # deterministic driver for tests / demos
            frame = scripted.pop(0)
            ctx.append(tok.encode(frame))
            text += frame
        for m in CALL.finditer(text, seen_to):            # dispatch: do not wait
            cid, code = m.group(1), m.group(2)
            if cid not in pending:
                pending[cid] = asyncio.ensure_future(run_tool(code, latency))
        trap = TRAP in text[seen_to:]
        seen_to = len(text)
        if trap and pending:                              # the model asked to wait for every call
            traps += 1
            await asyncio.wait(list(pending.values()))
        for cid in [c for c, f in pending.items() if f.done()]:
            frame = f"[INTR] {cid} [HEAD] {pending.pop(cid).result()} [END]"
            ctx.append(tok.encode(frame))                 # injected between decode steps
            injected.append(frame)
            text += frame
            seen_to = len(text)
    for f in pending.values():
        f.cancel()
    ctx.release()
    return json.dumps({"tokens": produced, "calls": len(injected) + len(pending), "injected": injected, "traps": traps})
