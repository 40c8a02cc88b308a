"""Workflows: a JSON DSL that composes inferlet processes, run by an async tree-walking executor.

Nodes (`{"op": ...}`):
  process  {program, input}                 run one inferlet; value = its return (JSON-decoded when possible)
  pipe     {steps: [...]}                   run in sequence; each step sees the previous value as `$prev`
  fork     {branches: [...]}                run concurrently; value = list of branch values
  map      {over, body}                     body once per element (`$item`, `$index`), concurrently
  fold     {over, init, body}               sequential reduction (`$acc`, `$item`)
  cond     {if, then, else}                 expression test
  iterate  {body, until, max}               repeat body (`$prev`, `$iter`) until the expression holds
  value    {value}                          literal / expression
Expressions are strings starting with `$` (variable paths like `$prev.answer`, `$item`) or small
comparisons `{"eq": [a, b]}`, `{"lt": ...}`, `{"contains": ...}`, `{"not": x}`, `{"len": x}`.
Workflows can be cancelled and attached to (events: node_started, node_done, return, error).
Counterpart of runtime/src/workflow.rs:1-22, workflow/executor.rs, workflow/expr.rs.
"""
from __future__ import annotations

import asyncio
import json
import uuid
from typing import Any, Callable, Dict, List, Optional


class WorkflowError(RuntimeError):
    pass


def evaluate(expr: Any, env: Dict[str, Any]) -> Any:
    if isinstance(expr, str) and expr.startswith("$"):
        path = expr[1:].split(".")
        if path[0] not in env:
            raise WorkflowError(f"unknown variable ${path[0]}")
        v = env[path[0]]
        for p in path[1:]:
            v = v[int(p)] if isinstance(v, list) else v[p]
        return v
    if isinstance(expr, dict) and len(expr) == 1:
        (k, a), = expr.items()
        ev = lambda x: evaluate(x, env)
        if k == "eq": return ev(a[0]) == ev(a[1])
        if k == "ne": return ev(a[0]) != ev(a[1])
        if k == "lt": return ev(a[0]) < ev(a[1])
        if k == "gt": return ev(a[0]) > ev(a[1])
        if k == "and": return all(ev(x) for x in a)
        if k == "or": return any(ev(x) for x in a)
        if k == "not": return not ev(a)
        if k == "len": return len(ev(a))
        if k == "contains": return ev(a[1]) in ev(a[0])
        if k == "concat": return "".join(str(ev(x)) for x in a)
    if isinstance(expr, dict):
        return {k: evaluate(v, env) for k, v in expr.items()}
    if isinstance(expr, list):
        return [evaluate(v, env) for v in expr]
    return expr


class _Run:
    def __init__(self, wid: str, username: str):
        self.id, self.username = wid, username
        self.listeners: List[Callable] = []
        self.task: Optional[asyncio.Task] = None
        self.procs: set = set()
        self.events: List[tuple] = []
        self.result: Any = None
        self.error: Optional[str] = None
        self.done = False

    def emit(self, event: str, value: Any) -> None:
        v = value if isinstance(value, str) else json.dumps(value)
        self.events.append((event, v))
        for cb in list(self.listeners):
            try:
                cb(self.id, event, v)
            except Exception:  # noqa: BLE001
                pass


class WorkflowExecutor:
    def __init__(self, engine):
        self.engine = engine
        self.runs: Dict[str, _Run] = {}

    def submit(self, spec: dict, username: str = "local", listener: Optional[Callable] = None) -> str:
        run = _Run("wf-" + uuid.uuid4().hex[:12], username)
        if listener:
            run.listeners.append(listener)
        self.runs[run.id] = run

        def start():
            run.task = self.engine.loop.create_task(self._drive(run, spec))
        self.engine.call_soon(start)
        return run.id

    def cancel(self, wid: str) -> bool:
        run = self.runs.get(wid)
        if run is None or run.done:
            return False
        self.engine.call_soon(lambda: run.task and run.task.cancel())
        return True

    def attach(self, wid: str, cb: Callable) -> bool:
        run = self.runs.get(wid)
        if run is None:
            return False
        for ev, v in run.events:
            cb(wid, ev, v)
        run.listeners.append(cb)
        return True

    def detach(self, wid: str, cb: Callable) -> bool:
        run = self.runs.get(wid)
        if run is None or cb not in run.listeners:
            return False
        run.listeners.remove(cb)
        return True

    def wait(self, wid: str, timeout: float = 60.0):
        import time
        t0 = time.time()
        run = self.runs[wid]
        while not run.done:
            if time.time() - t0 > timeout:
                raise TimeoutError(wid)
            time.sleep(0.005)
        if run.error:
            raise WorkflowError(run.error)
        return run.result

    async def _drive(self, run: _Run, spec: dict) -> None:
        try:
            run.result = await self._node(run, spec, {})
            run.emit("return", run.result)
        except asyncio.CancelledError:
            for p in list(run.procs):
                p.terminate()
            run.error = "cancelled"
            run.emit("error", "cancelled")
        except Exception as e:  # noqa: BLE001
            run.error = f"{type(e).__name__}: {e}"
            run.emit("error", run.error)
        finally:
            run.done = True

    async def _process(self, run: _Run, program: str, inp: Any) -> Any:
        proc = self.engine.launch(program, inp, username=run.username, capture_outputs=False)
        run.procs.add(proc)
        ev = asyncio.Event()
        loop = asyncio.get_running_loop()
        proc.on_done(lambda _p: loop.call_soon_threadsafe(ev.set))
        try:
            await ev.wait()
        finally:
            run.procs.discard(proc)
        if proc.error is not None:
            raise WorkflowError(f"{program}: {proc.error}")
        try:
            return json.loads(proc.result)
        except (json.JSONDecodeError, TypeError):
            return proc.result

    async def _node(self, run: _Run, node: dict, env: Dict[str, Any]) -> Any:
        op = node.get("op")
        run.emit("node_started", {"op": op})
        if op == "process":
            out = await self._process(run, node["program"], evaluate(node.get("input"), env))
        elif op == "value":
            out = evaluate(node.get("value"), env)
        elif op == "pipe":
            out = env.get("prev")
            for step in node["steps"]:
                out = await self._node(run, step, {**env, "prev": out})
        elif op == "fork":
            out = list(await asyncio.gather(*[self._node(run, b, dict(env)) for b in node["branches"]]))
        elif op == "map":
            items = evaluate(node["over"], env)
            out = list(await asyncio.gather(*[self._node(run, node["body"], {**env, "item": it, "index": i})
                                              for i, it in enumerate(items)]))
        elif op == "fold":
            out = evaluate(node.get("init"), env)
            for it in evaluate(node["over"], env):
                out = await self._node(run, node["body"], {**env, "acc": out, "item": it})
        elif op == "cond":
            branch = node["then"] if evaluate(node["if"], env) else node.get("else", {"op": "value", "value": None})
            out = await self._node(run, branch, env)
        elif op == "iterate":
            out = env.get("prev")
            for i in range(int(node.get("max", 8))):
                out = await self._node(run, node["body"], {**env, "prev": out, "iter": i})
                if "until" in node and evaluate(node["until"], {**env, "prev": out, "iter": i}):
                    break
        else:
            raise WorkflowError(f"unknown workflow op {op!r}")
        run.emit("node_done", {"op": op})
        return out
