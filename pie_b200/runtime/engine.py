"""The engine: models + drivers + KV page manager + batch schedulers + inferlet processes in
one address space.

`Engine` is the embedded public API (the `pie serve` / `pie run` front ends and the
benchmark use it):

    eng = Engine(EngineConfig(...))
    eng.add_model("llama", driver)                  # a TorchDriver / MockDriver / DummyDriver
    eng.register_program("text-completion", main)   # async def main(input) -> str
    proc = eng.launch("text-completion", {"prompt": ...})
    result = eng.wait(proc)

Counterpart of runtime/src/bootstrap.rs:186-291 (wiring order), runtime/src/model.rs:18-95
(model registry), server/src/serve/lifecycle.rs:50-66 (driver watchdog) and
runtime/src/server/handler.rs:48-332 (model_status metrics).
"""
from __future__ import annotations

import asyncio
import logging
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

from ..driver.schema import Capabilities, CopyRequest
from .cohort import DecodeCohort
from .context import ContextManager
from .inference import InferenceService
from .market import Market
from .messaging import Messaging
from .pagestore import PageStore
from .process import Process, current_process
from . import telemetry
from .scheduler import BatchScheduler

VERSION = "0.1.0"


@dataclass
class EngineConfig:
    batch_policy: str = "adaptive"
    speculation_depth: int = 1
    system_spec_tokens: int = 0               # > 0: runtime-side prompt-look-up drafts per generator step (replaces the chain)
    max_concurrent_processes: int = 4096
    request_timeout_secs: float = 120.0
    default_token_budget: Optional[int] = None
    watchdog_interval_s: float = 1.0
    swap_pages: int = 0
    default_endowment_pages: int = 64
    admission_oversubscription_factor: float = 4.0
    fs_policy: str = "scratch"               # "scratch": private directory per process | "none"
    scratch_root: Optional[str] = None
    adapter_dir: Optional[str] = None        # where named adapters are saved (<name>.safetensors)
    network_allow: tuple = ()                # CIDR[:port] rules inferlets may connect to; empty = no network


class ModelEntry:
    def __init__(self, name: str, drivers: list, tokenizer=None, instruct=None, arch: str = ""):
        self.name, self.drivers, self.tokenizer, self.instruct = name, drivers, tokenizer, instruct
        self.caps: List[Capabilities] = [d.capabilities() for d in drivers]
        self.page_size = self.caps[0].kv_page_size
        self.arch = arch or self.caps[0].arch_name
        self.ctxm: ContextManager = None
        self.adapters = None          # AdapterService
        self.media = None             # MediaRegistry when every driver declares an encoder
        self.inference: InferenceService = None
        self.schedulers: List[BatchScheduler] = []


class Engine:
    def __init__(self, config: Optional[EngineConfig] = None):
        self.config = config or EngineConfig()
        self.log = logging.getLogger("pie_b200")
        self.models: Dict[str, ModelEntry] = {}
        self.programs: Dict[str, Callable] = {}
        self.confined_programs: set = set()
        self.program_resolver: Optional[Callable[[str], bool]] = None   # called for programs that are not registered
        self.manifests: Dict[str, dict] = {}
        self.processes: Dict[str, Process] = {}
        self.messaging: Messaging = None
        self.loop = asyncio.new_event_loop()
        self.admission: asyncio.Semaphore = None
        self._ready = threading.Event()
        self.thread = threading.Thread(target=self._run_loop, name="pie-runtime", daemon=True)
        self.thread.start()
        self._ready.wait()
        self._watchdog_stop = threading.Event()
        self._watchdog = threading.Thread(target=self._watch, name="pie-watchdog", daemon=True)
        self._watchdog.start()
        self.t_start = time.time()
        self.adapters: Dict[str, dict] = {}
        self.mcp_servers: Dict[str, Any] = {}

    # ------------------------------------------------------------------ event loop
    def _run_loop(self) -> None:
        asyncio.set_event_loop(self.loop)
        self.messaging = Messaging()
        self.admission = asyncio.Semaphore(self.config.max_concurrent_processes)
        self._ready.set()
        self.loop.run_forever()

    def call_soon(self, fn, *args) -> None:
        self.loop.call_soon_threadsafe(fn, *args)

    # ------------------------------------------------------------------ models
    def add_model(self, name: str, drivers, tokenizer=None, instruct=None) -> ModelEntry:
        """Register a model served by one driver per data-parallel replica group."""
        drivers = drivers if isinstance(drivers, (list, tuple)) else [drivers]
        entry = ModelEntry(name, list(drivers), tokenizer, instruct)
        stores = [PageStore(c.total_pages) for c in entry.caps]
        swap = min((c.swap_pool_size for c in entry.caps), default=0)

        def copy_fn(driver_idx: int, req: CopyRequest) -> None:
            entry.drivers[driver_idx].copy(req)

        entry.ctxm = ContextManager(name, entry.page_size, stores, copy_fn, swap_pages=swap,
                                    rs_slots=[c.rs_cache_slots for c in entry.caps],
                                    rs_copy_fn=lambda d, src, dst: entry.drivers[d].copy_rs(src, dst))
        if all(getattr(c, "media", ()) for c in entry.caps):
            from .media import MediaRegistry
            entry.media = entry.ctxm.media = MediaRegistry(entry.drivers)
        from .adapter import AdapterService
        entry.adapters = AdapterService(entry.drivers, self.config.adapter_dir)
        for i, (drv, caps) in enumerate(zip(entry.drivers, entry.caps)):
            sched = BatchScheduler(drv, caps, entry.page_size, self.config.batch_policy,
                                   name=f"pie-sched-{name}-{i}")
            sched.expected_cohort = entry.ctxm.pinned_count
            sched.delivery_guard = entry.ctxm.lock
            # the array-form decode cohort does not carry recurrent-state slots: such models step per request
            sched.cohort = (DecodeCohort(entry.ctxm, entry.page_size, caps.max_forward_requests)
                            if not caps.rs_cache_slots and getattr(caps, "cohort_decode", True) and hasattr(drv, "decode_async") else None)
            entry.schedulers.append(sched)
        entry.inference = InferenceService(entry.ctxm, entry.schedulers,
                                           0 if self.config.system_spec_tokens > 0 else self.config.speculation_depth)
        entry.inference.system_spec_tokens = self.config.system_spec_tokens
        entry.inference.cohorts = [s.cohort for s in entry.schedulers] if all(
            s.cohort is not None for s in entry.schedulers) else []
        for s in entry.schedulers:
            if s.cohort is not None:
                s.cohort.on_finish = lambda st, e=entry: self._charge(e, st.ctx_id, getattr(st, "kept", 0))
        entry.inference.on_tokens = lambda cid, n, e=entry: self._charge(e, cid, n)
        entry.market = Market(sum(c.total_pages for c in entry.caps), self.config.default_endowment_pages,
                              self.config.admission_oversubscription_factor)
        entry.ctxm.market = entry.market
        for i, s in enumerate(entry.schedulers):
            s.post_fire_hooks.append(lambda ctx_ids, e=entry, d=i: self._market_tick(e, d, ctx_ids))
        self.models[name] = entry
        return entry

    def _market_tick(self, entry: ModelEntry, driver: int, ctx_ids) -> None:
        batch = []
        with entry.ctxm.lock:              # once for the batch, not once per context
            for cid in ctx_ids:
                ctx = entry.ctxm.contexts.get(int(cid))
                if ctx is not None:
                    try:
                        batch.append((ctx.id, ctx.owner, ctx.bid, entry.ctxm.effective_pages(ctx.id)))
                    except Exception:  # noqa: BLE001
                        pass
        entry.market.tick(entry.ctxm.pages_used(driver), batch)

    def _charge(self, entry: ModelEntry, cid: int, n: int) -> None:
        ctx = entry.ctxm.contexts.get(cid)
        if ctx is not None:
            p = self.processes.get(ctx.owner)
            if p is not None:
                p.charge_tokens(n)
                entry.market.debit_tokens(ctx.owner, n)

    def model(self, name: Optional[str] = None) -> ModelEntry:
        if name is None:
            name = next(iter(self.models))
        if name not in self.models:
            raise KeyError(f"model {name!r} is not loaded")
        return self.models[name]

    # ------------------------------------------------------------------ programs / processes
    def register_program(self, name: str, entry: Callable, manifest: Optional[dict] = None,
                         confined: bool = False) -> None:
        """`confined`: the program did not ship with the package (upload, disk cache): its processes run under
        the audit-hook confinement of `runtime/policy.py`."""
        if confined:
            self.confined_programs.add(name)
        else:
            self.confined_programs.discard(name)
        self.programs[name] = entry
        self.manifests[name] = manifest or {"package": {"name": name, "version": "0.1.0"}}

    def launch(self, program: str, input_value: Any = None, username: str = "local",
               capture_outputs: bool = True, token_budget: Optional[int] = None,
               parent: Optional[str] = None, listener: Optional[Callable] = None) -> Process:
        if program not in self.programs and program.split("@")[0] not in self.programs and self.program_resolver:
            self.program_resolver(program)       # e.g. the program store's registry download
        if program not in self.programs:
            base = program.split("@")[0]
            if base not in self.programs:
                raise KeyError(f"program {program!r} is not installed")
            program = base
        proc = Process(self, program, self.programs[program], input_value, username, capture_outputs,
                       token_budget if token_budget is not None else self.config.default_token_budget, parent)
        if listener is not None:
            proc.listeners.append(listener)
        self.processes[proc.id] = proc

        def start():
            proc.task = self.loop.create_task(proc.run())

        self.call_soon(start)
        return proc

    async def admit_process(self, proc: Process) -> None:
        """KV admission: wait until the process's page claim fits every model's market."""
        for entry in self.models.values():
            loop = asyncio.get_running_loop()
            fut = loop.create_future()
            ok = entry.market.try_admit(proc.id, None, proc.token_budget,
                                        on_admit=lambda f=fut: loop.call_soon_threadsafe(
                                            lambda: f.done() or f.set_result(True)))
            if not ok:
                await fut

    def release_process(self, proc: Process) -> None:
        for entry in self.models.values():
            entry.market.release(proc.id)
            for cid in list(entry.ctxm.by_owner.get(proc.id, ())):
                entry.inference.drop_context(cid)
            entry.ctxm.destroy_owner(proc.id)
            if entry.adapters is not None:
                entry.adapters.release_owner(proc.id)

    def wait(self, proc: Process, timeout: Optional[float] = None) -> str:
        ev = threading.Event()
        proc.on_done(lambda _p: ev.set())
        if not ev.wait(timeout):
            raise TimeoutError(f"process {proc.id} still running after {timeout}s")
        if proc.error is not None:
            raise RuntimeError(proc.error)
        return proc.result

    def run(self, program: str, input_value: Any = None, timeout: Optional[float] = None, **kw) -> str:
        return self.wait(self.launch(program, input_value, **kw), timeout)

    def terminate(self, process_id: str) -> bool:
        p = self.processes.get(process_id)
        if p is None:
            return False
        self.call_soon(p.terminate)
        return True

    def list_processes(self) -> List[dict]:
        return [p.stats() for p in self.processes.values() if not p.finished]

    # ------------------------------------------------------------------ supervision
    def _watch(self) -> None:
        """Poll driver health; when a driver died, abort its channels so that every in-flight
        and future submit fails fast instead of hanging."""
        while not self._watchdog_stop.wait(self.config.watchdog_interval_s):
            for entry in self.models.values():
                for drv, sched in zip(entry.drivers, entry.schedulers):
                    try:
                        ok = drv.health()
                    except Exception as e:  # noqa: BLE001
                        ok = False
                        self.log.error("driver of model %s failed its health check: %s", entry.name, e)
                    if not ok and sched.aborted is None:
                        sched.abort(RuntimeError(f"driver of model {entry.name} died"))

    def model_status(self) -> dict:
        out = {"version": VERSION, "uptime_s": time.time() - self.t_start, "models": {}}
        for name, e in self.models.items():
            m = {"kv_pages_total": sum(c.total_pages for c in e.caps),
                 "kv_pages_used": sum(e.ctxm.pages_used(i) for i in range(len(e.drivers))),
                 "contexts": len(e.ctxm.contexts), "snapshots": len(e.ctxm.snapshots)}
            for k in ("total_batches", "total_requests", "total_tokens", "cum_latency_us", "failed_batches",
                      "chunked_requests"):
                m[k] = sum(s.stats[k] for s in e.schedulers)
            m["last_batch_latency_us"] = max((s.stats["last_latency_us"] for s in e.schedulers), default=0.0)
            m["avg_batch_latency_us"] = m["cum_latency_us"] / max(1, m["total_batches"])
            m["batch_size_hist"] = [sum(s.stats["batch_size_hist"][i] for s in e.schedulers) for i in range(8)]
            m.update(e.inference.stats)
            m.update({"market_price": e.market.clearing_price, "market_ticks": e.market.ticks,
                      "market_rent": e.market.total_rent, "market_waiting": len(e.market.waiting)})
            m.update({f"ctx_{k}": v for k, v in e.ctxm.counters.items()})
            if e.media is not None:          # encoded clips: encoder runs, content hits, slots in use, encoder rows held
                m.update({f"media_{k}": v for k, v in e.media.stats().items()})
            out["models"][name] = m
        live = [p for p in self.processes.values() if not p.finished]
        out["processes"] = len(live)
        # the busiest live processes and the scheduler's per-fire probe tree (when telemetry is on)
        out["process_table"] = [
            {"id": p.id, "program": p.program, "user": p.username, "age_s": round(time.time() - p.t_start, 1),
             "tokens": p.tokens_used}
            for p in sorted(live, key=lambda q: -q.tokens_used)[:12]]
        tel = telemetry.get()
        if tel.enabled:
            snap = tel.snapshot()
            out["fire"] = {k: v for k, v in snap["probes"].items() if k.startswith(("fire_", "driver_"))}
            out["counters"] = snap["counters"]
        return out

    def metrics_text(self) -> str:
        """Prometheus exposition of `model_status` plus the telemetry counters and probes."""
        from . import telemetry
        st = self.model_status()
        lines = [f"pie_b200_uptime_seconds {st['uptime_s']:.3f}", f"pie_b200_processes {st['processes']}"]
        for name, m in st["models"].items():
            for k, v in m.items():
                if isinstance(v, bool):
                    v = int(v)
                if isinstance(v, (int, float)):
                    lines.append(f'pie_b200_model_{k}{{model="{name}"}} {v:g}')
                elif isinstance(v, list) and all(isinstance(x, (int, float)) for x in v):
                    lines += [f'pie_b200_model_{k}{{model="{name}",bucket="{i}"}} {x:g}' for i, x in enumerate(v)]
        return "\n".join(lines) + "\n" + telemetry.get().prometheus()

    def shutdown(self) -> None:
        self._watchdog_stop.set()
        for p in list(self.processes.values()):
            if not p.finished:
                self.call_soon(p.terminate)
        for e in self.models.values():
            for s in e.schedulers:
                s.shutdown()
            if e.media is not None:
                e.media.close()
            for d in e.drivers:
                try:
                    d.shutdown()
                except Exception:  # noqa: BLE001
                    pass
        self.loop.call_soon_threadsafe(self.loop.stop)
        self.thread.join(timeout=5)
