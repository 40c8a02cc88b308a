"""Benchmark harness for the serving configurations (synthetic random-token prompts,
random-init weights).

Two measurements of the same decode workload:

* device-only (`run_device_decode`): every step's integer inputs are staged on the device
  beforehand, the sampled tokens of step k are fed to step k+1 on the device, and K steps are
  bracketed by CUDA events - the kernel path alone.
* end to end (`run_engine_workload`): N concurrent `text-completion-bench` inferlets through
  the engine's public API; every fire copies its inputs from pinned host memory and reads the
  sampled tokens back. Gives output tokens/s over a window of K steady-state decode fires,
  whole-workload tokens/s, p50 TTFT and p50 inter-token latency.

The reference's bench driver is benches/pie_bench.py (requests/s, output tok/s, latency
percentiles; it has no TTFT/ITL capture).
"""
from __future__ import annotations

import json
import statistics
import subprocess
import threading
import time
from typing import List, Optional

import numpy as np
import torch

from ..driver.schema import SamplerKind, SamplerSpec
from ..runtime.scheduler import PendingRequest, fold


def make_prompts(n: int, lo: int, hi: int, vocab: int, seed: int = 1) -> List[List[int]]:
    rng = np.random.default_rng(seed)
    lens = rng.integers(lo, hi + 1, n)
    return [rng.integers(0, vocab, int(l)).tolist() for l in lens]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.proc = None
        self.lines: List[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms), "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._t = threading.Thread(target=self._read, daemon=True)
            self._t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=3)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


class PageAllocator:
    """Hands out page ids for harness-owned synthetic contexts."""

    def __init__(self, num_pages: int):
        self.next, self.num_pages = 0, num_pages

    def alloc(self, n: int) -> List[int]:
        if self.next + n > self.num_pages:
            raise RuntimeError(f"bench needs more KV pages than the pool has ({self.num_pages})")
        out = list(range(self.next, self.next + n))
        self.next += n
        return out


def prefill_contexts(driver, prompts: List[List[int]], out_tokens: int, sampler: SamplerSpec):
    """Prefill every prompt through the driver (batches bounded by its limits). Returns the
    per-context page lists and the first sampled token of each."""
    ps = driver.page_size
    alloc = PageAllocator(driver.kv.num_pages)
    pages = [alloc.alloc(-(-(len(p) + out_tokens + 1) // ps)) for p in prompts]
    first = [0] * len(prompts)
    order = sorted(range(len(prompts)), key=lambda i: len(prompts[i]))
    batch, tokens = [], 0
    t_fire = []

    def fire():
        nonlocal batch, tokens
        if not batch:
            return
        items = [PendingRequest(i, prompts[i], list(range(len(prompts[i]))), pages[i], 0,
                                [(len(prompts[i]) - 1, sampler)]) for i in batch]
        t0 = time.perf_counter()
        resp = driver.fire_batch(fold(items, ps))
        t_fire.append((time.perf_counter() - t0, tokens))
        for i, s in zip(batch, resp.slots):
            first[i] = s.token
        batch, tokens = [], 0

    for i in order:
        n = len(prompts[i])
        if tokens + n > driver.max_tokens or len(batch) + 1 > driver.max_requests:
            fire()
        batch.append(i)
        tokens += n
    fire()
    return pages, first, t_fire


def decode_request(driver, prompts, pages, tokens, step: int, sampler: SamplerSpec):
    items = [PendingRequest(i, [tokens[i]], [len(prompts[i]) + step], pages[i], len(prompts[i]) + step,
                            [(0, sampler)]) for i in range(len(prompts))]
    return fold(items, driver.page_size)


def run_pipelined_decode(driver, prompts, out_tokens: int, sampler: SamplerSpec, warmup: int, steps: int,
                         comm=None, barrier=None):
    """Device-timed decode through `decode_async` (the path the engine's cohort uses): step s is
    launched with its tokens fed on the device from step s-1, the host only trails one step behind
    to recycle its input slab. W untimed + K timed steps bracketed by synchronise (+ barrier and
    max over ranks under tensor parallelism) and CUDA events on the launching stream."""
    from ..driver.executor import CohortStep
    ps = driver.page_size
    pages, first, t_prefill = prefill_contexts(driver, prompts, out_tokens, sampler)
    r = len(prompts)
    plen = np.array([len(p) for p in prompts], dtype=np.int64)
    maxp = max(len(p) for p in pages)
    table = np.zeros((r, maxp), np.int32)
    for i, p in enumerate(pages):
        table[i, :len(p)] = p
    cols = np.arange(maxp, dtype=np.int32)[None, :]
    rng = np.random.default_rng(3)

    def make(step: int) -> CohortStep:
        kv_after = (plen + step + 1).astype(np.int32)
        used = (kv_after + ps - 1) // ps
        indptr = np.zeros(r + 1, np.int32)
        np.cumsum(used, out=indptr[1:])
        return CohortStep(
            r=r, host_tokens=np.asarray(first, np.int32),
            src_row=(np.arange(r, dtype=np.int32) if step > 0 else np.full(r, -1, np.int32)),
            positions=(plen + step).astype(np.int32), kv_lens=kv_after, page_indptr=indptr,
            page_indices=table[cols < used[:, None]],
            temperature=np.full(r, sampler.temperature, np.float32),
            top_k=np.full(r, sampler.top_k if sampler.kind.name.startswith("TOP_K") else 0, np.int32),
            top_p=np.full(r, sampler.top_p if "TOP_P" in sampler.kind.name else 1.0, np.float32),
            min_p=np.zeros(r, np.float32), seeds=rng.integers(1, 2**62, r, dtype=np.int64))

    prev = None
    ms = None
    ev0 = ev1 = None
    for s in range(warmup + steps):
        if s == warmup:
            if prev is not None:
                prev.wait()
            if comm is not None:
                comm.mark(False)
            else:
                torch.cuda.synchronize()
                if barrier is not None:     # data-parallel replicas start the timed region together
                    barrier()
                    torch.cuda.synchronize()
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record()
        h = driver.decode_async(make(s), s & 1)
        if prev is not None:
            prev.wait()
        prev = h
    if comm is not None:
        ms = comm.mark(True)
    else:
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1)
        if barrier is not None:
            barrier()
    prev.wait()
    driver.check_status_host()
    prefill_tokens = sum(t for _, t in t_prefill)
    prefill_s = sum(d for d, _ in t_prefill)
    rb = driver._bucket(r) if driver.use_graphs else r
    return {"ms_total": ms, "ms_per_step": ms / steps, "tokens_per_s": r * steps / (ms / 1e3),
            "prefill_tokens_per_s": prefill_tokens / max(prefill_s, 1e-9), "rb": rb}


def run_device_decode(driver, prompts, out_tokens: int, sampler: SamplerSpec, warmup: int, steps: int,
                      barrier=None):
    """Device-only decode: W untimed + K timed steps, CUDA events on the launching stream."""
    pages, first, t_prefill = prefill_contexts(driver, prompts, out_tokens, sampler)
    staged = [driver.stage_decode(decode_request(driver, prompts, pages, first, s, sampler))
              for s in range(warmup + steps)]
    driver.sampled[:len(first)].copy_(torch.tensor(first, dtype=torch.int32))
    for s in range(warmup):
        driver.replay_staged(staged[s], feed_sampled=True)
    torch.cuda.synchronize()
    if barrier:
        barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    ev0.record()
    for s in range(warmup, warmup + steps):
        driver.replay_staged(staged[s], feed_sampled=True)
    ev1.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    from .. import ops
    ops.check_kernel_status(driver.device)
    ms = ev0.elapsed_time(ev1)
    prefill_tokens = sum(t for _, t in t_prefill)
    prefill_s = sum(d for d, _ in t_prefill)
    return {"ms_total": ms, "ms_per_step": ms / steps, "tokens_per_s": len(prompts) * steps / (ms / 1e3),
            "prefill_tokens_per_s": prefill_tokens / max(prefill_s, 1e-9), "rb": staged[0]["rb"]}


def run_engine_workload(engine, model_name: str, prompts, out_tokens: int, sampler_args: dict,
                        window_skip: int, window_steps: int, timeout: float = 1800.0, extra_args=None):
    """All inferlets at once through the public API. Returns e2e metrics. `extra_args`: per-inferlet
    overrides, a dict for all or a callable index -> dict (e.g. {"per_step": True} for the
    inferlet-driven loop, or a JSON-schema constraint on some of them)."""
    entry = engine.model(model_name)
    fires = []   # (t_end, n_requests, n_tokens, latency)

    def on_batch(n_requests, n_tokens, lat, kind):
        fires.append((time.perf_counter(), n_requests, n_tokens, lat))

    for s in entry.schedulers:
        s.on_batch = on_batch
    t_launch = time.perf_counter()
    def extra(i):
        if extra_args is None:
            return {}
        return extra_args(i) if callable(extra_args) else extra_args
    procs = [engine.launch("text-completion-bench",
                           dict(prompt_tokens=p, max_tokens=out_tokens, **sampler_args, **extra(i)))
             for i, p in enumerate(prompts)]
    results = [json.loads(engine.wait(p, timeout)) for p in procs]
    t_done = time.perf_counter()
    for s in entry.schedulers:
        s.on_batch = None
    total_out = sum(r["n_tokens"] for r in results)
    ttft = [r["stamps"][0] - t_launch for r in results if r["stamps"]]
    itl = [b - a for r in results for a, b in zip(r["stamps"], r["stamps"][1:])]
    # steady-state decode window: fires that are pure decode (one token per request)
    dec = [f for f in fires if f[1] == f[2]]
    out = {"total_out_tokens": total_out, "wall_s": t_done - t_launch,
           "workload_tokens_per_s": total_out / (t_done - t_launch),
           "p50_ttft_s": statistics.median(ttft) if ttft else None,
           "p50_itl_s": statistics.median(itl) if itl else None,
           "fires": len(fires), "decode_fires": len(dec)}
    # steady-state decode window: consecutive pure-decode fires that carry (nearly) all requests,
    # after skipping `window_skip` of them; shorter than asked when the workload leaves fewer
    full = [i for i, f in enumerate(fires) if f[1] == f[2] and f[1] >= 0.9 * len(prompts)]
    runs, cur = [], []
    for i in full:
        if cur and i != cur[-1] + 1:
            runs.append(cur)
            cur = []
        cur.append(i)
    if cur:
        runs.append(cur)
    if runs:
        best = max(runs, key=len)
        skip = min(window_skip, max(0, len(best) - 2))
        span = [fires[i] for i in best[skip:skip + window_steps + 1]]
        if len(span) >= 2:
            toks = sum(f[2] for f in span[1:])
            out["window_steps_used"] = len(span) - 1
            out["window_tokens_per_s"] = toks / (span[-1][0] - span[0][0])
            out["window_ms_per_step"] = (span[-1][0] - span[0][0]) / (len(span) - 1) * 1e3
            out["window_requests_per_fire"] = statistics.mean(f[1] for f in span[1:])
    return out


def run_agentic_fork(engine, model_name: str, agents: int, prefix_len: int, branches: int, tokens: int, rounds: int,
                     vocab: int, timeout: float = 3600.0) -> dict:
    """`agents` agentic-fork inferlets at once (each: shared prefix, `branches`-way fork, `rounds`
    rounds of `tokens` tokens per branch). Returns whole-workload metrics."""
    rng = np.random.default_rng(7)
    args = [{"prefix_tokens": rng.integers(0, vocab, prefix_len).tolist(), "branches": branches, "tokens": tokens,
             "rounds": rounds, "seed": 1 + i, "top_k": 50, "temperature": 1.0} for i in range(agents)]
    entry = engine.model(model_name)
    t0 = time.perf_counter()
    procs = [engine.launch("agentic-fork", a) for a in args]
    results = [json.loads(engine.wait(p, timeout)) for p in procs]
    wall = time.perf_counter() - t0
    total = sum(r["tokens"] for r in results)
    st = engine.model_status()["models"][model_name]
    sched = entry.schedulers[0].stats
    return {"wall_s": wall, "output_tokens": total, "tokens_per_s": total / wall,
            "p50_prefill_s": statistics.median(r["prefill_s"] for r in results),
            "p50_round_s": statistics.median(r["round_ends_s"][-1] / len(r["round_ends_s"]) for r in results),
            "prefix_pages_per_agent": results[0]["prefix_pages"], "decode_steps": sched.get("decode_steps", 0),
            "kv_pages_used_after": st["kv_pages_used"]}
