"""page-trim-bench: decode with a sliding-window attention mask over a long context and report
how many pages the runtime dropped from the requests (pages masked out in every row do not travel
to the driver). Counterpart of inferlets/page-trim-bench/src/lib.rs."""
import json
import time

from pie_b200.sdk import Sampler

from ._common import load_model, prompt_context

NAME = "page-trim-bench"


async def main(args):
    args = args or {}
    model = load_model(args)
    window, steps = int(args.get("window", 32)), int(args.get("steps", 8))
    ctx = prompt_context(model, args)
    pending, ctx._buffer = ctx.buffer, []
    sched = ctx._entry.schedulers[0]
    before = sched.stats.get("trimmed_pages", 0)
    t0 = time.perf_counter()
    for _ in range(steps):
        start = ctx.seq_len
        fwd = ctx.forward().input(pending)
        rows = []
        for i in range(len(pending)):
            kv = start + i + 1
            rows.append([0, kv] if kv <= window else [kv - window, window])
        fwd.attention_mask(rows)
        h = fwd.sample([len(pending) - 1], Sampler.argmax())
        pending = [(await fwd.execute()).token(h)]
    dt = time.perf_counter() - t0
    pages = ctx.committed_page_count() + ctx.working_page_count()
    ctx.release()
    return json.dumps({"steps": steps, "context_pages": pages, "pages_trimmed": sched.stats.get("trimmed_pages", 0) - before,
                       "ms_per_step": dt / steps * 1e3})
