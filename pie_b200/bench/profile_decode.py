"""Small decode workload for profilers: R contexts of a given KV length (page tables assigned,
KV content zero) and a few eager decode steps of the named architecture, so that each kernel
is an individual launch. Prints device time per step.

    python -m pie_b200.bench.profile_decode --requests 512 --kv-len 600 --layers 2 --steps 3

Under `python -m torch.distributed.run --nproc-per-node T ... -m pie_b200.bench.profile_decode` the model
runs as one fused tensor-parallel group (rank 0 drives, the others follow its fires). `--timeline`
adds a per-kernel table (count, total and mean device time per step, from CUPTI activity records
of graph-replayed steps): shares of a step, not benchmark numbers.
"""
from __future__ import annotations

import argparse

import numpy as np
import torch

from ..driver.executor import TorchDriver
from ..driver.schema import SamplerKind, SamplerSpec
from ..models.config import preset
from ..runtime.scheduler import PendingRequest, fold


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3.1-8b")
    ap.add_argument("--requests", type=int, default=512)
    ap.add_argument("--kv-len", type=int, default=600)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--gemm", default="tcgen05")
    ap.add_argument("--graphs", action="store_true")
    ap.add_argument("--prefill", type=int, default=0, help="also run one prefill batch of this many tokens per request")
    ap.add_argument("--prefill-timeline", action="store_true",
                    help="per-kernel device time of the prefill batch (one warm-up prefill first; one GPU)")
    ap.add_argument("--timeline", action="store_true", help="per-kernel device time of the decode steps (implies --graphs)")
    ap.add_argument("--tp-backend", default="fused", choices=["fused", "nccl"])
    a = ap.parse_args()
    import os
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    par, comm = None, None
    if world > 1:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed as dist
        from ..models.transformer import ParallelContext
        from ..parallel.comm import TPComm
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        comm = TPComm(rank, world, torch.device("cuda", local), fused=a.tp_backend == "fused")
        par = ParallelContext(world, rank, comm)
    if a.timeline:
        a.graphs = True
    cfg = preset(a.model, num_hidden_layers=a.layers)
    ps = 16
    per = -(-(a.kv_len + a.steps + a.prefill + 2) // ps)
    drv = TorchDriver(cfg, f"cuda:{local}", num_pages=per * a.requests + 8, page_size=ps, max_requests=a.requests,
                      max_tokens=max(8192, a.requests * max(1, a.prefill)), gemm_backend=a.gemm, use_graphs=a.graphs,
                      par=par)
    prof = None
    if a.timeline:
        from torch.profiler import ProfilerActivity, profile
        prof = profile(activities=[ProfilerActivity.CUDA])
    if comm is not None:
        comm.attach(drv)
        if rank != 0:
            if prof is not None:
                # every rank traces (same overhead everywhere). Starting the tracer takes seconds, far
                # longer than a kernel waits for a peer, so it happens at rank 0's first mark, between
                # two barriers, and never while a fused kernel is in flight.
                orig, state = comm._mark_local, {"n": 0}

                def mark_local(end):
                    out = orig(end)
                    state["n"] += 1
                    if state["n"] == 1:
                        prof.start()
                    return out
                comm._mark_local = mark_local
            comm.follower_loop(drv)
            comm.close()
            os._exit(0)
    pages = [list(range(i * per, (i + 1) * per)) for i in range(a.requests)]
    sp = SamplerSpec(SamplerKind.TOP_P, temperature=1.0, top_p=0.9)
    rng = np.random.default_rng(0)
    kv = a.kv_len
    if a.prefill:
        items = [PendingRequest(i, rng.integers(0, cfg.vocab_size, a.prefill).tolist(),
                                list(range(kv, kv + a.prefill)), pages[i], kv, [(a.prefill - 1, sp)])
                 for i in range(a.requests)]
        pprof = None
        if a.prefill_timeline:
            from torch.profiler import ProfilerActivity, profile
            drv.fire_batch(fold(items, ps))                      # warm-up: same pages are written again below
            torch.cuda.synchronize()
            pprof = profile(activities=[ProfilerActivity.CUDA])
            pprof.start()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        drv.fire_batch(fold(items, ps))
        ev1.record()
        torch.cuda.synchronize()
        print(f"prefill {a.requests}x{a.prefill} tokens: {ev0.elapsed_time(ev1):.3f} ms")
        if pprof is not None:
            pprof.stop()
            rows = {}
            for e in pprof.events():
                if e.device_type is not None and "cuda" in str(e.device_type).lower():
                    c, t = rows.get(e.name, (0, 0.0))
                    rows[e.name] = (c + 1, t + e.device_time)
            total = sum(t for _, t in rows.values())
            print(f"prefill kernel timeline ({total / 1e3:.3f} ms of kernels)")
            for name, (c, t) in sorted(rows.items(), key=lambda kv: -kv[1][1])[:24]:
                print(f"{t:10.1f} us  {c:5d} launches  {t / c:9.2f} us each  {name[:110]}")
        kv += a.prefill
    toks = rng.integers(0, cfg.vocab_size, a.requests).tolist()
    warm = 2 if a.timeline else 0
    for s in range(a.steps + warm):
        if prof is not None and s == warm:
            torch.cuda.synchronize()
            if comm is not None:
                comm.mark(False)
            prof.start()
            if comm is not None:
                comm.mark(False)
        items = [PendingRequest(i, [toks[i]], [kv + s], pages[i], kv + s, [(0, sp)]) for i in range(a.requests)]
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        resp = drv.fire_batch(fold(items, ps))
        ev1.record()
        torch.cuda.synchronize()
        toks = [sl.token for sl in resp.slots]
        print(f"decode step {s}: {ev0.elapsed_time(ev1):.3f} ms")
    if prof is not None:
        torch.cuda.synchronize()
        prof.stop()
        rows = {}
        for e in prof.events():
            if e.device_type is not None and "cuda" in str(e.device_type).lower():
                c, t = rows.get(e.name, (0, 0.0))
                rows[e.name] = (c + 1, t + e.device_time)
        total = sum(t for _, t in rows.values())
        print(f"kernel timeline over {a.steps} graph-replayed steps ({total / a.steps / 1e3:.3f} ms of kernels per step)")
        for name, (c, t) in sorted(rows.items(), key=lambda kv: -kv[1][1]):
            print(f"{t / a.steps:10.1f} us/step  {c / a.steps:7.1f} launches/step  {t / c:8.2f} us each  {name[:110]}")
    from .. import ops
    st = ops.kernel_status(drv.device).cpu().numpy()
    w = st[2:6].view("uint64")
    if st[6] or st[7]:
        print(f"peer waits seen by CTA 0: all-gather flags {w[0] / max(1, st[6]) / 1e3:.1f} us x {st[6]} waits, "
              f"reduce-scatter flags {w[1] / max(1, st[7]) / 1e3:.1f} us x {st[7]} waits (whole run)")
    ops.check_kernel_status(drv.device)
    if comm is not None:
        comm.stop_followers()
        comm.close()
        os._exit(0)


if __name__ == "__main__":
    main()
