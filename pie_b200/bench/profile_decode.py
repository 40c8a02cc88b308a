"""Small decode workload for profilers: R contexts of a given KV length (page tables assigned,
KV content zero) and a few eager decode steps of the named architecture, so that each kernel
is an individual launch. Prints device time per step.

    python -m pie_b200.bench.profile_decode --requests 512 --kv-len 600 --layers 2 --steps 3
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
    a = ap.parse_args()
    cfg = preset(a.model, num_hidden_layers=a.layers)
    ps = 16
    per = -(-(a.kv_len + a.steps + a.prefill + 2) // ps)
    drv = TorchDriver(cfg, "cuda:0", num_pages=per * a.requests + 8, page_size=ps, max_requests=a.requests,
                      max_tokens=max(8192, a.requests * max(1, a.prefill)), gemm_backend=a.gemm, use_graphs=a.graphs)
    pages = [list(range(i * per, (i + 1) * per)) for i in range(a.requests)]
    sp = SamplerSpec(SamplerKind.TOP_P, temperature=1.0, top_p=0.9)
    rng = np.random.default_rng(0)
    kv = a.kv_len
    if a.prefill:
        items = [PendingRequest(i, rng.integers(0, cfg.vocab_size, a.prefill).tolist(),
                                list(range(kv, kv + a.prefill)), pages[i], kv, [(a.prefill - 1, sp)])
                 for i in range(a.requests)]
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        drv.fire_batch(fold(items, ps))
        ev1.record()
        torch.cuda.synchronize()
        print(f"prefill {a.requests}x{a.prefill} tokens: {ev0.elapsed_time(ev1):.3f} ms")
        kv += a.prefill
    toks = rng.integers(0, cfg.vocab_size, a.requests).tolist()
    for s in range(a.steps):
        items = [PendingRequest(i, [toks[i]], [kv + s], pages[i], kv + s, [(0, sp)]) for i in range(a.requests)]
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        resp = drv.fire_batch(fold(items, ps))
        ev1.record()
        torch.cuda.synchronize()
        toks = [sl.token for sl in resp.slots]
        print(f"decode step {s}: {ev0.elapsed_time(ev1):.3f} ms")
    from .. import ops
    ops.check_kernel_status(drv.device)


if __name__ == "__main__":
    main()
