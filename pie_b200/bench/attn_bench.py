"""Prefill attention micro-benchmark: the tcgen05 kernel (one / two MMA tiles per CTA) against the
mma.sync kernel on causal prompts over a paged KV cache. CUDA events, warm-up, L2 flushed between
timed launches; FLOPs counted for the causal half only.

    python -m pie_b200.bench.attn_bench [--reqs 16 --len 2048] [--rows 64,128,256] [--iters 5]
"""
from __future__ import annotations

import argparse
import math

import numpy as np
import torch

from .. import ops


def run(reqs: int, plen: int, rows_list, iters: int, hq: int = 32, hkv: int = 8, d: int = 128, page: int = 16,
        warmup: int = 2):
    dev = "cuda:0"
    npg = plen // page
    g = torch.Generator(device=dev).manual_seed(1)
    kv = (torch.randn(reqs * npg + 1, 2, hkv, page, d, device=dev, generator=g) * 0.5).bfloat16()
    q = (torch.randn(reqs * plen, hq, d, device=dev, generator=g) * 0.5).bfloat16()
    pages = np.random.default_rng(0).permutation(reqs * npg).astype(np.int32)
    indptr = (np.arange(reqs + 1) * npg).astype(np.int32)
    qo = (np.arange(reqs + 1) * plen).astype(np.int32)
    batch = ops.AttnBatch(qo, indptr, pages, np.full(reqs, plen, np.int32), None, -1)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    flops = 4.0 * plen * plen / 2 * hq * d * reqs
    out = torch.empty_like(q)
    res = {}
    for rows in rows_list:
        plan = ops.build_prefill_plan(batch, hq // hkv, page, dev, tile_rows=rows)
        for _ in range(warmup):
            ops.paged_prefill_attention(q, kv, plan, 1 / math.sqrt(d), out=out)
        ts = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ops.paged_prefill_attention(q, kv, plan, 1 / math.sqrt(d), out=out)
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ops.check_kernel_status(dev)
        ms = sorted(ts)[len(ts) // 2]
        res[rows] = ms
        kind = "mma.sync" if rows == 64 else f"tcgen05 x{rows // 128}"
        print(f"{reqs} x {plen} ({kind:10s}): {ms:7.3f} ms  {flops / ms / 1e9:6.0f} TFLOP/s", flush=True)
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reqs", type=int, default=0)
    ap.add_argument("--len", type=int, default=0)
    ap.add_argument("--rows", default="64,128,256")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--head-dim", type=int, default=128, choices=[64, 128])
    ap.add_argument("--heads", default="32,8", help="query heads, KV heads")
    a = ap.parse_args()
    hq, hkv = (int(v) for v in a.heads.split(","))
    rows = [int(r) for r in a.rows.split(",")]
    shapes = [(a.reqs, a.len)] if a.reqs and a.len else [(64, 512), (16, 2048), (8, 4096), (2, 16384)]
    for reqs, plen in shapes:
        run(reqs, plen, rows, a.iters, hq=hq, hkv=hkv, d=a.head_dim, warmup=a.warmup)


if __name__ == "__main__":
    main()
