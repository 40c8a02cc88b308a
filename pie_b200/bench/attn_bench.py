"""Prefill attention micro-benchmark: the tcgen05 kernel (one / two MMA tiles per CTA) against the
mma.sync kernel on causal prompts over a paged KV cache. CUDA events, warm-up, L2 flushed between
timed launches; FLOPs counted for the causal half only.

    python -m pie_b200.bench.attn_bench [--reqs 16 --len 2048] [--rows 64,128,256] [--iters 5]
    python -m pie_b200.bench.attn_bench --decode [--reqs 512 --len 1200] [--heads 32,8] [--head-dim 256] [--softcap 50]

`--decode`: split-KV decode attention over bf16 pages and over fp8 pages (bytes of KV actually streamed
per launch over the CUDA-event time, against the measured copy bandwidth), and with `--fork B` over
groups of B requests that share all but their last page (the shared-prefix plan against the plain one).
"""
from __future__ import annotations

import argparse
import math

import numpy as np
import torch

from .. import ops


def run(reqs: int, plen: int, rows_list, iters: int, hq: int = 32, hkv: int = 8, d: int = 128, page: int = 16,
        warmup: int = 2, softcap: float = 0.0):
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
    if d == 256:                        # only the 64-row kernel covers it
        rows_list = [64]
    elif softcap:                       # the tcgen05 kernel takes a soft cap in its two-tile form
        rows_list = [r for r in rows_list if r in (64, 256)]
    for rows in rows_list:
        plan = ops.build_prefill_plan(batch, hq // hkv, page, dev, tile_rows=rows)
        for _ in range(warmup):
            ops.paged_prefill_attention(q, kv, plan, 1 / math.sqrt(d), out=out, softcap=softcap)
        ts = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ops.paged_prefill_attention(q, kv, plan, 1 / math.sqrt(d), out=out, softcap=softcap)
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ops.check_kernel_status(dev)
        ms = sorted(ts)[len(ts) // 2]
        res[rows] = ms
        kind = "mma.sync" if rows == 64 else f"tcgen05 x{rows // 128}"
        print(f"{reqs} x {plen} hq {hq} hkv {hkv} d {d}{' softcap' if softcap else ''} ({kind:10s}): {ms:7.3f} ms  "
              f"{flops / ms / 1e9:6.0f} TFLOP/s", flush=True)
    return res


def run_decode(reqs: int, kv_len: int, iters: int, hq: int, hkv: int, d: int, fork: int = 0, page: int = 16,
               warmup: int = 3, softcap: float = 0.0):
    dev = "cuda:0"
    npg = -(-kv_len // page)
    rng = np.random.default_rng(0)
    if fork > 1:                    # groups of `fork` requests: npg - 1 shared pages + one private page each
        groups = reqs // fork
        total = groups * (npg - 1) + reqs
        perm = rng.permutation(total).astype(np.int32)
        tables = [list(perm[g * (npg - 1):(g + 1) * (npg - 1)]) + [perm[groups * (npg - 1) + g * fork + b]]
                  for g in range(groups) for b in range(fork)]
        reqs = groups * fork
    else:
        total = reqs * npg
        perm = rng.permutation(total).astype(np.int32)
        tables = [list(perm[i * npg:(i + 1) * npg]) for i in range(reqs)]
    pages = np.concatenate(tables).astype(np.int32)
    indptr = (np.arange(reqs + 1) * npg).astype(np.int32)
    kv_lens = np.full(reqs, kv_len, np.int32)
    g = torch.Generator(device=dev).manual_seed(1)
    kv = (torch.randn(total + 1, 2, hkv, page, d, device=dev, generator=g) * 0.5).bfloat16()
    amax = kv.float().abs().amax(-1).clamp_min(1e-12)
    sc = (amax / 448.0).contiguous()
    kv8 = (kv.float() / sc[..., None]).to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
    q = (torch.randn(reqs, hq, d, device=dev, generator=g) * 0.5).bfloat16()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
    ctas = ops.num_sms(dev) * 2
    max_items = reqs + ctas * 8
    scratch = torch.empty(ops.decode_scratch_floats(max_items, hq, d), device=dev)
    item_req, st, en, iptr = ops.plan_decode_items(kv_lens, hkv, ctas, max_items)
    plain = ops.DecodePlan(t(pages), t(indptr), t(item_req), t(st), t(en), t(iptr),
                           torch.tensor([len(item_req)], dtype=torch.int32, device=dev), scratch, max_items, reqs, ctas, page)
    variants = [("bf16 pages", plain, kv, None, 2.0), ("fp8 pages", plain, kv8, sc, 1.0 + 4.0 / d)]
    if softcap or d == 256:             # the fp8-page kernel covers neither
        variants = [("bf16 pages" + (f", softcap {softcap:g}" if softcap else ""), plain, kv, None, 2.0)]
    if fork > 1 and not softcap:
        grp = ops.find_shared_prefixes(kv_lens, indptr, pages, page)
        cp = ops.plan_decode_cascade(kv_lens, grp, hkv, hq // hkv, ctas, max_items)
        if cp is not None:
            casc = ops.DecodePlan(t(pages), t(indptr), t(cp.item_req), t(cp.item_start), t(cp.item_end), t(cp.req_slot_indptr),
                                  torch.tensor([len(cp.item_req)], dtype=torch.int32, device=dev), scratch, max_items, reqs,
                                  ctas, page, item_slot=t(cp.item_slot), item_tile=t(cp.item_tile),
                                  tile_members=t(cp.tile_members))
            variants.append(("bf16 pages, shared-prefix plan", casc, kv, None, 2.0))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out = torch.empty_like(q)
    ref_out = None
    for name, plan, cache, scale, bytes_per_elem in variants:
        for _ in range(warmup):
            ops.paged_decode_attention(q, cache, plan, 1 / math.sqrt(d), out=out, kv_scale=scale, softcap=softcap)
        ts = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ops.paged_decode_attention(q, cache, plan, 1 / math.sqrt(d), out=out, kv_scale=scale, softcap=softcap)
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ops.check_kernel_status(dev)
        ms = sorted(ts)[len(ts) // 2]
        if ref_out is None:
            ref_out = out.float().clone()
        err = float((out.float() - ref_out).abs().max())
        logical = 2.0 * reqs * kv_len * hkv * d * bytes_per_elem          # K and V of every request, as a plain plan reads them
        print(f"decode {reqs} x {kv_len} hq {hq} hkv {hkv} d {d} ({name}): {ms * 1e3:8.1f} us  {logical / ms / 1e6:7.0f} GB/s of "
              f"per-request KV  (max |diff| vs bf16 plain {err:.3f})", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--decode", action="store_true")
    ap.add_argument("--fork", type=int, default=0)
    ap.add_argument("--reqs", type=int, default=0)
    ap.add_argument("--len", type=int, default=0)
    ap.add_argument("--rows", default="64,128,256")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--head-dim", type=int, default=128, choices=[64, 128, 256])
    ap.add_argument("--softcap", type=float, default=0.0, help="soft cap on the scores (Gemma-2: 50)")
    ap.add_argument("--heads", default="32,8", help="query heads, KV heads")
    a = ap.parse_args()
    hq, hkv = (int(v) for v in a.heads.split(","))
    if a.decode:
        run_decode(a.reqs or 512, a.len or 1200, a.iters, hq, hkv, a.head_dim, fork=a.fork, softcap=a.softcap)
        return
    rows = [int(r) for r in a.rows.split(",")]
    shapes = [(a.reqs, a.len)] if a.reqs and a.len else [(64, 512), (16, 2048), (8, 4096), (2, 16384)]
    for reqs, plen in shapes:
        run(reqs, plen, rows, a.iters, hq=hq, hkv=hkv, d=a.head_dim, warmup=a.warmup, softcap=a.softcap)


if __name__ == "__main__":
    main()
