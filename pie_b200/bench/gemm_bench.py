"""GEMM micro-benchmark: the tcgen05 kernels (CTA pairs, single CTA) against cuBLAS (torch.matmul)
on the model's shapes. CUDA events, warm-up, L2 flushed between timed launches.

    python -m pie_b200.bench.gemm_bench [--shapes decode|prefill|all]
"""
from __future__ import annotations

import argparse

import torch

from .. import ops

ITERS = 0

DECODE = [(512, 6144, 4096), (512, 4096, 4096), (512, 28672, 4096), (512, 4096, 14336), (512, 128256, 4096),
          (512, 768, 4096), (512, 4096, 512), (512, 3584, 4096), (512, 4096, 1792), (64, 6144, 4096)]
# per-rank shards of the decode GEMMs (qkv, o, gate/up, down) under 2-, 4- and 8-way tensor parallelism
TP_SHARDS = [(512, 6144 // t, 4096) for t in (2, 4, 8)] + [(512, 4096, 4096 // t) for t in (2, 4, 8)] + \
            [(512, 28672 // t, 4096) for t in (2, 4, 8)] + [(512, 4096, 14336 // t) for t in (2, 4, 8)]
PREFILL = [(8192, 6144, 4096), (8192, 4096, 4096), (8192, 28672, 4096), (8192, 4096, 14336), (16384, 6144, 4096)]


def timeit(fn, flush, iters=10):
    iters = ITERS or iters
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="all")
    ap.add_argument("--m", type=int, default=0, help="override M of every shape (decode batch sweep)")
    ap.add_argument("--only", default="", help="N,K: run this weight shape only (profiling)")
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    shapes = {"decode": DECODE, "prefill": PREFILL, "tp": TP_SHARDS, "all": DECODE + PREFILL}[a.shapes]
    if a.m:
        shapes = sorted({(a.m, n, k) for _, n, k in shapes}, key=lambda t: (t[1], t[2]))
    if a.only:
        n0, k0 = (int(v) for v in a.only.split(","))
        shapes = [(m, n, k) for m, n, k in shapes if (n, k) == (n0, k0)][:1] or [(a.m or 512, n0, k0)]
    global ITERS
    ITERS = a.iters
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    import ctypes as C
    from ..ops import _lib
    thresholds = _lib.declare("pie_gemm_set_pair_thresholds", [C.c_double, C.c_double])
    print(f"{'M':>6} {'N':>7} {'K':>6} | {'cuBLAS us':>10} {'TF':>6} | {'default us':>9} {'TF':>6} | {'1-CTA us':>9} {'TF':>6} | "
          f"{'pairs us':>9} {'TF':>6} | max err")
    for m, n, k in shapes:
        x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        w = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
        fl = 2.0 * m * n * k
        t_cb = timeit(lambda: torch.matmul(x, w.t()), flush)
        ops.set_gemm_pairs(True)
        t_p = timeit(lambda: ops.gemm(x, w), flush)
        y = ops.gemm(x, w)
        ops.set_gemm_pairs(False)
        t_1 = timeit(lambda: ops.gemm(x, w), flush)
        ops.set_gemm_pairs(True)
        thresholds(0.0, 0.0)              # the CTA-pair kernel whatever the problem size
        t_f = timeit(lambda: ops.gemm(x, w), flush)
        thresholds(1.0e10, 2.0e10)
        err = (y.float() - torch.matmul(x, w.t()).float()).abs().max().item()
        print(f"{m:6d} {n:7d} {k:6d} | {t_cb*1e3:10.1f} {fl/t_cb/1e9:6.0f} | {t_p*1e3:9.1f} {fl/t_p/1e9:6.0f} | "
              f"{t_1*1e3:9.1f} {fl/t_1/1e9:6.0f} | {t_f*1e3:9.1f} {fl/t_f/1e9:6.0f} | {err:.3f}")
        ops.check_kernel_status()


if __name__ == "__main__":
    main()
