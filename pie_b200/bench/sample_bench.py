"""Sampler micro-benchmark on one GPU: the single-GPU sampler (`pie_sample`) over full rows and the
vocabulary-sharded sampler (`pie_tp_sample`) with all ranks of a group emulated as one cooperative launch
(blockIdx.y = rank; every rank's mailbox is local memory), both timed with CUDA events. Also the profiling
target of the two kernels:

    python -m pie_b200.bench.sample_bench --rows 512 --vocab 128256 --kind top_p --world 2
"""
from __future__ import annotations

import argparse
import ctypes as C

import torch

from .. import ops
from ..ops import _lib


def _params(rows, kind, dev):
    t = torch.ones(rows, device=dev)
    k = torch.zeros(rows, dtype=torch.int32, device=dev)
    p = torch.ones(rows, device=dev)
    mp = torch.zeros(rows, device=dev)
    if kind == "greedy":
        t.zero_()
    elif kind == "top_p":
        p.fill_(0.9)
    elif kind == "top_k":
        k.fill_(50)
    seeds = torch.randint(1, 2 ** 62, (rows,), dtype=torch.int64, device=dev)
    return t, k, p, mp, seeds


def _time(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=512)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--kind", default="top_p", choices=["greedy", "temperature", "top_p", "top_k"])
    ap.add_argument("--world", type=int, default=2, help="ranks emulated for the sharded sampler (0 = skip it)")
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args(argv)
    dev = "cuda:0"
    torch.manual_seed(0)
    logits = (torch.randn(a.rows, a.vocab, device=dev) * 0.3).to(torch.bfloat16)   # near-flat, like random-init weights
    t, k, p, mp, seeds = _params(a.rows, a.kind, dev)
    out = torch.empty(a.rows, dtype=torch.int32, device=dev)
    us = _time(lambda: ops.sample(logits, t, k, p, mp, seeds, out=out), a.iters)
    print(f"pie_sample       {a.rows} x {a.vocab} {a.kind}: {us:8.1f} us  ({a.rows * a.vocab * 2 / us / 1e6:.2f} TB/s of logits)")
    if a.world:
        w, vl = a.world, a.vocab // a.world
        lib = _lib.load(required=True)
        grid = 1024
        box = _lib.declare("pie_tp_sample_mailbox_bytes", [C.c_int, C.c_int], C.c_long)(grid, w)
        xbuf = [torch.zeros(box, dtype=torch.uint8, device=dev) for _ in range(w)]
        seq = [torch.zeros(grid, dtype=torch.int32, device=dev) for _ in range(w)]
        outs = [torch.full((a.rows,), -1, dtype=torch.int32, device=dev) for _ in range(w)]
        status = ops.kernel_status(dev)
        fn = lib.pie_tp_sample_emulated
        fn.restype = C.c_int
        fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_longlong,
                       C.c_void_p, C.c_long, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                       C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
        shards = [logits[:, r * vl:(r + 1) * vl].contiguous() for r in range(w)]
        arr = lambda ts: (C.c_void_p * w)(*[x.data_ptr() for x in ts])

        def go():
            rc = fn(arr(xbuf), arr(seq), status.data_ptr(), w, vl, grid, 0, arr(shards), vl, a.rows, t.data_ptr(),
                    k.data_ptr(), p.data_ptr(), mp.data_ptr(), seeds.data_ptr(), 0, 0, 0, arr(outs), ops.num_sms(dev),
                    torch.cuda.current_stream().cuda_stream)
            assert rc == 0, rc
        us2 = _time(go, a.iters)
        ops.check_kernel_status(dev)
        same = all(torch.equal(o, out) for o in outs)
        print(f"pie_tp_sample    {w} ranks x {vl} logits, emulated on one GPU (both ranks share its SMs): {us2:8.1f} us; "
              f"tokens equal to pie_sample: {same}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
