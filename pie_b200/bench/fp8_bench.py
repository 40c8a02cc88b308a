"""Block-scaled fp8 GEMM micro-benchmark on Qwen3-32B shapes: the fused fp8 x fp8 tcgen05 kernel
(activation quantisation included) against expanding the weight to bf16 followed by the bf16 GEMM
(the reference's scheme) and against a bf16 GEMM over weights that were expanded once.

    python -m pie_b200.bench.fp8_bench [--m 256] [--tp 8]
"""
from __future__ import annotations

import argparse

import torch

from .. import ops
from . import gemm_bench
from .gemm_bench import timeit


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=256)
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    gemm_bench.ITERS = a.iters
    t = a.tp
    shapes = [("qkv", 10240 // t, 5120), ("o", 5120, 8192 // t), ("gate_up", 51200 // t, 5120), ("down", 5120, 25600 // t)]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    print(f"M={a.m} TP={t} | {'shape':>22} | fused fp8 us | quant us | dequant+bf16 us | bf16 (pre-expanded) us | rel err")
    for name, n, k in shapes:
        w = torch.randn(n, k, device="cuda") * 0.05
        x = (torch.randn(a.m, k, device="cuda") * 0.5).to(torch.bfloat16)
        q = ops.quantize_fp8_block(w)
        wb = q.dequant()
        t_f = timeit(lambda: ops.gemm_fp8w(x, q, mode="fused"), flush)
        t_q = timeit(lambda: ops.quant_act_fp8(x), flush)
        t_d = timeit(lambda: ops.gemm_fp8w(x, q, mode="dequant"), flush)
        t_b = timeit(lambda: ops.gemm(x, wb), flush)
        y = ops.gemm_fp8w(x, q, mode="fused").float()
        exact = x.float() @ w.t()
        rel = ((y - exact).norm() / exact.norm()).item()
        print(f"{'':10} | {name:>8} {n:6d}x{k:<6d} | {t_f * 1e3:12.1f} | {t_q * 1e3:8.1f} | {t_d * 1e3:15.1f} | {t_b * 1e3:22.1f} | {rel:.4f}")
        ops.check_kernel_status()


if __name__ == "__main__":
    main()
