"""MoE block micro-benchmark: the routed expert MLP (router top-k, alignment, permute, two
grouped tcgen05 GEMMs with fused SwiGLU, weighted combine) against a per-expert loop of library
GEMMs, on Qwen3-30B-A3B shapes. CUDA events, warm-up, L2 flushed between timed runs.

    python -m pie_b200.bench.moe_bench [--tokens 1024] [--experts 128] [--topk 8] [--iters 10]
"""
from __future__ import annotations

import argparse

import torch

from .. import ops
from .gemm_bench import timeit
from . import gemm_bench


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=1024)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--inter", type=int, default=768)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    gemm_bench.ITERS = a.iters
    dev = torch.device("cuda")
    n, h, inter, e, k = a.tokens, a.hidden, a.inter, a.experts, a.topk
    x = (torch.randn(n, h, device=dev) * 0.5).to(torch.bfloat16)
    res = torch.zeros(n, h, device=dev, dtype=torch.bfloat16)
    logits = torch.randn(n, e, device=dev)
    wgu = (torch.randn(e, 2 * inter, h, device=dev) * 0.03).to(torch.bfloat16)
    wd = (torch.randn(e, h, inter, device=dev) * 0.03).to(torch.bfloat16)
    buf = ops.MoeBuffers(n, h, inter, e, k, dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def grouped():
        return ops.moe_experts(x, logits, wgu, wd, k, True, buf, residual=res)

    def looped():
        w, ids = torch.topk(torch.softmax(logits, -1), k, -1)
        w = w / w.sum(-1, keepdim=True)
        flat = ids.reshape(-1)
        order = torch.argsort(flat, stable=True)
        tok = order // k
        counts = torch.bincount(flat, minlength=e).tolist()
        xs = x[tok]
        ys = torch.empty_like(xs)
        s = 0
        for ei, c in enumerate(counts):
            if c:
                gu = xs[s:s + c] @ wgu[ei].t()
                ys[s:s + c] = (torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]) @ wd[ei].t()
            s += c
        out = torch.zeros(n, h, dtype=torch.float32, device=dev)
        out.index_add_(0, tok, ys.float() * w.reshape(-1)[order][:, None])
        return out.to(torch.bfloat16)

    t_g = timeit(grouped, flush)
    t_l = timeit(looped, flush)
    err = (grouped().float() - looped().float()).abs().max().item()
    wbytes = (wgu.numel() + wd.numel()) * 2
    flops = 2.0 * n * k * 3 * h * inter
    print(f"tokens {n} experts {e} top-{k}: grouped {t_g * 1e3:.1f} us ({wbytes / t_g / 1e6:.0f} GB/s of weights, "
          f"{flops / t_g / 1e9:.0f} TFLOP/s) | per-expert library loop {t_l * 1e3:.1f} us | max diff {err:.3f}")
    ops.check_kernel_status()


if __name__ == "__main__":
    main()
