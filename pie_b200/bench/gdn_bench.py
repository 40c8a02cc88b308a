"""Gated DeltaNet mixer micro-benchmark (one linear-attention layer of a Qwen3.5-style hybrid: 16 key heads,
32 value heads, head size 128): decode rows and prefill chunks, CUDA events after warm-up, against the state and
activation bytes the kernels must move.

    python -m pie_b200.bench.gdn_bench [--decode 256] [--prefill 4x2048] [--iters 10]
"""
from __future__ import annotations

import argparse

import numpy as np
import torch

from .. import ops
from ..driver.recurrent import RecurrentStateCache
from ..models.config import ModelConfig


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--decode", type=int, default=256, help="decode rows (one token per request)")
    ap.add_argument("--prefill", default="4x2048", help="requests x tokens of the prefill case")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--heads", default="16,32,128,128", help="key heads, value heads, key head size, value head size")
    a = ap.parse_args(argv)
    hk, hv, dk, dv = (int(x) for x in a.heads.split(","))
    dev = "cuda"
    cfg = ModelConfig(model_type="qwen3_5", num_hidden_layers=1, layer_types=["linear_attention"], linear_num_key_heads=hk,
                      linear_num_value_heads=hv, linear_key_head_dim=dk, linear_value_head_dim=dv)
    c, f = cfg.gdn_conv_channels, cfg.gdn_in_features
    torch.manual_seed(0)
    lw = {"gdn_conv": (torch.randn(c, 4, device=dev) * 0.3).to(torch.bfloat16), "gdn_A_log": torch.randn(hv, device=dev) * 0.5,
          "gdn_dt_bias": torch.randn(hv, device=dev) * 0.5, "gdn_norm": torch.ones(dv, device=dev, dtype=torch.bfloat16)}
    pr, pt = (int(x) for x in a.prefill.split("x"))
    for name, lens in (("decode", [1] * a.decode), ("prefill", [pt] * pr)):
        r, n = len(lens), sum(lens)
        cache = RecurrentStateCache(cfg, r, dev)
        qo = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        rs = cache.inputs(qo, np.arange(r, dtype=np.int32), np.zeros(r, np.int32))
        mix = (torch.randn(n, f, device=dev) * 1.0).to(torch.bfloat16)
        run = lambda: ops.gdn_mixer(mix, lw, cfg, rs, 0)
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            run()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / a.iters * 1e3
        state = r * hv * dk * dv * 4 * 2                      # recurrent state read + written
        act = n * (f * 2 + c * 4 * 2 + hv * dv * 2)           # projection read, conv scratch written + read, output
        print(f"{name:8s} {r} requests x {lens[0]} tokens: {us:9.1f} us   state {state / 1e6:.1f} MB + activations "
              f"{act / 1e6:.1f} MB -> {(state + act) / us / 1e6:.2f} TB/s   {us / max(lens[0], 1):.2f} us per token step")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
