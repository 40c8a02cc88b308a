"""LoRA adapters held by a driver: per layer low-rank pairs for the fused QKV projection and
the attention output projection, y += (x A^T) B^T * (alpha / rank). New adapters start with
B = 0 (identity). Zeroth-order updates (`zo_apply`) add seeded Gaussian directions to every
matrix: params += coeff * N(seed), the primitive under the SDK's ZO API.

The reference routes these operations to its drivers as AdapterRequest{op, adapter_id, path}
(driver/bridge/src/schema.rs:293-353, runtime/src/adapter.rs:1-90); its native CUDA driver
accepts and ignores them (driver/cuda/src/service/inproc_service.cpp:31-191).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch


class LoraAdapter:
    def __init__(self, cfg, rank: int, alpha: float, device, dtype, hq_local: int, hkv_local: int, seed: int = 0):
        self.rank, self.alpha = rank, float(alpha)
        self.scale = self.alpha / max(1, rank)
        h, d = cfg.hidden_size, cfg.head_dim
        nqkv, no = (hq_local + 2 * hkv_local) * d, hq_local * d
        g = torch.Generator(device="cpu").manual_seed(seed or 1)

        def a_init(cols):
            return (torch.randn(rank, cols, generator=g) / cols ** 0.5).to(dtype).to(device)

        self.layers: List[Dict[str, torch.Tensor]] = []
        for _ in range(cfg.num_hidden_layers):
            self.layers.append({"qkv_a": a_init(h), "qkv_b": torch.zeros(nqkv, rank, dtype=dtype, device=device),
                                "o_a": a_init(no), "o_b": torch.zeros(h, rank, dtype=dtype, device=device)})

    def tensors(self) -> Dict[str, torch.Tensor]:
        return {f"layers.{i}.{k}": v for i, lw in enumerate(self.layers) for k, v in lw.items()}

    def load_tensors(self, named: Dict[str, torch.Tensor]) -> None:
        for name, t in named.items():
            _, i, k = name.split(".")
            dst = self.layers[int(i)][k]
            if tuple(dst.shape) != tuple(t.shape):
                raise ValueError(f"adapter tensor {name}: shape {tuple(t.shape)} != {tuple(dst.shape)}")
            dst.copy_(t.to(dst.dtype))

    def copy_from(self, other: "LoraAdapter") -> None:
        for mine, theirs in zip(self.layers, other.layers):
            for k in mine:
                mine[k].copy_(theirs[k])

    def zo_apply(self, seed: int, coeff: float) -> None:
        g = torch.Generator(device="cpu").manual_seed(int(seed) & 0x7FFFFFFFFFFFFFFF)
        for lw in self.layers:
            for k in ("qkv_a", "qkv_b", "o_a", "o_b"):
                noise = torch.randn(lw[k].shape, generator=g)
                lw[k].add_(noise.to(lw[k].dtype).to(lw[k].device), alpha=coeff)

    def delta(self, layer: int, which: str, x: torch.Tensor) -> torch.Tensor:
        lw = self.layers[layer]
        return (x @ lw[which + "_a"].t()) @ lw[which + "_b"].t() * self.scale


def apply_lora(lora: Optional[list], layer: int, which: str, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """y[rows] += adapter.delta(x[rows]) for every (adapter, rows) binding of the batch."""
    if not lora:
        return y
    for adapter, rows in lora:
        y.index_add_(0, rows, adapter.delta(layer, which, x.index_select(0, rows)).to(y.dtype))
    return y
