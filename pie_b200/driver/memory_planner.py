"""Memory planner: after the weights are resident, split what is left of the device between KV
pages, the activation arena of the largest forward pass, and (optionally) recurrent-state slots,
and derive the forward limits the driver advertises. A profile trades batch capacity against
prefill chunk size:

    latency     small decode batch (64 requests), large prefill chunk
    balanced    256 requests, 8k-token passes
    throughput  1024 requests, 16k-token passes
    capacity    as many KV pages as possible, small passes
    auto        throughput when the KV pool can hold >= 512 average contexts, else balanced

Counterpart of driver/cuda/src/cuda_memory_planner.hpp:30-84 and its lattice sweep
(cuda_memory_planner.cpp).
"""
from __future__ import annotations

from dataclasses import dataclass

from ..models.config import ModelConfig

PROFILES = {
    "latency": dict(max_requests=64, max_tokens=8192),
    "balanced": dict(max_requests=256, max_tokens=8192),
    "throughput": dict(max_requests=1024, max_tokens=16384),
    "capacity": dict(max_requests=512, max_tokens=2048),
}


@dataclass
class MemoryPlan:
    profile: str
    kv_page_size: int
    kv_pages: int
    max_requests: int
    max_tokens: int
    state_slots: int
    arena_bytes: int
    kv_bytes: int

    def summary(self) -> str:
        return (f"profile={self.profile} pages={self.kv_pages}x{self.kv_page_size} tok "
                f"({self.kv_bytes / 2**30:.1f} GiB) requests<={self.max_requests} tokens/pass<={self.max_tokens} "
                f"arena={self.arena_bytes / 2**20:.0f} MiB")


def kv_bytes_per_page(cfg: ModelConfig, page_size: int, tp: int = 1, kv_dtype_bytes: int = 2) -> int:
    hkv = max(1, cfg.num_key_value_heads // tp)
    return cfg.num_hidden_layers * 2 * hkv * page_size * cfg.head_dim * kv_dtype_bytes


def arena_bytes(cfg: ModelConfig, max_tokens: int, max_requests: int, tp: int = 1) -> int:
    """Peak activation footprint of one pass: hidden, qkv, attention out, gate/up, logits rows."""
    h = cfg.hidden_size
    inter = (cfg.moe_intermediate_size * cfg.num_experts_per_tok if cfg.is_moe else cfg.intermediate_size) // tp
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim // tp
    per_token = 2 * (3 * h + qkv + cfg.num_attention_heads * cfg.head_dim // tp + 3 * inter)
    logits = max_requests * cfg.vocab_size * (2 + 4)       # bf16 logits + fp32 rows for probes
    return max_tokens * per_token + logits


def plan(cfg: ModelConfig, free_bytes: int, gpu_mem_utilization: float = 0.9, profile: str = "auto",
         page_size: int = 16, tp: int = 1, avg_context_tokens: int = 2048, rs_bytes_per_slot: int = 0) -> MemoryPlan:
    budget = int(free_bytes * gpu_mem_utilization)
    per_page = kv_bytes_per_page(cfg, page_size, tp)

    def build(name: str) -> MemoryPlan:
        lim = PROFILES[name]
        arena = arena_bytes(cfg, lim["max_tokens"], lim["max_requests"], tp)
        slots = lim["max_requests"] if rs_bytes_per_slot else 0
        left = budget - arena - slots * rs_bytes_per_slot
        pages = max(0, left // per_page)
        return MemoryPlan(name, page_size, int(pages), lim["max_requests"], lim["max_tokens"], slots, arena,
                          int(pages) * per_page)

    if profile != "auto":
        if profile not in PROFILES:
            raise ValueError(f"unknown memory profile {profile!r}")
        return build(profile)
    thr = build("throughput")
    if thr.kv_pages * page_size >= 512 * avg_context_tokens:
        return thr
    bal = build("balanced")
    return bal if bal.kv_pages > 0 else build("capacity")
