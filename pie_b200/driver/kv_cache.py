"""Paged KV cache and its host swap pool.

Device layout: one tensor ``[layers, pages, 2, kv_heads_local, page_size, head_dim]`` so that a
(page, head) K or V block is a contiguous run (bulk copies, tensor-core tiles) and a page of
every layer can be copied with one kernel launch. Page id ``num_pages`` (one extra page at
the end) is a scratch page that padded graph-bucket requests point at.

Reference counterparts: driver/cuda/src/kv_cache.hpp:1-202 (per-layer K/V page pools),
driver/cuda/src/swap_pool.hpp:25-84 (pinned host mirror, D2H/H2D/D2D/H2H page copies).
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops
from .schema import CopyDir, CopyRequest


class KVCache:
    def __init__(self, layers: int, num_pages: int, kv_heads: int, page_size: int, head_dim: int,
                 dtype, device, swap_pages: int = 0, kv_dtype: str = "auto"):
        """kv_dtype "auto": pages in the activation dtype. "fp8_e4m3": one byte per element plus one
        fp32 scale per (token, KV head) row in `scale` [layers, pages + 1, 2, kv_heads, page_size]
        (written by the RoPE + KV-write kernel, read by decode attention; prefill attention works on
        pages expanded to bf16 for the batch). Counterpart of the reference's per-token-head fp8 format
        (driver/cuda/src/kv_cache_format.hpp, kernels/kv_paged.cu:188-325)."""
        if page_size % 16:
            raise ValueError("kv page size must be a multiple of 16")
        if kv_dtype not in ("auto", "bf16", "fp8_e4m3"):
            raise ValueError(f"unknown kv_dtype {kv_dtype!r} (auto | bf16 | fp8_e4m3)")
        self.kv_dtype = kv_dtype
        self.scale = None
        if kv_dtype == "fp8_e4m3":
            if torch.device(device).type != "cuda":
                raise NotImplementedError("fp8 KV pages need the CUDA kernels")
            dtype = torch.uint8
            self.scale = torch.zeros(layers, num_pages + 1, 2, kv_heads, page_size, dtype=torch.float32, device=device)
        self.layers, self.num_pages, self.kv_heads = layers, num_pages, kv_heads
        self.page_size, self.head_dim, self.dtype = page_size, head_dim, dtype
        self.device = torch.device(device)
        # zero-filled: unwritten slots are multiplied by p == 0 in attention and must be finite
        self.data = torch.zeros(layers, num_pages + 1, 2, kv_heads, page_size, head_dim, dtype=dtype,
                                device=self.device)
        self.pad_page = num_pages
        self.swap_pages = swap_pages
        self.host = None
        if swap_pages > 0:
            self.host = torch.zeros(layers, swap_pages, 2, kv_heads, page_size, head_dim, dtype=dtype,
                                    pin_memory=self.device.type == "cuda")
        self._copy_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None

    @property
    def page_bytes_all_layers(self) -> int:
        return self.layers * 2 * self.kv_heads * self.page_size * self.head_dim * self.data.element_size()

    @staticmethod
    def bytes_per_page(layers, kv_heads, page_size, head_dim, elem_size=2) -> int:
        return layers * 2 * kv_heads * page_size * head_dim * elem_size

    def copy(self, req: CopyRequest) -> None:
        """Execute a page copy on every layer. D2D runs on the compute stream (it orders with
        forward passes that read the pages); swaps run on a side stream and are awaited."""
        src = np.ascontiguousarray(req.srcs, dtype=np.int32)
        dst = np.ascontiguousarray(req.dsts, dtype=np.int32)
        if len(src) == 0:
            return
        if req.direction == CopyDir.D2D:
            s = torch.from_numpy(src).to(self.device)
            d = torch.from_numpy(dst).to(self.device)
            ops.copy_pages(self.data, s, d)
            if self.scale is not None:
                ops.copy_pages(self.scale, s, d)
            return
        if self.scale is not None:
            raise NotImplementedError("host swap of fp8 KV pages")
        if self.host is None:
            raise RuntimeError("no swap pool configured")
        if req.direction == CopyDir.H2H:
            self.host[:, torch.from_numpy(dst).long()] = self.host[:, torch.from_numpy(src).long()]
            return
        if self._copy_stream is None:
            for s, d in zip(src.tolist(), dst.tolist()):
                if req.direction == CopyDir.D2H:
                    self.host[:, d] = self.data[:, s]
                else:
                    self.data[:, d] = self.host[:, s]
            return
        cur = torch.cuda.current_stream(self.device)
        self._copy_stream.wait_stream(cur)
        with torch.cuda.stream(self._copy_stream):
            for s, d in zip(src.tolist(), dst.tolist()):
                if req.direction == CopyDir.D2H:
                    self.host[:, d].copy_(self.data[:, s], non_blocking=True)
                else:
                    self.data[:, d].copy_(self.host[:, s], non_blocking=True)
        if req.direction == CopyDir.H2D:
            cur.wait_stream(self._copy_stream)
        else:
            self._copy_stream.synchronize()
