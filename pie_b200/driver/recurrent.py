"""Recurrent-state cache of the Gated DeltaNet and Mamba-2 layers: per (recurrent layer, slot) the tail of the
short convolution's inputs and the fp32 state (delta-rule state [heads, dk, dv], or state-space state
[heads, head_dim, state]). A slot belongs to one resident context; the runtime's
slot pool (`runtime/rs_cache.py`) hands slots out, tells the driver when a slot must start from zero
(`rs_reset`) and asks for a slot copy when a context forks.

Counterpart of driver/cuda/src/recurrent_state_cache.hpp:1-40 (slabs per layer and slot, slot D2D copy).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from ..models.config import ModelConfig


@dataclass
class RecurrentInputs:
    """What the mixer of every linear layer needs for one fire."""
    qo_indptr: torch.Tensor        # int32 [R + 1] on the device
    tok_req: torch.Tensor          # int32 [N] request of every token row
    slots: torch.Tensor            # int32 [R]
    reset: torch.Tensor            # int32 [R] 1 = start this request's state from zero
    qo_host: List[int]
    slots_host: List[int]
    reset_host: List[int]
    conv_state: torch.Tensor       # [L, S, C, K - 1] fp32
    rec_state: torch.Tensor        # [L, S, Hv, dk, dv] fp32
    layer_index: Dict[int, int]    # model layer -> index into the first dimension of the caches
    scratch: Optional[torch.Tensor] = None   # [N, C] fp32 convolution output (device path)


class RecurrentStateCache:
    def __init__(self, cfg: ModelConfig, num_slots: int, device):
        self.cfg, self.num_slots, self.device = cfg, num_slots, torch.device(device)
        lin = cfg.recurrent_layers
        if cfg.linear_layers and cfg.mamba_layers:
            raise NotImplementedError("Gated DeltaNet and Mamba-2 layers in one model")
        self.layer_index = {li: i for i, li in enumerate(lin)}
        if cfg.mamba_layers:       # [heads, head_dim, state] per slot, convolution over x | B | C
            c, k = cfg.mamba_conv_channels, 4
            hv, dk, dv = cfg.mamba_num_heads, cfg.mamba_head_dim, cfg.ssm_state_size
        else:
            c, k = cfg.gdn_conv_channels, cfg.linear_conv_kernel_dim
            hv, dk, dv = cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.conv_channels = c
        self.conv_state = torch.zeros(len(lin), num_slots, c, k - 1, dtype=torch.float32, device=self.device)
        self.rec_state = torch.zeros(len(lin), num_slots, hv, dk, dv, dtype=torch.float32, device=self.device)

    @property
    def bytes_per_slot(self) -> int:
        return (self.conv_state[:, 0].numel() + self.rec_state[:, 0].numel()) * 4

    def inputs(self, qo_indptr, rs_slots, rs_reset) -> RecurrentInputs:
        qo = np.ascontiguousarray(qo_indptr, dtype=np.int32)
        r = len(qo) - 1
        if rs_slots is None or len(rs_slots) != r:
            raise ValueError("this model has recurrent layers: every request needs a recurrent-state slot")
        slots = np.ascontiguousarray(rs_slots, dtype=np.int32)
        if len(slots) and (slots.min() < 0 or slots.max() >= self.num_slots):
            raise ValueError(f"recurrent-state slot outside 0..{self.num_slots - 1}")
        if len(set(slots.tolist())) != len(slots):
            raise ValueError("two requests of one fire share a recurrent-state slot")
        reset = np.ascontiguousarray(rs_reset if rs_reset is not None else np.zeros(r, np.int32), dtype=np.int32)
        tok_req = np.repeat(np.arange(r, dtype=np.int32), np.diff(qo))
        dev = self.device
        t = lambda a: torch.from_numpy(a).to(dev)
        n = int(qo[-1])
        scratch = (torch.empty(max(n, 1), self.conv_channels, dtype=torch.float32, device=dev)
                   if dev.type == "cuda" else None)
        return RecurrentInputs(t(qo), t(tok_req), t(slots), t(reset), qo.tolist(), slots.tolist(), reset.tolist(),
                               self.conv_state, self.rec_state, self.layer_index, scratch)

    def copy_slot(self, src: int, dst: int) -> None:
        """dst <- src in every layer (a forked context continues from its parent's state)."""
        if src == dst:
            return
        if self.device.type != "cuda":
            self.conv_state[:, dst].copy_(self.conv_state[:, src])
            self.rec_state[:, dst].copy_(self.rec_state[:, src])
            return
        from .. import ops
        for buf in (self.conv_state, self.rec_state):
            ops.gdn_copy_slot(buf, src, dst)
