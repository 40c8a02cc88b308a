"""Vision encoder for image / video inputs: a Qwen2-VL style vision transformer.

Patch rows come from `runtime.multimodal.patchify` (one row per patch, features ordered channel, temporal
frame, patch row, patch column; rows ordered so that the `merge x merge` neighbours that the merger joins are
adjacent). The tower is: linear patch embedding -> `depth` pre-LayerNorm blocks (full attention inside each
temporal frame group with 2-D rotary positions: half of the rotary pairs turn with the patch's row, half with
its column; QuickGELU MLP) -> merger (LayerNorm, concatenate each `merge x merge` neighbourhood, two-layer
MLP into the language model's hidden size). One output row per merged patch: these rows replace the
embeddings of the image's placeholder tokens in the language model.

The encoder is a prefill-time component off the decode hot path; its matrix products and attention go
through torch (cuBLAS / SDPA). Counterpart of the reference's vision encoders
(driver/cuda/src/model/qwen3_vl_vision.cpp, driver/cuda/src/kernels/vision_*.cu).
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass
from typing import Dict, List, Sequence, Tuple

import torch
import torch.nn.functional as F


@dataclass
class VisionConfig:
    depth: int = 32
    embed_dim: int = 1280
    num_heads: int = 16
    mlp_ratio: float = 4.0
    patch_size: int = 14
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    in_channels: int = 3
    hidden_size: int = 3584          # the language model's width (output of the merger)
    rope_theta: float = 10000.0

    @property
    def patch_features(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size

    @property
    def merge_unit(self) -> int:
        return self.spatial_merge_size * self.spatial_merge_size

    def to_dict(self) -> dict:
        return asdict(self)

    @staticmethod
    def from_hf(cfg: dict, llm_hidden: int = 0) -> "VisionConfig":
        """From the `vision_config` section of a Hugging Face multimodal `config.json`."""
        return VisionConfig(
            depth=cfg.get("depth", 32), embed_dim=cfg.get("embed_dim", 1280), num_heads=cfg.get("num_heads", 16),
            mlp_ratio=cfg.get("mlp_ratio", 4.0), patch_size=cfg.get("patch_size", 14),
            spatial_merge_size=cfg.get("spatial_merge_size", 2), temporal_patch_size=cfg.get("temporal_patch_size", 2),
            in_channels=cfg.get("in_channels", cfg.get("in_chans", 3)), hidden_size=cfg.get("hidden_size") or llm_hidden)


VISION_PRESETS = {
    "tiny-vit": dict(depth=2, embed_dim=64, num_heads=4, mlp_ratio=2.0, patch_size=14, spatial_merge_size=2,
                     temporal_patch_size=2, in_channels=3, hidden_size=256),
    "qwen2-vl-7b-vit": dict(depth=32, embed_dim=1280, num_heads=16, mlp_ratio=4.0, hidden_size=3584),
}


def vision_preset(name: str, **over) -> VisionConfig:
    kw = dict(VISION_PRESETS[name])
    kw.update(over)
    return VisionConfig(**kw)


def random_vision_weights(cfg: VisionConfig, device="cpu", dtype=torch.float32, seed: int = 0) -> Dict[str, torch.Tensor]:
    """N(0, 0.05) weights under the checkpoint's own names (`patch_embed.proj.weight` as the flattened
    convolution kernel [embed_dim, patch_features])."""
    g = torch.Generator().manual_seed(seed)
    E, M = cfg.embed_dim, int(cfg.embed_dim * cfg.mlp_ratio)
    U = E * cfg.merge_unit

    def n(*shape, std=0.05):
        return (torch.randn(*shape, generator=g) * std).to(dtype).to(device)

    w = {"patch_embed.proj.weight": n(E, cfg.patch_features)}
    for i in range(cfg.depth):
        B = f"blocks.{i}."
        w.update({B + "norm1.weight": 1 + n(E, std=0.1), B + "norm1.bias": n(E), B + "norm2.weight": 1 + n(E, std=0.1),
                  B + "norm2.bias": n(E), B + "attn.qkv.weight": n(3 * E, E), B + "attn.qkv.bias": n(3 * E),
                  B + "attn.proj.weight": n(E, E), B + "attn.proj.bias": n(E), B + "mlp.fc1.weight": n(M, E),
                  B + "mlp.fc1.bias": n(M), B + "mlp.fc2.weight": n(E, M), B + "mlp.fc2.bias": n(E)})
    w.update({"merger.ln_q.weight": 1 + n(E, std=0.1), "merger.ln_q.bias": n(E), "merger.mlp.0.weight": n(U, U),
              "merger.mlp.0.bias": n(U), "merger.mlp.2.weight": n(cfg.hidden_size, U), "merger.mlp.2.bias": n(cfg.hidden_size)})
    return w


def load_vision_weights(reader, device="cpu", dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """The vision tower's tensors of a multimodal checkpoint (`visual.*` or `model.visual.*`), prefix removed;
    the patch embedding's convolution kernel [E, C, T, P, P] is flattened to [E, C*T*P*P]."""
    out = {}
    for name in reader.names():
        for pre in ("model.visual.", "visual."):
            if name.startswith(pre):
                t = reader.get(name)
                key = name[len(pre):]
                if key == "patch_embed.proj.weight":
                    t = t.reshape(t.shape[0], -1)
                out[key] = t.to(dtype).to(device)
                break
    if "patch_embed.proj.weight" not in out:
        raise KeyError("checkpoint has no vision tower (no visual.patch_embed.proj.weight)")
    return out


def rotary_angles(cfg: VisionConfig, grids: Sequence[Tuple[int, int, int]], device) -> torch.Tensor:
    """[rows, head_dim / 2] rotary angles: the first half of the pairs turn with the patch's row, the second half
    with its column, in the row order of `patchify` (merge blocks adjacent)."""
    hd = cfg.embed_dim // cfg.num_heads
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd // 2, 2, dtype=torch.float32, device=device) / (hd // 2)))
    m, parts = cfg.spatial_merge_size, []
    for t, h, w in grids:
        hp = torch.arange(h, device=device).unsqueeze(1).expand(-1, w)
        wp = torch.arange(w, device=device).unsqueeze(0).expand(h, -1)
        blk = lambda x: x.reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
        pos = torch.stack([blk(hp), blk(wp)], dim=-1).repeat(t, 1).float()          # [t*h*w, 2]
        parts.append(torch.cat([pos[:, 0:1] * inv, pos[:, 1:2] * inv], dim=-1))
    return torch.cat(parts, 0)


class VisionEncoder:
    def __init__(self, cfg: VisionConfig, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        first = weights["patch_embed.proj.weight"]
        self.device, self.dtype = first.device, first.dtype

    def _lin(self, x, name):
        return F.linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))

    def _ln(self, x, name):
        return F.layer_norm(x, (x.shape[-1],), self.w[name + ".weight"], self.w[name + ".bias"], 1e-6)

    @torch.no_grad()
    def forward(self, patches, grids: Sequence[Tuple[int, int, int]]) -> torch.Tensor:
        """patches [rows, patch_features] of one or more images (rows = sum of t*h*w), grids their (t, h, w) in
        patches. Returns [rows / merge^2, hidden_size]."""
        cfg = self.cfg
        x = torch.as_tensor(patches).to(self.device, self.dtype)
        rows = sum(t * h * w for t, h, w in grids)
        if x.shape != (rows, cfg.patch_features):
            raise ValueError(f"patch rows {tuple(x.shape)} do not match grids {list(grids)} x {cfg.patch_features} features")
        if any(h % cfg.spatial_merge_size or w % cfg.spatial_merge_size for _, h, w in grids):
            raise ValueError("grid sides must be multiples of the spatial merge size")
        H, hd = cfg.num_heads, cfg.embed_dim // cfg.num_heads
        x = F.linear(x, self.w["patch_embed.proj.weight"])
        ang = rotary_angles(cfg, grids, self.device)
        ang = torch.cat([ang, ang], dim=-1)                     # rotate-half layout over the head
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        # attention runs inside each temporal frame group
        seqs = [h * w for t, h, w in grids for _ in range(t)]

        def rope(v):
            vf = v.float()
            rot = torch.cat([-vf[..., hd // 2:], vf[..., :hd // 2]], dim=-1)
            return (vf * cos + rot * sin).to(v.dtype)

        for i in range(cfg.depth):
            B = f"blocks.{i}"
            qkv = self._lin(self._ln(x, B + ".norm1"), B + ".attn.qkv").reshape(rows, 3, H, hd)
            q, k, v = rope(qkv[:, 0]), rope(qkv[:, 1]), qkv[:, 2]
            outs, a = [], 0
            for n in seqs:
                qs, ks, vs = (z[a:a + n].transpose(0, 1)[None] for z in (q, k, v))      # [1, H, n, hd]
                outs.append(F.scaled_dot_product_attention(qs, ks, vs)[0].transpose(0, 1).reshape(n, H * hd))
                a += n
            x = x + self._lin(torch.cat(outs, 0), B + ".attn.proj")
            y = self._lin(self._ln(x, B + ".norm2"), B + ".mlp.fc1")
            x = x + self._lin(y * torch.sigmoid(1.702 * y), B + ".mlp.fc2")             # QuickGELU
        x = self._ln(x, "merger.ln_q").reshape(rows // cfg.merge_unit, cfg.merge_unit * cfg.embed_dim)
        return self._lin(F.gelu(self._lin(x, "merger.mlp.0")), "merger.mlp.2")

    __call__ = forward

    def num_tokens(self, grid: Tuple[int, int, int]) -> int:
        t, h, w = grid
        return t * h * w // self.cfg.merge_unit
