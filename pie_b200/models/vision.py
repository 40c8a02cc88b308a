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


# ----------------------------------------------------------------------------- SigLIP tower + Gemma-3 projector
@dataclass
class SiglipConfig:
    """The fixed-resolution vision tower of Gemma-3: `image_size / patch_size` patches a side with learned position
    rows, plain pre-LayerNorm blocks (biased projections, tanh-GELU MLP), a final LayerNorm; the projector averages
    the patch grid down to `mm_tokens_per_image` rows, applies a (1 + w) RMSNorm and one matrix into the language
    model's width."""
    image_size: int = 896
    patch_size: int = 14
    embed_dim: int = 1152
    intermediate_size: int = 4304
    depth: int = 27
    num_heads: int = 16
    mm_tokens_per_image: int = 256
    layer_norm_eps: float = 1e-6
    in_channels: int = 3
    hidden_size: int = 2560            # the language model's width

    @property
    def side(self) -> int:
        return self.image_size // self.patch_size

    @property
    def pool(self) -> int:
        return self.side // int(self.mm_tokens_per_image ** 0.5)

    @property
    def patch_features(self) -> int:
        return self.in_channels * self.patch_size * self.patch_size

    def to_dict(self) -> dict:
        return asdict(self)

    @staticmethod
    def from_hf(cfg: dict, llm_hidden: int = 0) -> "SiglipConfig":
        """From a Gemma-3 `config.json` (`vision_config` section + `mm_tokens_per_image`)."""
        v = cfg.get("vision_config") or {}
        return SiglipConfig(image_size=v.get("image_size", 896), patch_size=v.get("patch_size", 14), embed_dim=v.get("hidden_size", 1152),
                            intermediate_size=v.get("intermediate_size", 4304), depth=v.get("num_hidden_layers", 27),
                            num_heads=v.get("num_attention_heads", 16), mm_tokens_per_image=cfg.get("mm_tokens_per_image", 256),
                            layer_norm_eps=v.get("layer_norm_eps", 1e-6), in_channels=v.get("num_channels", 3), hidden_size=llm_hidden)


SIGLIP_PRESETS = {
    "tiny-siglip": dict(image_size=112, patch_size=14, embed_dim=64, intermediate_size=128, depth=2, num_heads=4,
                        mm_tokens_per_image=16, hidden_size=256),
    "gemma3-siglip": dict(hidden_size=2560),
}


def siglip_preset(name: str, **over) -> SiglipConfig:
    kw = dict(SIGLIP_PRESETS[name])
    kw.update(over)
    return SiglipConfig(**kw)


def random_siglip_weights(cfg: SiglipConfig, device="cpu", dtype=torch.float32, seed: int = 0) -> Dict[str, torch.Tensor]:
    """N(0, 0.05) weights under the checkpoint's names below `vision_tower.vision_model.` (patch embedding flattened to
    [E, C*p*p]) plus the projector's two tensors as `projector.*`; the projector's norm gain holds the full multiplier."""
    g = torch.Generator().manual_seed(seed)
    E, M = cfg.embed_dim, cfg.intermediate_size

    def n(*shape, std=0.05):
        return (torch.randn(*shape, generator=g) * std).to(dtype).to(device)

    w = {"embeddings.patch_embedding.weight": n(E, cfg.patch_features), "embeddings.patch_embedding.bias": n(E),
         "embeddings.position_embedding.weight": n(cfg.side * cfg.side, E), "post_layernorm.weight": 1 + n(E, std=0.1),
         "post_layernorm.bias": n(E), "projector.mm_soft_emb_norm.weight": 1 + n(E, std=0.1),
         "projector.mm_input_projection_weight": n(E, cfg.hidden_size)}
    for i in range(cfg.depth):
        L = f"encoder.layers.{i}."
        for nm in ("layer_norm1", "layer_norm2"):
            w[L + nm + ".weight"], w[L + nm + ".bias"] = 1 + n(E, std=0.1), n(E)
        for p in ("q_proj", "k_proj", "v_proj", "out_proj"):
            w[L + f"self_attn.{p}.weight"], w[L + f"self_attn.{p}.bias"] = n(E, E), n(E)
        w[L + "mlp.fc1.weight"], w[L + "mlp.fc1.bias"], w[L + "mlp.fc2.weight"], w[L + "mlp.fc2.bias"] = n(M, E), n(M), n(E, M), n(E)
    return w


def load_siglip_weights(reader, device="cpu", dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """`vision_tower.vision_model.*` and `multi_modal_projector.*` of a Gemma-3 checkpoint (with or without the leading
    `model.`); the projector's RMSNorm gain is stored as (w - 1) like the language model's and gets its 1 here."""
    out = {}
    for name in reader.names():
        key = name[len("model."):] if name.startswith("model.") else name
        if key.startswith("vision_tower.vision_model."):
            k = key[len("vision_tower.vision_model."):]
            t = reader.get(name)
            out[k] = (t.reshape(t.shape[0], -1) if k == "embeddings.patch_embedding.weight" else t).to(dtype).to(device)
        elif key.startswith("multi_modal_projector."):
            k = key[len("multi_modal_projector."):]
            t = reader.get(name)
            out["projector." + k] = ((t.float() + 1.0) if k == "mm_soft_emb_norm.weight" else t).to(dtype).to(device)
    if "embeddings.patch_embedding.weight" not in out:
        raise KeyError("checkpoint has no SigLIP tower (no vision_tower.vision_model.embeddings.patch_embedding.weight)")
    return out


class SiglipEncoder:
    """forward(patches, grids): patches [images * side^2, C*p*p] in row-major patch order (`multimodal.patchify_fixed`),
    grids [(1, side, side)] per image -> [images * mm_tokens_per_image, hidden_size]."""

    def __init__(self, cfg: SiglipConfig, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        first = weights["embeddings.patch_embedding.weight"]
        self.device, self.dtype = first.device, first.dtype

    def _lin(self, x, name):
        return F.linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))

    def _ln(self, x, name):
        return F.layer_norm(x, (x.shape[-1],), self.w[name + ".weight"], self.w[name + ".bias"], self.cfg.layer_norm_eps)

    @torch.no_grad()
    def forward(self, patches, grids) -> torch.Tensor:
        cfg = self.cfg
        S, E, H = cfg.side * cfg.side, cfg.embed_dim, cfg.num_heads
        x = torch.as_tensor(patches).to(self.device, self.dtype)
        if any(tuple(g) != (1, cfg.side, cfg.side) for g in grids) or x.shape != (len(grids) * S, cfg.patch_features):
            raise ValueError(f"this tower takes images of {cfg.side} x {cfg.side} patches with {cfg.patch_features} features; "
                             f"got rows {tuple(x.shape)} for grids {list(grids)}")
        B, hd = len(grids), E // H
        x = self._lin(x, "embeddings.patch_embedding").reshape(B, S, E) + self.w["embeddings.position_embedding.weight"]
        for i in range(cfg.depth):
            L = f"encoder.layers.{i}."
            y = self._ln(x, L + "layer_norm1")
            q, k, v = (self._lin(y, L + "self_attn." + p).reshape(B, S, H, hd).transpose(1, 2) for p in ("q_proj", "k_proj", "v_proj"))
            a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, S, E)
            x = x + self._lin(a, L + "self_attn.out_proj")
            x = x + self._lin(F.gelu(self._lin(self._ln(x, L + "layer_norm2"), L + "mlp.fc1"), approximate="tanh"), L + "mlp.fc2")
        x = self._ln(x, "post_layernorm")
        # projector: average the patch grid down, RMSNorm, one matrix into the language model's width
        x = F.avg_pool2d(x.transpose(1, 2).reshape(B, E, cfg.side, cfg.side), cfg.pool, cfg.pool).flatten(2).transpose(1, 2)
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + cfg.layer_norm_eps) * self.w["projector.mm_soft_emb_norm.weight"].float()
        return (xf.to(self.dtype) @ self.w["projector.mm_input_projection_weight"]).reshape(B * cfg.mm_tokens_per_image, cfg.hidden_size)

    __call__ = forward
