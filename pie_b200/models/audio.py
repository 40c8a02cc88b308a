"""Audio encoder for speech / sound inputs: a Whisper-style encoder with a linear projector (the layout of
Qwen2-Audio's audio tower).

Input is the log-mel spectrogram of `runtime.multimodal.audio_features` ([n_mels, frames], 10 ms per frame). Two
1-D convolutions (the second with stride 2) lift it to `d_model` at 20 ms per step, learned-size sinusoidal
position rows are added, `layers` pre-LayerNorm transformer blocks with full attention follow (key projection
without bias, GELU MLP), an average pool halves the rate again (40 ms per output row), a final LayerNorm and a
linear projector map into the language model's width. One output row per 40 ms: these rows replace the
embeddings of the clip's placeholder tokens.

Prefill-time component off the decode hot path; matrix products and attention go through torch.
Counterpart of the reference's audio encoders (driver/cuda/src/model/gemma4_audio.cpp).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Dict

import torch
import torch.nn.functional as F


@dataclass
class AudioConfig:
    num_mel_bins: int = 128
    d_model: int = 1280
    layers: int = 32
    heads: int = 20
    ffn_dim: int = 5120
    max_source_positions: int = 1500     # rows of the position table (20 ms steps: 30 s)
    hidden_size: int = 4096              # the language model's width (output of the projector)

    def to_dict(self) -> dict:
        return asdict(self)

    @staticmethod
    def from_hf(cfg: dict, llm_hidden: int = 0) -> "AudioConfig":
        """From the `audio_config` section of a Hugging Face multimodal `config.json`."""
        return AudioConfig(num_mel_bins=cfg.get("num_mel_bins", 128), d_model=cfg.get("d_model", 1280),
                           layers=cfg.get("encoder_layers", 32), heads=cfg.get("encoder_attention_heads", 20),
                           ffn_dim=cfg.get("encoder_ffn_dim", 5120), max_source_positions=cfg.get("max_source_positions", 1500),
                           hidden_size=llm_hidden)


AUDIO_PRESETS = {
    "tiny-audio": dict(num_mel_bins=80, d_model=64, layers=2, heads=4, ffn_dim=128, max_source_positions=1500, hidden_size=256),
    "qwen2-audio-encoder": dict(num_mel_bins=128, d_model=1280, layers=32, heads=20, ffn_dim=5120, hidden_size=4096),
}


def audio_preset(name: str, **over) -> AudioConfig:
    kw = dict(AUDIO_PRESETS[name])
    kw.update(over)
    return AudioConfig(**kw)


def audio_rows(frames: int) -> int:
    """Output rows for a spectrogram of `frames` frames: the stride-2 convolution, then the stride-2 pool."""
    return ((frames - 1) // 2 + 1) // 2 if frames > 0 else 0


def sinusoids(length: int, channels: int) -> torch.Tensor:
    """The fixed position rows Whisper checkpoints store in `embed_positions.weight`."""
    import math
    inc = math.log(10000.0) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2, dtype=torch.float32))
    t = torch.arange(length, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat([t.sin(), t.cos()], dim=1)


def random_audio_weights(cfg: AudioConfig, device="cpu", dtype=torch.float32, seed: int = 0) -> Dict[str, torch.Tensor]:
    """N(0, 0.05) weights under the checkpoint's names (`audio_tower.*` prefix removed, projector as `projector.*`)."""
    g = torch.Generator().manual_seed(seed)
    D, M = cfg.d_model, cfg.ffn_dim

    def n(*shape, std=0.05):
        return (torch.randn(*shape, generator=g) * std).to(dtype).to(device)

    w = {"conv1.weight": n(D, cfg.num_mel_bins, 3), "conv1.bias": n(D), "conv2.weight": n(D, D, 3), "conv2.bias": n(D),
         "embed_positions.weight": sinusoids(cfg.max_source_positions, D).to(dtype).to(device),
         "layer_norm.weight": 1 + n(D, std=0.1), "layer_norm.bias": n(D),
         "projector.linear.weight": n(cfg.hidden_size, D), "projector.linear.bias": n(cfg.hidden_size)}
    for i in range(cfg.layers):
        L = f"layers.{i}."
        w.update({L + "self_attn.q_proj.weight": n(D, D), L + "self_attn.q_proj.bias": n(D), L + "self_attn.k_proj.weight": n(D, D),
                  L + "self_attn.v_proj.weight": n(D, D), L + "self_attn.v_proj.bias": n(D),
                  L + "self_attn.out_proj.weight": n(D, D), L + "self_attn.out_proj.bias": n(D),
                  L + "self_attn_layer_norm.weight": 1 + n(D, std=0.1), L + "self_attn_layer_norm.bias": n(D),
                  L + "fc1.weight": n(M, D), L + "fc1.bias": n(M), L + "fc2.weight": n(D, M), L + "fc2.bias": n(D),
                  L + "final_layer_norm.weight": 1 + n(D, std=0.1), L + "final_layer_norm.bias": n(D)})
    return w


def load_audio_weights(reader, device="cpu", dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """The audio tower (`audio_tower.*`) and projector (`multi_modal_projector.*`) of a multimodal checkpoint."""
    out = {}
    for name in reader.names():
        for pre, new in (("model.audio_tower.", ""), ("audio_tower.", ""), ("model.multi_modal_projector.", "projector."),
                         ("multi_modal_projector.", "projector.")):
            if name.startswith(pre):
                out[new + name[len(pre):]] = reader.get(name).to(dtype).to(device)
                break
    if "conv1.weight" not in out:
        raise KeyError("checkpoint has no audio tower (no audio_tower.conv1.weight)")
    return out


class AudioEncoder:
    def __init__(self, cfg: AudioConfig, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        first = weights["conv1.weight"]
        self.device, self.dtype = first.device, first.dtype

    def _lin(self, x, name):
        return F.linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))

    def _ln(self, x, name):
        return F.layer_norm(x, (x.shape[-1],), self.w[name + ".weight"], self.w[name + ".bias"], 1e-5)

    @torch.no_grad()
    def forward(self, mel, grids=None) -> torch.Tensor:
        """mel [n_mels, frames] -> [audio_rows(frames), hidden_size]."""
        cfg = self.cfg
        x = torch.as_tensor(mel).to(self.device, self.dtype)
        if x.dim() != 2 or x.shape[0] != cfg.num_mel_bins:
            raise ValueError(f"spectrogram of shape {tuple(x.shape)}; the encoder takes [{cfg.num_mel_bins}, frames]")
        if (x.shape[1] - 1) // 2 + 1 > cfg.max_source_positions:
            raise ValueError(f"clip of {x.shape[1]} frames is longer than the encoder's {cfg.max_source_positions * 2}")
        x = F.gelu(F.conv1d(x[None], self.w["conv1.weight"], self.w["conv1.bias"], padding=1))
        x = F.gelu(F.conv1d(x, self.w["conv2.weight"], self.w["conv2.bias"], stride=2, padding=1))[0].t()      # [T, D]
        T, H = x.shape[0], cfg.heads
        hd = cfg.d_model // H
        x = x + self.w["embed_positions.weight"][:T]
        for i in range(cfg.layers):
            L = f"layers.{i}."
            y = self._ln(x, L + "self_attn_layer_norm")
            q, k, v = (self._lin(y, L + "self_attn." + p).reshape(T, H, hd).transpose(0, 1)[None] for p in ("q_proj", "k_proj", "v_proj"))
            a = F.scaled_dot_product_attention(q, k, v)[0].transpose(0, 1).reshape(T, H * hd)
            x = x + self._lin(a, L + "self_attn.out_proj")
            x = x + self._lin(F.gelu(self._lin(self._ln(x, L + "final_layer_norm"), L + "fc1")), L + "fc2")
        x = F.avg_pool1d(x.t()[None], 2, 2)[0].t()
        return self._lin(self._ln(x, "layer_norm"), "projector.linear")

    __call__ = forward
