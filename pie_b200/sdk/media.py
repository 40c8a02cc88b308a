"""Media inputs and audio output for inferlets (WIT `pie:core/media`, `pie:core/audio-out`).

Preprocessing runs on the host (`pie_b200.runtime.multimodal`); whether a model can consume the
result depends on its driver declaring an encoder (`Capabilities.media`). A driver built with a vision
encoder (`models.vision`) declares "image" and "video", one with an audio encoder (`models.audio`) "audio":
`Context.append_image` / `append_video` / `append_audio` then hand the patch rows or the spectrogram to the
driver and splice one placeholder token per encoder row into the context. Text-only models declare nothing
and those calls raise `MediaUnsupported`. The preprocessing itself is usable on its own.
Counterpart of sdk/python/src/inferlet/media.py and audio.py.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import numpy as np

from ..runtime import multimodal as mm


class MediaUnsupported(RuntimeError):
    pass


@dataclass
class Image:
    features: mm.ImageFeatures

    @classmethod
    def from_bytes(cls, data: bytes, **kw) -> "Image":
        """Qwen-VL style preprocessing (smart resize, merge-block patch order)."""
        return cls(mm.patchify([mm.decode_image(data)], **kw))

    @classmethod
    def for_model(cls, model, data: bytes, **kw) -> "Image":
        """Preprocess the way the model's vision tower wants it (`Capabilities.media_spec`): an inferlet written with
        this call serves any vision model unchanged. `kw` overrides single settings (e.g. `max_pixels`)."""
        return cls(_features_for(model, [mm.decode_image(data)], kw))

    @property
    def num_tokens(self) -> int:
        return self.features.num_tokens


@dataclass
class Video:
    features: mm.ImageFeatures

    @classmethod
    def from_bytes(cls, data: bytes, max_frames: int = 16, **kw) -> "Video":
        return cls(mm.patchify(mm.decode_frames(data, max_frames), **kw))

    @classmethod
    def for_model(cls, model, data: bytes, max_frames: int = 16, **kw) -> "Video":
        return cls(_features_for(model, mm.decode_frames(data, max_frames), kw))

    @property
    def num_tokens(self) -> int:
        return self.features.num_tokens


@dataclass
class Audio:
    mel: np.ndarray       # [n_mels, frames], 10 ms per frame

    @classmethod
    def from_wav(cls, data: bytes, n_mels: int = 80) -> "Audio":
        return cls(mm.audio_features(data, n_mels=n_mels))

    @property
    def num_tokens(self) -> int:
        """Rows of the audio encoder's output (one per 40 ms: a stride-2 convolution, then a stride-2 pool)."""
        f = self.mel.shape[1]
        return ((f - 1) // 2 + 1) // 2 if f > 0 else 0

    # the shape `Context._append_clip` takes: the array that goes to the encoder and its grid
    @property
    def patches(self) -> np.ndarray:
        return self.mel

    @property
    def grid(self):
        return (int(self.mel.shape[1]),)


def _features_for(model, frames, kw: dict):
    spec = dict(getattr(model._entry.caps[0], "media_spec", None) or {})
    if spec.get("style") == "siglip":
        args = dict(image_size=spec["image_size"], patch=spec["patch"], pool=spec["pool"])
        args.update({k: v for k, v in kw.items() if k in ("mean", "std")})
        return mm.patchify_fixed(frames, **args)
    args = {k: spec[k] for k in ("patch", "merge", "temporal") if k in spec}
    args.update(kw)
    return mm.patchify(frames, **args)


def supported(model) -> List[str]:
    """Media kinds the model's driver can encode ([] for text-only models)."""
    return list(getattr(model._entry.caps[0], "media", ()) or ())


def require(model, kind: str) -> None:
    if kind not in supported(model):
        raise MediaUnsupported(f"model {model.name} has no {kind} encoder")


def positions_for(segments, merge: int = 2) -> np.ndarray:
    return mm.mrope_positions(segments, merge)


def wav_bytes(samples: np.ndarray, sample_rate: int = 24000) -> bytes:
    """Encode generated audio for `session.send_file` (audio-out)."""
    return mm.encode_wav(np.asarray(samples, dtype=np.float32), sample_rate)
