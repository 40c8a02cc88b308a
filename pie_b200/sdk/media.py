"""Media inputs and audio output for inferlets (WIT `pie:core/media`, `pie:core/audio-out`).

Preprocessing runs on the host (`pie_b200.runtime.multimodal`); whether a model can consume the
result depends on its driver declaring an encoder (`Capabilities.media`). A driver built with a vision
encoder (`models.vision`) declares "image" and "video": `Context.append_image` / `append_video` then hand
the patch rows to the driver and splice one placeholder token per encoder row into the context. Text-only
models declare nothing and those calls raise `MediaUnsupported`; there is no audio encoder, so
`append_audio` always does. The preprocessing itself is usable on its own.
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
        return cls(mm.patchify([mm.decode_image(data)], **kw))

    @property
    def num_tokens(self) -> int:
        return self.features.num_tokens


@dataclass
class Video:
    features: mm.ImageFeatures

    @classmethod
    def from_bytes(cls, data: bytes, max_frames: int = 16, **kw) -> "Video":
        return cls(mm.patchify(mm.decode_frames(data, max_frames), **kw))

    @property
    def num_tokens(self) -> int:
        return self.features.num_tokens


@dataclass
class Audio:
    mel: np.ndarray       # [n_mels, frames]

    @classmethod
    def from_wav(cls, data: bytes, n_mels: int = 80) -> "Audio":
        return cls(mm.audio_features(data, n_mels=n_mels))


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
