"""Host-side preprocessing of media inputs, producing the tensors and position ids that a
vision / audio encoder consumes:

  images  (SigLIP towers) decode -> fixed square resize -> [-1, 1] -> row-major patch rows (`patchify_fixed`)
  images  decode (PIL) -> smart resize (both sides multiples of patch*merge, pixel budget) ->
          normalise -> patchify into [grid_h*grid_w, C*patch*patch] rows (+ temporal duplication)
  M-RoPE  3-axis (t, h, w) position ids for a text + image token sequence
  video   GIF / multi-frame image -> evenly sampled frames, grouped in temporal pairs
  audio   WAV decode -> mono -> resample to 16 kHz -> log-mel spectrogram (Whisper-style)

Counterpart of runtime/src/multimodal.rs:1-24 (overview), :239 (smart resize), :369 (M-RoPE
positions), :670+ (audio front end). The encoders that consume these tensors are `models.vision` and
`models.audio`; the media API hands the features to drivers that declare one.
"""
from __future__ import annotations

import io
import math
import wave
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np

IMAGENET_MEAN = np.array([0.48145466, 0.4578275, 0.40821073], dtype=np.float32)
IMAGENET_STD = np.array([0.26862954, 0.26130258, 0.27577711], dtype=np.float32)


# ------------------------------------------------------------------------------ images
def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56,
                 max_pixels: int = 14 * 14 * 4 * 1280) -> Tuple[int, int]:
    """Target size: both sides multiples of `factor`, aspect ratio kept as far as possible,
    area within [min_pixels, max_pixels]."""
    if min(height, width) <= 0:
        raise ValueError("empty image")
    if max(height, width) / min(height, width) > 200:
        raise ValueError("aspect ratio above 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


@dataclass
class ImageFeatures:
    patches: np.ndarray          # float32 [grid_t * grid_h * grid_w, C * temporal * patch * patch]
    grid: Tuple[int, int, int]   # (t, h, w) in patches
    merge: int                   # spatial merge of the encoder's output (tokens = t*h*w / merge^2)

    @property
    def num_tokens(self) -> int:
        t, h, w = self.grid
        return t * h * w // (self.merge * self.merge)


def decode_image(data: bytes) -> np.ndarray:
    from PIL import Image
    img = Image.open(io.BytesIO(data))
    return np.asarray(img.convert("RGB"), dtype=np.uint8)


def decode_frames(data: bytes, max_frames: int = 16) -> List[np.ndarray]:
    """Frames of an animated image (GIF / APNG / multi-page), evenly sampled."""
    from PIL import Image, ImageSequence
    img = Image.open(io.BytesIO(data))
    frames = [np.asarray(f.convert("RGB"), dtype=np.uint8) for f in ImageSequence.Iterator(img)]
    if len(frames) > max_frames:
        idx = np.linspace(0, len(frames) - 1, max_frames).round().astype(int)
        frames = [frames[i] for i in idx]
    return frames


def _resize(rgb: np.ndarray, h: int, w: int) -> np.ndarray:
    from PIL import Image
    return np.asarray(Image.fromarray(rgb).resize((w, h), Image.BICUBIC), dtype=np.uint8)


def patchify(frames: Sequence[np.ndarray], patch: int = 14, merge: int = 2, temporal: int = 2,
             min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280,
             mean: np.ndarray = IMAGENET_MEAN, std: np.ndarray = IMAGENET_STD) -> ImageFeatures:
    """Qwen-VL style patch rows. A single image is one frame repeated `temporal` times."""
    frames = list(frames)
    h0, w0 = frames[0].shape[:2]
    h, w = smart_resize(h0, w0, patch * merge, min_pixels, max_pixels)
    x = np.stack([(_resize(f, h, w).astype(np.float32) / 255.0 - mean) / std for f in frames])   # [T,H,W,C]
    if x.shape[0] % temporal:
        x = np.concatenate([x, np.repeat(x[-1:], temporal - x.shape[0] % temporal, axis=0)])
    x = x.transpose(0, 3, 1, 2)                                                                   # [T,C,H,W]
    gt, gh, gw = x.shape[0] // temporal, h // patch, w // patch
    x = x.reshape(gt, temporal, 3, gh // merge, merge, patch, gw // merge, merge, patch)
    # rows ordered (t, h-block, w-block, h-in-block, w-in-block) so that merged neighbours are adjacent
    x = x.transpose(0, 3, 6, 4, 7, 2, 1, 5, 8)
    return ImageFeatures(np.ascontiguousarray(x.reshape(gt * gh * gw, 3 * temporal * patch * patch)), (gt, gh, gw), merge)


def patchify_fixed(frames: Sequence[np.ndarray], image_size: int = 896, patch: int = 14, pool: int = 4,
                   mean: float = 0.5, std: float = 0.5) -> ImageFeatures:
    """SigLIP-style patch rows (Gemma-3): every frame is resized to `image_size` squared whatever its aspect ratio,
    normalised to [-1, 1], and cut into `patch`-sized squares in row-major order; a row holds (channel, patch row,
    patch column). `pool` is the side of the average pool of the model's projector: tokens = patches / pool^2."""
    side = image_size // patch
    rows = []
    for f in frames:
        x = (_resize(f, image_size, image_size).astype(np.float32) / 255.0 - mean) / std          # [H, W, C]
        x = x.transpose(2, 0, 1).reshape(3, side, patch, side, patch).transpose(1, 3, 0, 2, 4)
        rows.append(x.reshape(side * side, 3 * patch * patch))
    return ImageFeatures(np.ascontiguousarray(np.concatenate(rows)), (len(rows), side, side), pool)


def mrope_positions(segments: Sequence[tuple], merge: int = 2) -> np.ndarray:
    """3-axis position ids [3, N] for a sequence of segments: ("text", n) or ("image", (t, h, w)).
    Text advances all three axes together; an image block starts at the running position and
    spans (t, h/merge, w/merge); the next segment starts past the largest id used."""
    out, pos = [], 0
    for kind, v in segments:
        if kind == "text":
            ids = np.arange(pos, pos + v)
            out.append(np.stack([ids, ids, ids]))
            pos += v
        else:
            t, h, w = v
            h, w = h // merge, w // merge
            tt, hh, ww = np.meshgrid(np.arange(t), np.arange(h), np.arange(w), indexing="ij")
            out.append(np.stack([tt.ravel(), hh.ravel(), ww.ravel()]) + pos)
            pos += max(t, h, w)
    return np.concatenate(out, axis=1).astype(np.int32) if out else np.zeros((3, 0), np.int32)


# ------------------------------------------------------------------------------ audio
def decode_wav(data: bytes) -> Tuple[np.ndarray, int]:
    """PCM WAV (8/16/24/32-bit) -> float32 mono in [-1, 1] and its sample rate."""
    with wave.open(io.BytesIO(data)) as w:
        n, ch, sw, sr = w.getnframes(), w.getnchannels(), w.getsampwidth(), w.getframerate()
        raw = w.readframes(n)
    if sw == 1:
        x = (np.frombuffer(raw, dtype=np.uint8).astype(np.float32) - 128.0) / 128.0
    elif sw == 2:
        x = np.frombuffer(raw, dtype="<i2").astype(np.float32) / 32768.0
    elif sw == 3:
        b = np.frombuffer(raw, dtype=np.uint8).reshape(-1, 3).astype(np.int32)
        v = b[:, 0] | (b[:, 1] << 8) | (b[:, 2] << 16)
        x = (v - ((v & 0x800000) << 1)).astype(np.float32) / 8388608.0
    elif sw == 4:
        x = np.frombuffer(raw, dtype="<i4").astype(np.float32) / 2147483648.0
    else:
        raise ValueError(f"unsupported sample width {sw}")
    return x.reshape(-1, ch).mean(axis=1), sr


def encode_wav(samples: np.ndarray, sample_rate: int) -> bytes:
    """float mono [-1, 1] -> 16-bit PCM WAV (audio-out results)."""
    buf = io.BytesIO()
    with wave.open(buf, "wb") as w:
        w.setnchannels(1)
        w.setsampwidth(2)
        w.setframerate(sample_rate)
        w.writeframes((np.clip(samples, -1, 1) * 32767).astype("<i2").tobytes())
    return buf.getvalue()


def resample(x: np.ndarray, sr_in: int, sr_out: int) -> np.ndarray:
    if sr_in == sr_out or len(x) == 0:
        return x.astype(np.float32)
    from scipy.signal import resample_poly
    g = math.gcd(sr_in, sr_out)
    return resample_poly(x, sr_out // g, sr_in // g).astype(np.float32)


def mel_filterbank(n_mels: int = 80, n_fft: int = 400, sr: int = 16000) -> np.ndarray:
    """Slaney-style triangular filters [n_mels, n_fft/2+1]."""
    def hz_to_mel(f):
        f = np.asarray(f, dtype=np.float64)
        lin = f / (200.0 / 3)
        log = 15.0 + np.log(np.maximum(f, 1e-10) / 1000.0) / (np.log(6.4) / 27.0)
        return np.where(f >= 1000.0, log, lin)

    def mel_to_hz(m):
        m = np.asarray(m, dtype=np.float64)
        return np.where(m >= 15.0, 1000.0 * np.exp((np.log(6.4) / 27.0) * (m - 15.0)), m * (200.0 / 3))

    freqs = np.linspace(0, sr / 2, n_fft // 2 + 1)
    pts = mel_to_hz(np.linspace(hz_to_mel(0.0), hz_to_mel(sr / 2), n_mels + 2))
    fb = np.zeros((n_mels, len(freqs)))
    for i in range(n_mels):
        lo, c, hi = pts[i], pts[i + 1], pts[i + 2]
        fb[i] = np.maximum(0, np.minimum((freqs - lo) / (c - lo), (hi - freqs) / (hi - c)))
        fb[i] *= 2.0 / (hi - lo)
    return fb.astype(np.float32)


def log_mel(x: np.ndarray, sr: int = 16000, n_fft: int = 400, hop: int = 160, n_mels: int = 80,
            pad_to_seconds: Optional[float] = None) -> np.ndarray:
    """Whisper-style log-mel spectrogram [n_mels, frames] of 16 kHz mono audio."""
    if pad_to_seconds:
        want = int(pad_to_seconds * sr)
        x = np.pad(x[:want], (0, max(0, want - len(x))))
    x = np.pad(x, (n_fft // 2, n_fft // 2), mode="reflect")
    frames = 1 + (len(x) - n_fft) // hop
    idx = np.arange(n_fft)[None, :] + hop * np.arange(frames)[:, None]
    win = np.hanning(n_fft + 1)[:-1].astype(np.float32)
    spec = np.abs(np.fft.rfft(x[idx] * win, axis=1)) ** 2
    mel = mel_filterbank(n_mels, n_fft, sr) @ spec[:-1].T if frames > 1 else mel_filterbank(n_mels, n_fft, sr) @ spec.T
    logm = np.log10(np.maximum(mel, 1e-10))
    logm = np.maximum(logm, logm.max() - 8.0)
    return ((logm + 4.0) / 4.0).astype(np.float32)


def audio_features(data: bytes, sr: int = 16000, n_mels: int = 80) -> np.ndarray:
    x, sr_in = decode_wav(data)
    return log_mel(resample(x, sr_in, sr), sr, n_mels=n_mels)
