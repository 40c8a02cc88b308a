"""Media preprocessing: smart resize invariants, patch layout, M-RoPE ids, WAV codec,
resampling and the log-mel front end."""
import io

import numpy as np
import pytest

from pie_b200.runtime import multimodal as mm


def test_smart_resize_invariants():
    for h, w in [(480, 640), (31, 900), (4000, 3000), (20, 20), (1080, 1920)]:
        H, W = mm.smart_resize(h, w)
        assert H % 28 == 0 and W % 28 == 0
        assert 56 * 56 <= H * W <= 14 * 14 * 4 * 1280
        assert abs((H / W) - (h / w)) / (h / w) < 0.35
    with pytest.raises(ValueError):
        mm.smart_resize(1, 1000)


def test_patchify_layout_and_tokens():
    from PIL import Image
    rng = np.random.default_rng(0)
    img = rng.integers(0, 255, (112, 168, 3), dtype=np.uint8)
    buf = io.BytesIO()
    Image.fromarray(img).save(buf, format="PNG")
    rgb = mm.decode_image(buf.getvalue())
    assert rgb.shape == (112, 168, 3) and (rgb == img).all()
    f = mm.patchify([rgb])
    t, h, w = f.grid
    assert (t, h, w) == (1, 8, 12) and f.patches.shape == (96, 3 * 2 * 14 * 14) and f.num_tokens == 24
    # row 0 is the top-left patch, channel 0, first temporal copy
    want = (img[:14, :14, 0].astype(np.float32) / 255 - mm.IMAGENET_MEAN[0]) / mm.IMAGENET_STD[0]
    got = f.patches[0].reshape(3, 2, 14, 14)[0, 0]
    assert np.abs(got - want).max() < 1e-5
    # row 1 is its right neighbour inside the same 2x2 merge block
    want1 = (img[:14, 14:28, 1].astype(np.float32) / 255 - mm.IMAGENET_MEAN[1]) / mm.IMAGENET_STD[1]
    assert np.abs(f.patches[1].reshape(3, 2, 14, 14)[1, 1] - want1).max() < 1e-5


def test_video_frames_pair_up():
    from PIL import Image
    frames = [Image.fromarray(np.full((56, 56, 3), 10 * i, dtype=np.uint8)) for i in range(5)]
    buf = io.BytesIO()
    frames[0].save(buf, format="GIF", save_all=True, append_images=frames[1:], duration=40)
    got = mm.decode_frames(buf.getvalue(), max_frames=4)
    assert len(got) == 4
    f = mm.patchify(got)
    assert f.grid[0] == 2


def test_mrope_positions():
    pos = mm.mrope_positions([("text", 3), ("image", (1, 4, 6)), ("text", 2)])
    assert pos.shape == (3, 3 + 6 + 2)
    assert pos[:, :3].tolist() == [[0, 1, 2]] * 3
    img = pos[:, 3:9]
    assert img[0].tolist() == [3] * 6 and img[1].tolist() == [3, 3, 3, 4, 4, 4] and img[2].tolist() == [3, 4, 5] * 2
    assert pos[:, 9:].tolist() == [[6, 7]] * 3            # continues past max(t, h, w) = 3


def test_wav_roundtrip_resample_and_mel():
    sr = 44100
    t = np.arange(sr) / sr
    x = 0.5 * np.sin(2 * np.pi * 440 * t).astype(np.float32)
    data = mm.encode_wav(x, sr)
    y, sr2 = mm.decode_wav(data)
    assert sr2 == sr and np.abs(x - y).max() < 1e-3
    z = mm.resample(y, sr, 16000)
    assert abs(len(z) - 16000) <= 1
    mel = mm.audio_features(data)
    assert mel.shape[0] == 80 and abs(mel.shape[1] - 100) <= 1
    fb = mm.mel_filterbank()
    peak_bin = int(np.argmax(mel.mean(axis=1)))
    centre = np.argmax(fb[peak_bin]) * 16000 / 400
    assert abs(centre - 440) < 80                          # the loudest mel band sits at the tone
