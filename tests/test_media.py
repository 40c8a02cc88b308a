"""Media inputs end to end on the CPU driver: vision tower against transformers' Qwen2-VL tower; placeholder
tokens -> media spans -> embedding override in the driver; generation over an image equals the dense oracle fed
with the encoder's rows; chunked prefill through an image; content-addressed sharing of clips and of their KV
pages; slot release with the last context; replay after eviction; the wire format; the example inferlets."""
import base64
import io
import json

import numpy as np
import pytest
import torch

from pie_b200.driver import abi
from pie_b200.driver.executor import TorchDriver
from pie_b200.driver.schema import MEDIA_TOKEN_BASE, ForwardRequest, media_tokens, split_media_spans
from pie_b200.inferlets import install_all
from pie_b200.models.config import preset
from pie_b200.models.transformer import dense_reference_forward
from pie_b200.models.vision import VisionEncoder, random_vision_weights, vision_preset
from pie_b200.models.weights import random_weights
from pie_b200.runtime import multimodal as mm
from pie_b200.runtime.engine import Engine, EngineConfig
from pie_b200.runtime.scheduler import PendingRequest, fold
from pie_b200.runtime.tokenizer import ByteTokenizer


def png_bytes(seed: int, h: int = 60, w: int = 90) -> bytes:
    from PIL import Image
    rng = np.random.default_rng(seed)
    buf = io.BytesIO()
    Image.fromarray(rng.integers(0, 255, (h, w, 3), dtype=np.uint8)).save(buf, format="PNG")
    return buf.getvalue()


def gif_bytes(frames: int = 4) -> bytes:
    from PIL import Image
    rng = np.random.default_rng(9)
    ims = [Image.fromarray(rng.integers(0, 255, (56, 56, 3), dtype=np.uint8)) for _ in range(frames)]
    buf = io.BytesIO()
    ims[0].save(buf, format="GIF", save_all=True, append_images=ims[1:])
    return buf.getvalue()


def test_vision_tower_equals_transformers_qwen2_vl():
    from transformers.models.qwen2_vl import modeling_qwen2_vl as m
    from transformers.models.qwen2_vl.configuration_qwen2_vl import Qwen2VLVisionConfig
    cfg = vision_preset("tiny-vit", hidden_size=128)
    w = random_vision_weights(cfg, seed=1)
    c = Qwen2VLVisionConfig(depth=cfg.depth, embed_dim=cfg.embed_dim, hidden_size=cfg.hidden_size, num_heads=cfg.num_heads,
                            mlp_ratio=int(cfg.mlp_ratio), patch_size=14, spatial_merge_size=2, temporal_patch_size=2, in_channels=3)
    c._attn_implementation = "eager"
    tower = m.Qwen2VisionTransformerPretrainedModel(c).float().eval()
    sd = dict(w)
    sd["patch_embed.proj.weight"] = w["patch_embed.proj.weight"].reshape(cfg.embed_dim, 3, 2, 14, 14)
    tower.load_state_dict(sd, strict=True)
    # a real preprocessing result (row order and feature order of `patchify`) and a two-frame-group clip
    f1 = mm.patchify([mm.decode_image(png_bytes(1))], min_pixels=28 * 28, max_pixels=28 * 28 * 12)
    f2 = mm.patchify(mm.decode_frames(gif_bytes(4)), min_pixels=28 * 28, max_pixels=28 * 28 * 4)
    assert f2.grid[0] == 2
    x = torch.from_numpy(np.concatenate([f1.patches, f2.patches]))
    with torch.no_grad():
        want = tower(x, torch.tensor([f1.grid, f2.grid]))
    want = want if torch.is_tensor(want) else want.pooler_output
    got = VisionEncoder(cfg, w)(x, [f1.grid, f2.grid])
    assert got.shape == (f1.num_tokens + f2.num_tokens, 128) and (got - want).abs().max() < 1e-5


def test_placeholders_become_spans_and_cross_the_wire():
    t = [5, 6] + media_tokens(3, 4) + [7] + media_tokens(3, 2, 4) + media_tokens(9, 3)
    toks, slot, src, dst, cnt = split_media_spans(np.array(t))
    assert toks.tolist() == [5, 6, 0, 0, 0, 0, 7, 0, 0, 0, 0, 0]
    assert (slot.tolist(), src.tolist(), dst.tolist(), cnt.tolist()) == ([3, 3, 9], [0, 4, 0], [2, 7, 9], [4, 2, 3])
    assert split_media_spans(np.array([1, 2, 3]))[1] is None
    a = PendingRequest(0, [11] + media_tokens(2, 5), list(range(6)), [0], 0, [])
    b = PendingRequest(1, media_tokens(2, 3, 5) + [12], list(range(6, 10)), [1], 6, [])
    req = fold([a, b], 16)
    assert req.tokens.tolist() == [11, 0, 0, 0, 0, 0, 0, 0, 0, 12]
    # the two requests carry consecutive rows of one clip at consecutive batch rows: one span covers both
    assert (req.media_slot.tolist(), req.media_src.tolist(), req.media_dst.tolist(), req.media_count.tolist()) == \
        ([2], [0], [1], [8])
    back = abi.unpack_forward_request(abi.pack_forward_request(req))
    for k in ("media_slot", "media_src", "media_dst", "media_count", "tokens"):
        assert np.array_equal(getattr(back, k), getattr(req, k)), k
    plain = abi.unpack_forward_request(abi.pack_forward_request(fold([PendingRequest(0, [1, 2], [0, 1], [0], 0, [])], 16)))
    assert plain.media_slot is None


@pytest.fixture()
def eng():
    cfg = preset("tiny-llama")
    w = random_weights(cfg, "cpu", torch.float32, seed=3)
    vcfg = vision_preset("tiny-vit", hidden_size=cfg.hidden_size)
    enc = VisionEncoder(vcfg, random_vision_weights(vcfg, seed=5))
    drv = TorchDriver(cfg, "cpu", weights=w, num_pages=64, page_size=16, max_requests=8, max_tokens=48, vision=enc)
    e = Engine(EngineConfig())
    e.add_model("vlm", drv, tokenizer=ByteTokenizer(cfg.vocab_size))
    install_all(e)
    yield e, cfg, w, enc, drv
    e.shutdown()


def oracle(cfg, w, enc, feats, pre, post, n):
    """Greedy continuation of pre + image + post by the dense model, the image rows replaced by the encoder's output."""
    rows = enc(feats.patches, [feats.grid])
    toks = list(pre) + [0] * rows.shape[0] + list(post)
    emb = {len(pre) + i: rows[i] for i in range(rows.shape[0])}
    out = []
    for _ in range(n):
        nxt = int(dense_reference_forward(cfg, w, torch.tensor(toks), embeds=emb)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out


def test_generation_over_an_image_equals_the_oracle_and_shares_work(eng):
    e, cfg, w, enc, drv = eng
    assert drv.capabilities().media == ("image", "video") and e.models["vlm"].media is not None
    data = png_bytes(2, 280, 420)
    resize = dict(min_pixels=28 * 28, max_pixels=28 * 28 * 80)
    feats = mm.patchify([mm.decode_image(data)], **resize)
    assert feats.num_tokens > 48                 # more image rows than one fire takes: the prefill is chunked inside the image
    q = "What is this?"
    args = {"image_b64": base64.b64encode(data).decode(), "question": q, "max_tokens": 5, "temperature": 0.0, "resize": resize}
    out = json.loads(e.run("image-qa", args, 300))
    assert out["ok"] and out["image_tokens"] == feats.num_tokens and out["grid"] == list(feats.grid)
    assert out["tokens"] == oracle(cfg, w, enc, feats, [], ByteTokenizer(cfg.vocab_size).encode(q), 5)
    entry = e.models["vlm"]
    assert entry.schedulers[0].stats["chunked_requests"] >= 1
    # the context is gone: so is the clip, on the registry and (once its worker has run) on the driver
    entry.media.drain()
    assert entry.media.stats()["resident"] == 0 and drv.media == {}
    # the same image twice in a row inside one program: encoded once; the second context reuses the first one's pages
    before = entry.ctxm.counters["dedup_pages"]
    out2 = json.loads(e.run("multi-image-test", {"images_b64": [args["image_b64"], base64.b64encode(png_bytes(7)).decode()],
                                                 "rounds": 2, "max_tokens": 3, "resize": resize}, 300))
    assert out2["ok"] and out2["same_output"] and out2["image_tokens"][0] == feats.num_tokens
    assert out2["media"]["encoded"] - 1 == 2 and out2["media"]["shared"] == 2     # (one clip was encoded by image-qa above)
    assert out2["media"]["resident"] == 2 and entry.ctxm.counters["dedup_pages"] - before >= feats.num_tokens // 16
    assert entry.media.stats()["resident"] == 0


def test_fork_keeps_the_clip_and_eviction_replays_it(eng):
    e, cfg, w, enc, drv = eng
    from pie_b200.sdk import Context, Model, Sampler, media

    async def prog(args):
        model = Model.load("vlm")
        im = media.Image.from_bytes(png_bytes(4), min_pixels=28 * 28, max_pixels=28 * 28 * 12)
        ctx = Context(model)
        ctx.append([10, 11]).append_image(im).append([12])
        await ctx.flush()
        child = ctx.fork()
        ctx.release()                                   # the child still holds the clip
        assert model._entry.media.stats()["resident"] == 1
        child.suspend()                                 # KV goes away; the lineage (placeholders included) is replayed
        toks = await child.append([13]).generate(Sampler.argmax(), max_tokens=4).collect_tokens()
        child.release()
        return json.dumps({"tokens": toks, "image_tokens": im.num_tokens})
    e.register_program("fork-evict", prog)
    out = json.loads(e.run("fork-evict", {}, 300))
    feats = mm.patchify([mm.decode_image(png_bytes(4))], min_pixels=28 * 28, max_pixels=28 * 28 * 12)
    assert out["tokens"] == oracle(cfg, w, enc, feats, [10, 11], [12, 13], 4)
    e.models["vlm"].media.drain()
    assert e.models["vlm"].media.stats()["resident"] == 0 and drv.media == {}


def test_video_clip_and_text_only_models(eng):
    e, cfg, w, enc, drv = eng
    out = json.loads(e.run("video-qa", {"video_b64": base64.b64encode(gif_bytes(4)).decode(), "max_tokens": 3,
                                        "resize": dict(min_pixels=28 * 28, max_pixels=28 * 28 * 4)}, 300))
    assert out["ok"] and out["grid"][0] == 2 and len(out["tokens"]) == 3
    # a driver without an encoder declares nothing; the SDK refuses, the driver rejects spans it cannot serve
    plain = TorchDriver(cfg, "cpu", weights=w, num_pages=8, page_size=16, max_requests=2, max_tokens=32)
    assert plain.capabilities().media == ()
    with pytest.raises(ValueError, match="no encoder"):
        plain.put_media(0, "image", np.zeros((4, 1176), np.float32), [(1, 2, 2)])
    req = fold([PendingRequest(0, media_tokens(0, 4), [0, 1, 2, 3], [0], 0, [])], 16)
    with pytest.raises(ValueError, match="no such encoded clip"):
        plain.fire_batch(req)
    assert MEDIA_TOKEN_BASE > cfg.vocab_size


def test_media_crosses_the_driver_channel(eng):
    from pie_b200.driver.channel import ChannelDriver, InProcChannel
    e, cfg, w, enc, drv = eng
    ch = ChannelDriver(InProcChannel(drv))
    try:
        feats = mm.patchify([mm.decode_image(png_bytes(5))], min_pixels=28 * 28, max_pixels=28 * 28 * 4)
        n = ch.put_media(7, "image", feats.patches, [feats.grid])
        assert n == feats.num_tokens and 7 in drv.media and tuple(ch.capabilities().media) == ("image", "video")
        # patch rows travel as float16: the stored rows match the direct path to that rounding
        direct = enc(feats.patches.astype(np.float16).astype(np.float32), [feats.grid])
        assert (drv.media[7] - direct).abs().max() < 1e-5
        ch.release_media(7)
        assert 7 not in drv.media
    finally:
        ch.channel.close()


def test_registry_encodes_off_thread_shares_by_content_and_reports_errors():
    import threading
    import time
    from pie_b200.runtime.media import MediaRegistry

    class FakeDriver:
        def __init__(self):
            self.gate, self.held, self.calls = threading.Event(), {}, []

        def put_media(self, slot, kind, patches, grids):
            self.gate.wait(5)
            self.calls.append(("put", slot))
            if patches[0, 0] < 0:
                raise ValueError("bad clip")
            self.held[slot] = len(patches) // 4
            return len(patches) // 4

        def release_media(self, slot):
            self.calls.append(("release", slot))
            self.held.pop(slot, None)
    d = FakeDriver()
    reg = MediaRegistry([d])
    a = np.ones((8, 4), np.float32)
    t0 = time.monotonic()
    toks, e1 = reg.put(1, "image", a, [(1, 2, 4)], 2)
    assert time.monotonic() - t0 < 1.0 and not e1.ready.done()          # the caller did not wait for the encoder
    toks2, e2 = reg.put(2, "image", a.copy(), [(1, 2, 4)], 2)            # same content: same entry, same placeholders
    assert e2 is e1 and toks2 == toks and reg.stats()["encoded"] == 1 and reg.stats()["shared"] == 1
    reg.drop(1)
    assert reg.stats()["resident"] == 1                                  # context 2 still holds it
    d.gate.set()
    assert e1.ready.result(5) is True and d.held == {e1.slot: 2}
    reg.drop(2)
    reg.drain()
    assert d.held == {} and reg.stats()["resident"] == 0 and ("release", e1.slot) in d.calls
    # the freed slot is taken again; an encoder error reaches whoever waits, and a wrong row count is an error too
    _, bad = reg.put(3, "image", -a, [(1, 2, 4)], 2)
    with pytest.raises(ValueError, match="bad clip"):
        bad.ready.result(5)
    _, again = reg.put(4, "image", -a, [(1, 2, 4)], 2)           # a failed clip is not remembered: the same content is tried again
    assert again is not bad and again.slot != bad.slot
    with pytest.raises(ValueError, match="bad clip"):
        again.ready.result(5)
    reg.drop(4)
    _, short = reg.put(3, "image", a * 2, [(1, 2, 4)], 3)
    with pytest.raises(RuntimeError, match="planned with 3"):
        short.ready.result(5)
    with pytest.raises(ValueError, match="outside the placeholder range"):
        reg.put(3, "image", a, [(1, 2, 4)], 0)
    reg.drop(3)
    reg.drain()
    assert reg.stats()["resident"] == 0
    reg.close()


def wav_bytes_of(seconds: float, freq: float, sr: int = 8000) -> bytes:
    t = np.arange(int(seconds * sr)) / sr
    return mm.encode_wav((0.5 * np.sin(2 * np.pi * freq * t)).astype(np.float32), sr)


def test_audio_tower_equals_transformers_qwen2_audio():
    from transformers.models.qwen2_audio import modeling_qwen2_audio as m
    from transformers.models.qwen2_audio.configuration_qwen2_audio import Qwen2AudioEncoderConfig
    from pie_b200.models.audio import AudioEncoder, audio_preset, audio_rows, random_audio_weights
    cfg = audio_preset("tiny-audio", num_mel_bins=16, max_source_positions=50, hidden_size=96)
    w = random_audio_weights(cfg, seed=2)
    c = Qwen2AudioEncoderConfig(num_mel_bins=16, encoder_layers=cfg.layers, encoder_attention_heads=cfg.heads,
                                encoder_ffn_dim=cfg.ffn_dim, d_model=cfg.d_model, max_source_positions=50)
    c._attn_implementation = "eager"
    tower = m.Qwen2AudioEncoder(c).float().eval()
    tower.load_state_dict({k: v for k, v in w.items() if not k.startswith("projector.")}, strict=True)
    mel = torch.randn(16, 100)                       # the full window of this tower: 2 * max_source_positions frames
    with torch.no_grad():
        want = tower(mel[None]).last_hidden_state[0] @ w["projector.linear.weight"].t() + w["projector.linear.bias"]
    got = AudioEncoder(cfg, w)(mel)
    assert got.shape == (audio_rows(100), 96) and (got - want).abs().max() < 1e-5
    assert AudioEncoder(cfg, w)(torch.randn(16, 37)).shape[0] == audio_rows(37) == 9       # shorter clips are not padded
    with pytest.raises(ValueError, match="longer than"):
        AudioEncoder(cfg, w)(torch.randn(16, 203))


def test_audio_clips_through_the_engine():
    from pie_b200.models.audio import AudioEncoder, audio_preset, random_audio_weights
    cfg = preset("tiny-llama")
    w = random_weights(cfg, "cpu", torch.float32, seed=3)
    acfg = audio_preset("tiny-audio", hidden_size=cfg.hidden_size)
    enc = AudioEncoder(acfg, random_audio_weights(acfg, seed=6))
    drv = TorchDriver(cfg, "cpu", weights=w, num_pages=64, page_size=16, max_requests=8, max_tokens=48, audio=enc)
    assert drv.capabilities().media == ("audio",)
    e = Engine(EngineConfig())
    try:
        e.add_model("alm", drv, tokenizer=ByteTokenizer(cfg.vocab_size))
        install_all(e)
        wav = wav_bytes_of(2.5, 440.0)
        q = "What do you hear?"
        out = json.loads(e.run("audio-qa", {"audio_b64": base64.b64encode(wav).decode(), "question": q, "max_tokens": 4,
                                            "temperature": 0.0}, 300))
        mel = mm.audio_features(wav)
        rows = enc(mel)
        assert out["ok"] and out["audio_tokens"] == rows.shape[0] > 48 and out["frames"] == mel.shape[1]
        toks = [0] * rows.shape[0] + ByteTokenizer(cfg.vocab_size).encode(q)
        emb = {i: rows[i] for i in range(rows.shape[0])}
        want = []
        for _ in range(4):
            want.append(int(dense_reference_forward(cfg, w, torch.tensor(toks), embeds=emb)[-1].argmax()))
            toks.append(want[-1])
        assert out["tokens"] == want
        b64 = lambda x: base64.b64encode(x).decode()
        two = json.loads(e.run("multi-audio-test", {"audios_b64": [b64(wav), b64(wav_bytes_of(1.0, 880.0)), b64(wav)], "max_tokens": 2}, 300))
        assert two["ok"] and two["audio_tokens"][0] == two["audio_tokens"][2] and two["media"]["resident"] == 2
        # an image on this model is refused by the SDK: the driver declares audio only
        out = json.loads(e.run("image-qa", {"image_b64": base64.b64encode(png_bytes(1)).decode()}, 60))
        assert not out["ok"] and "no image encoder" in out["error"]
    finally:
        e.shutdown()


def test_siglip_tower_and_gemma3_projector_equal_transformers():
    from transformers import Gemma3Config, Gemma3TextConfig
    from transformers.models.gemma3 import modeling_gemma3 as g
    from transformers.models.siglip import modeling_siglip as m
    from transformers.models.siglip.configuration_siglip import SiglipVisionConfig
    from pie_b200.models.vision import SiglipEncoder, random_siglip_weights, siglip_preset
    cfg = siglip_preset("tiny-siglip", hidden_size=96)
    w = random_siglip_weights(cfg, seed=3)
    vc = SiglipVisionConfig(hidden_size=cfg.embed_dim, intermediate_size=cfg.intermediate_size, num_hidden_layers=cfg.depth,
                            num_attention_heads=cfg.num_heads, image_size=cfg.image_size, patch_size=cfg.patch_size, vision_use_head=False)
    vc._attn_implementation = "eager"
    tower = m.SiglipVisionModel(vc).float().eval()
    sd = {"vision_model." + k: v for k, v in w.items() if not k.startswith("projector.")}
    sd["vision_model.embeddings.patch_embedding.weight"] = sd["vision_model.embeddings.patch_embedding.weight"].reshape(cfg.embed_dim, 3, 14, 14)
    tower.load_state_dict(sd, strict=True)
    gc = Gemma3Config(text_config=Gemma3TextConfig(hidden_size=96, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1,
                                                   head_dim=16, intermediate_size=64, vocab_size=100).to_dict(),
                      vision_config=vc.to_dict(), mm_tokens_per_image=cfg.mm_tokens_per_image)
    proj = g.Gemma3MultiModalProjector(gc).float().eval()
    proj.load_state_dict({"mm_input_projection_weight": w["projector.mm_input_projection_weight"],
                          "mm_soft_emb_norm.weight": w["projector.mm_soft_emb_norm.weight"] - 1})
    # the host's own preprocessing on two real images: pixel tensors for transformers, patch rows for the encoder
    frames = [mm.decode_image(png_bytes(1, 80, 130)), mm.decode_image(png_bytes(2, 200, 90))]
    feats = mm.patchify_fixed(frames, image_size=cfg.image_size, patch=cfg.patch_size, pool=cfg.pool)
    assert feats.grid == (2, cfg.side, cfg.side) and feats.num_tokens == 2 * cfg.mm_tokens_per_image
    pix = torch.from_numpy(feats.patches).reshape(2, cfg.side, cfg.side, 3, 14, 14).permute(0, 3, 1, 4, 2, 5).reshape(2, 3, 112, 112)
    assert float(pix.min()) >= -1.0 and float(pix.max()) <= 1.0
    with torch.no_grad():
        want = proj(tower(pixel_values=pix).last_hidden_state).reshape(-1, 96)
    got = SiglipEncoder(cfg, w)(feats.patches, [(1, cfg.side, cfg.side)] * 2)
    assert got.shape == want.shape == (32, 96) and (got - want).abs().max() < 1e-5


def test_gemma3_with_a_siglip_tower_answers_over_an_image():
    from pie_b200.models.vision import SiglipEncoder, random_siglip_weights, siglip_preset
    cfg = preset("tiny-gemma3")
    w = random_weights(cfg, "cpu", torch.float32, seed=3)
    scfg = siglip_preset("tiny-siglip", hidden_size=cfg.hidden_size)
    enc = SiglipEncoder(scfg, random_siglip_weights(scfg, seed=8))
    drv = TorchDriver(cfg, "cpu", weights=w, num_pages=64, page_size=16, max_requests=8, max_tokens=48, vision=enc)
    spec = drv.capabilities().media_spec
    assert spec == {"style": "siglip", "image_size": 112, "patch": 14, "pool": 2, "bidirectional": True}
    e = Engine(EngineConfig())
    try:
        e.add_model("gemma-vlm", drv, tokenizer=ByteTokenizer(cfg.vocab_size))
        install_all(e)
        data = png_bytes(3, 300, 200)
        q = "Describe."
        out = json.loads(e.run("image-qa", {"image_b64": base64.b64encode(data).decode(), "question": q, "max_tokens": 4,
                                            "temperature": 0.0}, 300))
        # the inferlet asked for the model's own preprocessing: one 112 x 112 image, 16 soft tokens
        feats = mm.patchify_fixed([mm.decode_image(data)], image_size=112, patch=14, pool=2)
        assert out["ok"] and out["image_tokens"] == 16 and out["grid"] == [1, 8, 8]
        rows = enc(feats.patches, [(1, 8, 8)])
        toks = [0] * 16 + ByteTokenizer(cfg.vocab_size).encode(q)
        emb = {i: rows[i] for i in range(16)}          # image rows are not scaled by the embedding factor
        want = []
        for _ in range(4):
            want.append(int(dense_reference_forward(cfg, w, torch.tensor(toks), embeds=emb, spans=[(0, 16)])[-1].argmax()))
            toks.append(want[-1])
        assert out["tokens"] == want
        # a clip of several frames is a batch of images for this tower
        vid = json.loads(e.run("video-qa", {"video_b64": base64.b64encode(gif_bytes(3)).decode(), "max_tokens": 2}, 300))
        assert vid["ok"] and vid["video_tokens"] == 3 * 16
    finally:
        e.shutdown()


def test_gemma3_multimodal_equals_transformers_end_to_end(tmp_path):
    """A whole Gemma-3 vision-language model (SigLIP tower, pooling projector, Gemma-3 text with local / global layers)
    assembled in transformers from this build's weights: text + image + text through the engine - preprocessing,
    encoder on the driver, placeholder rows, embedding override without the embedding factor, rows of the image attending
    to each other in both directions - gives transformers' next-token logits."""
    from transformers import Gemma3Config, Gemma3ForConditionalGeneration, Gemma3TextConfig
    from transformers.models.siglip.configuration_siglip import SiglipVisionConfig
    from pie_b200.models import loader
    from pie_b200.models.vision import SiglipEncoder, random_siglip_weights, siglip_preset
    from pie_b200.sdk import Context, Model, media, sample as sm
    cfg = preset("tiny-gemma3", sliding_window=64)
    w = random_weights(cfg, "cpu", torch.float32, seed=11)
    scfg = siglip_preset("tiny-siglip", hidden_size=cfg.hidden_size)
    sw = random_siglip_weights(scfg, seed=12)
    # transformers' model from the same tensors
    loader.export_hf_checkpoint(cfg, w, tmp_path)
    from safetensors.torch import load_file
    text_sd = load_file(str(tmp_path / "model.safetensors"))
    tcfg = json.loads((tmp_path / "config.json").read_text())
    tcfg.pop("model_type")
    vc = SiglipVisionConfig(hidden_size=scfg.embed_dim, intermediate_size=scfg.intermediate_size, num_hidden_layers=scfg.depth,
                            num_attention_heads=scfg.num_heads, image_size=scfg.image_size, patch_size=scfg.patch_size, vision_use_head=False)
    IMG = 31999
    gc = Gemma3Config(text_config=Gemma3TextConfig(**tcfg).to_dict(), vision_config=vc.to_dict(), mm_tokens_per_image=16,
                      image_token_index=IMG, boi_token_index=31998, eoi_token_index=31997)
    gc._attn_implementation = "eager"
    hf = Gemma3ForConditionalGeneration(gc).float().eval()
    sd = {}
    for k, v in text_sd.items():
        sd["model.language_model." + k[len("model."):]] = v
    sd["lm_head.weight"] = text_sd["model.embed_tokens.weight"]
    for k, v in sw.items():
        if k.startswith("projector."):
            name = k[len("projector."):]
            sd["model.multi_modal_projector." + name] = (v - 1) if name == "mm_soft_emb_norm.weight" else v
        else:
            sd["model.vision_tower.vision_model." + k] = v.reshape(scfg.embed_dim, 3, 14, 14) if k == "embeddings.patch_embedding.weight" else v
    missing, unexpected = hf.load_state_dict(sd, strict=False)
    assert not unexpected and all("rotary" in m or "inv_freq" in m for m in missing), (missing, unexpected)
    pre, post = [5, 6, 7], [40, 41, 42, 43]
    data = png_bytes(21, 90, 160)
    feats = mm.patchify_fixed([mm.decode_image(data)], image_size=112, patch=14, pool=2)
    pix = torch.from_numpy(feats.patches).reshape(1, 8, 8, 3, 14, 14).permute(0, 3, 1, 4, 2, 5).reshape(1, 3, 112, 112)
    ids = torch.tensor([pre + [IMG] * 16 + post])
    tt = torch.tensor([[0] * 3 + [1] * 16 + [0] * 4])
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=pix, token_type_ids=tt, attention_mask=torch.ones_like(ids)).logits[0, -1]

    enc = SiglipEncoder(scfg, sw)
    drv = TorchDriver(cfg, "cpu", weights=w, num_pages=64, page_size=16, max_requests=8, max_tokens=48, vision=enc)
    assert drv.capabilities().media_spec["bidirectional"]
    e = Engine(EngineConfig())
    try:
        e.add_model("g3", drv, tokenizer=ByteTokenizer(cfg.vocab_size))

        async def prog(args):
            model = Model.load("g3")
            ctx = Context(model)
            ctx.append(pre).append_image(media.Image.for_model(model, data)).append(post)
            await ctx.flush()                       # image rows run with their masks; nothing is left pending
            assert ctx.seq_len == 23
            # read the logits of the last row again through a one-token pass over a fork that re-feeds it
            probe = Context(model)
            probe.append(pre).append_image(media.Image.for_model(model, data)).append(post[:-1])
            await probe.flush()
            f = probe.forward().input([post[-1]])
            h = f.probe(0, sm.Logits())
            out = await f.execute()
            raw = out.logits(h)
            ctx.release()
            probe.release()
            return base64.b64encode(raw).decode()
        e.register_program("g3-probe", prog)
        got = np.frombuffer(base64.b64decode(e.run("g3-probe", {}, 300)), dtype=np.float32)
    finally:
        e.shutdown()
    assert np.abs(got - want.numpy()).max() < 2e-4 and int(got.argmax()) == int(want.argmax())
    # without the look-both-ways masks the answer differs: the masks were in force
    emb = {3 + i: enc(feats.patches, [(1, 8, 8)])[i] for i in range(16)}
    causal = dense_reference_forward(cfg, w, torch.tensor(pre + [0] * 16 + post), embeds=emb)[-1]
    assert (causal - want).abs().max() > 1e-3


def test_image_qa_bench_batch_mode_counts_tokens(eng):
    e, cfg, w, enc, drv = eng
    resize = dict(min_pixels=28 * 28, max_pixels=28 * 28 * 8)
    imgs = [base64.b64encode(png_bytes(s)).decode() for s in (31, 32, 31)]
    out = json.loads(e.run("image-qa-bench", {"images_b64": imgs, "questions": ["One?", "Two?"], "question": "Rest?", "max_tokens": 5,
                                              "temperature": 0.0, "resize": resize}, 300))
    assert out["ok"] and len(out["results"]) == 3
    tok = ByteTokenizer(cfg.vocab_size)
    for r, q in zip(out["results"], ["One?", "Two?", "Rest?"]):
        assert r["num_output_tokens"] == 5 and len(r["stamps"]) == 5
        assert r["num_prompt_tokens"] == r["num_image_tokens"] + len(tok.encode(q))
    e.models["vlm"].media.drain()
    assert e.models["vlm"].media.stats()["resident"] == 0 and e.models["vlm"].media.stats()["shared"] >= 1


def test_server_config_builds_a_multimodal_model(tmp_path):
    """`[model.driver] vision` / `audio` in the server configuration: the CPU driver comes up with both encoders, declares
    the media kinds and the preprocessing the tower wants, and answers image and audio programs through the embedded server."""
    from pie_b200.server.embed import Server
    toml = ('[auth]\nenabled = false\n[[model]]\nname = "mm"\npreset = "tiny-llama"\n'
            '[model.driver]\ntype = "cpu"\nvision = "tiny-vit"\naudio = "tiny-audio"\n')
    with Server.from_text(toml) as srv:
        entry = srv.engine.models["mm"]
        caps = entry.caps[0]
        assert tuple(caps.media) == ("image", "video", "audio") and caps.media_spec["style"] == "qwen"
        img = json.loads(srv.engine.run("image-qa", {"image_b64": base64.b64encode(png_bytes(41)).decode(), "max_tokens": 3,
                                                     "resize": dict(min_pixels=28 * 28, max_pixels=28 * 28 * 6)}, 300))
        assert img["ok"] and len(img["tokens"]) == 3
        st = srv.engine.model_status()["models"]["mm"]
        assert st["media_encoded"] == 1 and 'pie_b200_model_media_encoded{model="mm"} 1' in srv.engine.metrics_text()
        aud = json.loads(srv.engine.run("audio-qa", {"audio_b64": base64.b64encode(wav_bytes_of(0.6, 300.0)).decode(),
                                                     "max_tokens": 2}, 300))
        assert aud["ok"] and aud["audio_tokens"] > 0 and len(aud["tokens"]) == 2
    sig = ('[auth]\nenabled = false\n[[model]]\nname = "g"\npreset = "tiny-gemma3"\n[model.driver]\ntype = "cpu"\nvision = "tiny-siglip"\n')
    with Server.from_text(sig) as srv:
        assert srv.engine.models["g"].caps[0].media_spec == {"style": "siglip", "image_size": 112, "patch": 14, "pool": 2,
                                                             "bidirectional": True}


def test_wit_level_forward_pass_splices_an_image_and_an_audio_clip():
    """The contract-level API (`forward-pass.input-image` / `input-audio` with an anchor position): the pass carries
    ordinary tokens at the clip's positions, the host swaps in the clip's placeholders, waits for the encoders and the
    logits equal the SDK path's (same oracle)."""
    from pie_b200.models.audio import AudioEncoder, audio_preset, random_audio_weights
    cfg = preset("tiny-llama")
    w = random_weights(cfg, "cpu", torch.float32, seed=3)
    vcfg = vision_preset("tiny-vit", hidden_size=cfg.hidden_size)
    acfg = audio_preset("tiny-audio", hidden_size=cfg.hidden_size)
    venc, aenc = VisionEncoder(vcfg, random_vision_weights(vcfg, seed=5)), AudioEncoder(acfg, random_audio_weights(acfg, seed=6))
    drv = TorchDriver(cfg, "cpu", weights=w, num_pages=64, page_size=16, max_requests=8, max_tokens=128, vision=venc, audio=aenc)
    img, wav = png_bytes(51, 56, 84), wav_bytes_of(0.5, 500.0)

    async def prog(args):
        from pie_b200.sdk import wit
        m = wit.model.model.load(wit.runtime.models()[0])
        image = wit.media.image.from_bytes(m, img)
        clip = wit.media.audio.from_bytes(m, wav)
        ni, na = image.token_count(), clip.token_count()
        n = 2 + ni + 1 + na + 2
        ctx = wit.context.context.create(m)
        ctx.reserve_working_pages(-(-(n + 1) // ctx.tokens_per_page()))
        fp = wit.inference.forward_pass(m)
        fp.context(ctx)
        toks = [10, 11] + [0] * ni + [12] + [0] * na + [13, 14]
        fp.input_tokens(toks, list(range(n)))
        fp.input_image(image, 2)
        fp.input_audio(clip, 2 + ni + 1)
        fp.sampler([n - 1], "raw-logits")
        fut = fp.execute()
        await fut.pollable().block()
        out = fut.get()
        bad = wit.inference.forward_pass(m)
        bad.context(ctx)
        bad.input_tokens([1, 2], [n, n + 1])
        bad.input_image(image, n)            # the pass does not carry the clip's rows
        try:
            bad.execute()
            err = ""
        except wit.WitError as e:
            err = str(e)
        ctx.destroy()
        return json.dumps({"ni": ni, "na": na, "logits": base64.b64encode(out["slots"][0][1]).decode(), "err": err})
    e = Engine(EngineConfig())
    try:
        e.add_model("mm", drv, tokenizer=ByteTokenizer(cfg.vocab_size))
        e.register_program("wit-media", prog)
        out = json.loads(e.run("wit-media", {}, 300))
    finally:
        e.shutdown()
    feats = mm.patchify([mm.decode_image(img)])
    vrows, arows = venc(feats.patches, [feats.grid]), aenc(mm.audio_features(wav))
    ni, na = out["ni"], out["na"]
    assert (ni, na) == (vrows.shape[0], arows.shape[0]) and "consecutive positions" in out["err"]
    toks = [10, 11] + [0] * ni + [12] + [0] * na + [13, 14]
    emb = {2 + i: vrows[i] for i in range(ni)}
    emb.update({2 + ni + 1 + i: arows[i] for i in range(na)})
    want = dense_reference_forward(cfg, w, torch.tensor(toks), embeds=emb)[-1].numpy()
    got = np.frombuffer(base64.b64decode(out["logits"]), dtype=np.float32)
    assert np.abs(got - want).max() < 1e-4


def test_a_saved_context_keeps_its_clip_for_the_next_program(eng):
    e, cfg, w, enc, drv = eng
    from pie_b200.sdk import Context, Model, Sampler, media
    data = png_bytes(61)
    resize = dict(min_pixels=28 * 28, max_pixels=28 * 28 * 6)

    async def writer(args):
        model = Model.load("vlm")
        ctx = Context(model)
        ctx.append([3, 4]).append_image(media.Image.for_model(model, data, **resize)).append([5])
        await ctx.flush()
        ctx.save("with-image")
        ctx.release()
        return "saved"

    async def reader(args):
        model = Model.load("vlm")
        ctx = Context.open(model, "with-image")
        toks = await ctx.append([6]).generate(Sampler.argmax(), max_tokens=3).collect_tokens()
        ctx.release()
        if args.get("delete"):
            Context.delete(model, "with-image")
        return json.dumps(toks)
    e.register_program("mm-writer", writer)
    e.register_program("mm-reader", reader)
    assert e.run("mm-writer", {}, 120) == "saved"
    reg = e.models["vlm"].media
    reg.drain()
    assert reg.stats()["resident"] == 1 and len(drv.media) == 1      # the writer is gone, the snapshot holds the clip
    feats = mm.patchify([mm.decode_image(data)], **resize)
    want = oracle(cfg, w, enc, feats, [3, 4], [5, 6], 3)
    assert json.loads(e.run("mm-reader", {}, 120)) == want
    assert json.loads(e.run("mm-reader", {"delete": True}, 120)) == want      # opened twice: the snapshot is not consumed
    reg.drain()
    assert reg.stats()["resident"] == 0 and drv.media == {}


def test_span_markers_of_the_model_go_around_a_clip():
    cfg = preset("tiny-llama")
    w = random_weights(cfg, "cpu", torch.float32, seed=3)
    vcfg = vision_preset("tiny-vit", hidden_size=cfg.hidden_size)
    enc = VisionEncoder(vcfg, random_vision_weights(vcfg, seed=5))
    enc.delimiters = ("<img>", "</img>")
    drv = TorchDriver(cfg, "cpu", weights=w, num_pages=64, page_size=16, max_requests=8, max_tokens=128, vision=enc)
    assert drv.capabilities().media_spec["delimiters"] == {"image": ["<img>", "</img>"], "video": ["<img>", "</img>"]}
    tok = ByteTokenizer(cfg.vocab_size)

    async def prog(args):
        from pie_b200.sdk import Context, Model, media, wit
        model = Model.load("vlm")
        im = media.Image.for_model(model, png_bytes(71), min_pixels=28 * 28, max_pixels=28 * 28 * 4)
        ctx = Context(model)
        ctx.append([9]).append_image(im)
        buf = list(ctx.buffer)
        ctx.release()
        wm = wit.model.model.load("vlm")
        wi = wit.media.image.from_bytes(wm, png_bytes(71))
        return json.dumps({"buf": buf, "n": im.num_tokens, "pre": wi.prefix_tokens(), "suf": wi.suffix_tokens()})
    e = Engine(EngineConfig())
    try:
        e.add_model("vlm", drv, tokenizer=tok)
        e.register_program("marks", prog)
        out = json.loads(e.run("marks", {}, 120))
    finally:
        e.shutdown()
    pre, suf, n = tok.encode("<img>"), tok.encode("</img>"), out["n"]
    assert out["buf"][:1 + len(pre)] == [9] + pre and out["buf"][-len(suf):] == suf
    assert len(out["buf"]) == 1 + len(pre) + n + len(suf) and all(t >= MEDIA_TOKEN_BASE for t in out["buf"][1 + len(pre):-len(suf)])
    assert out["pre"] == pre and out["suf"] == suf


def test_server_loads_a_gemma3_vision_language_checkpoint(tmp_path):
    """A Gemma-3 vision-language checkpoint as transformers writes it (nested configuration, `model.language_model.*`,
    `model.vision_tower.*`, `model.multi_modal_projector.*`): `pie serve` with `vision = "checkpoint"` loads all three parts
    and the engine's logits over text + image + text equal transformers'."""
    from transformers import Gemma3Config, Gemma3ForConditionalGeneration, Gemma3TextConfig
    from transformers.models.siglip.configuration_siglip import SiglipVisionConfig
    from pie_b200.sdk import Context, Model, media, sample as sm
    from pie_b200.server.embed import Server
    torch.manual_seed(0)
    tcfg = Gemma3TextConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                            head_dim=64, vocab_size=2048, sliding_window=64, query_pre_attn_scalar=64,
                            layer_types=["sliding_attention", "sliding_attention", "full_attention"], max_position_embeddings=512)
    vc = SiglipVisionConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, image_size=112,
                            patch_size=14, vision_use_head=False)
    IMG = 2047
    gc = Gemma3Config(text_config=tcfg.to_dict(), vision_config=vc.to_dict(), mm_tokens_per_image=16, image_token_index=IMG,
                      boi_token_index=2046, eoi_token_index=2045)
    gc._attn_implementation = "eager"
    hf = Gemma3ForConditionalGeneration(gc).float().eval()
    for p in hf.parameters():           # norm gains away from zero so that a missed (w + 1) would show
        if p.dim() == 1:
            torch.nn.init.normal_(p, 0.0, 0.1)
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    pre, post = [5, 6, 7], [40, 41, 42, 43]
    data = png_bytes(81, 70, 120)
    feats = mm.patchify_fixed([mm.decode_image(data)], image_size=112, patch=14, pool=2)
    pix = torch.from_numpy(feats.patches).reshape(1, 8, 8, 3, 14, 14).permute(0, 3, 1, 4, 2, 5).reshape(1, 3, 112, 112)

    toml = (f'[auth]\nenabled = false\n[[model]]\nname = "g3"\npath = "{tmp_path}"\n[model.driver]\ntype = "cpu"\nvision = "checkpoint"\n')
    with Server.from_text(toml) as srv:
        caps = srv.engine.models["g3"].caps[0]
        assert caps.arch_name == "gemma3_text" and caps.media_spec["style"] == "siglip" and caps.media_spec["pool"] == 2
        assert caps.media_spec["delimiters"]["image"] == ["\n\n<start_of_image>", "<end_of_image>\n\n"]

        async def prog(args):
            model = Model.load("g3")
            ctx = Context(model)
            ctx.append(pre).append_image(media.Image.for_model(model, data)).append(post[:-1])
            await ctx.flush()
            f = ctx.forward().input([post[-1]])
            h = f.probe(0, sm.Logits())
            raw = (await f.execute()).logits(h)
            ctx.release()
            tok = model.tokenizer()         # the server gave the model a byte-level tokenizer: the span markers are real tokens
            return json.dumps({"logits": base64.b64encode(raw).decode(), "before": tok.encode("\n\n<start_of_image>"),
                               "after": tok.encode("<end_of_image>\n\n")})
        srv.engine.register_program("probe", prog)
        out = json.loads(srv.engine.run("probe", {}, 300))
    got = np.frombuffer(base64.b64decode(out["logits"]), dtype=np.float32)
    m0, m1 = out["before"], out["after"]
    assert m0 and m1 and max(m0 + m1) < IMG
    ids = torch.tensor([pre + m0 + [IMG] * 16 + m1 + post])
    tt = torch.tensor([[0] * (3 + len(m0)) + [1] * 16 + [0] * (len(m1) + 4)])
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=pix, token_type_ids=tt, attention_mask=torch.ones_like(ids)).logits[0, -1].numpy()
    assert np.abs(got - want).max() < 2e-4 and int(got.argmax()) == int(want.argmax())


def test_server_loads_a_qwen2_vl_checkpoint(tmp_path):
    """A Qwen2-VL checkpoint as transformers writes it: the language model loads as the Qwen2 block (text-only logits equal
    transformers': with equal components the three-axis rotary positions are the ordinary ones), the `visual.*` tower loads
    next to it and its rows equal transformers' image features; the clip's span markers come from the family."""
    from transformers import Qwen2VLConfig, Qwen2VLForConditionalGeneration
    from pie_b200.server.embed import Server
    torch.manual_seed(1)
    c = Qwen2VLConfig(text_config=dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                                       num_key_value_heads=2, vocab_size=2048, max_position_embeddings=512,
                                       rope_parameters={"rope_type": "default", "mrope_section": [4, 6, 6], "rope_theta": 10000.0}),
                      vision_config=dict(depth=2, embed_dim=64, hidden_size=128, num_heads=4, mlp_ratio=2, patch_size=14,
                                         spatial_merge_size=2, temporal_patch_size=2, in_channels=3))
    c._attn_implementation = "eager"
    hf = Qwen2VLForConditionalGeneration(c).float().eval()
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    toks = list(range(30, 60))
    feats = mm.patchify([mm.decode_image(png_bytes(91))], min_pixels=28 * 28, max_pixels=28 * 28 * 6)
    with torch.no_grad():
        want = hf(input_ids=torch.tensor([toks])).logits[0, -1].numpy()
        rows = hf.get_image_features(torch.from_numpy(feats.patches), torch.tensor([feats.grid]))
    rows = rows if torch.is_tensor(rows) else (rows.pooler_output if hasattr(rows, "pooler_output") else rows[0])
    rows = torch.cat(list(rows)) if isinstance(rows, (list, tuple)) else rows
    toml = f'[auth]\nenabled = false\n[[model]]\nname = "q"\npath = "{tmp_path}"\n[model.driver]\ntype = "cpu"\nvision = "checkpoint"\n'
    with Server.from_text(toml) as srv:
        entry = srv.engine.models["q"]
        caps = entry.caps[0]
        assert caps.arch_name == "qwen2" and caps.media_spec["style"] == "qwen" and tuple(caps.media) == ("image", "video")
        assert caps.media_spec["delimiters"]["image"] == ["<|vision_start|>", "<|vision_end|>"]
        drv = entry.drivers[0]
        assert drv.put_media(3, "image", feats.patches, [feats.grid]) == feats.num_tokens
        assert (drv.media[3] - rows.reshape(-1, 128)).abs().max() < 1e-5
        drv.release_media(3)
        from pie_b200.driver.schema import SamplerKind, SamplerSpec
        req = fold([PendingRequest(0, toks, list(range(30)), [0, 1], 0, [(29, SamplerSpec(SamplerKind.RAW_LOGITS))])], 16)
        got = np.frombuffer(drv.fire_batch(req).slots[0].logits, dtype=np.float32)
    assert np.abs(got - want).max() < 2e-4


def test_server_loads_a_qwen2_audio_checkpoint(tmp_path):
    """A Qwen2-Audio checkpoint as transformers writes it (`language_model.*` with an untied head, `audio_tower.*`,
    `multi_modal_projector.*`): text logits equal transformers', the audio tower's projected rows equal transformers'."""
    from transformers import Qwen2AudioConfig, Qwen2AudioForConditionalGeneration
    from pie_b200.driver.schema import SamplerKind, SamplerSpec
    from pie_b200.server.embed import Server
    torch.manual_seed(2)
    c = Qwen2AudioConfig(text_config=dict(model_type="qwen2", hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                          num_attention_heads=4, num_key_value_heads=2, vocab_size=2048, max_position_embeddings=512),
                         audio_config=dict(num_mel_bins=80, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=128, d_model=64,
                                           max_source_positions=50), audio_token_index=2047)
    c._attn_implementation = "eager"
    hf = Qwen2AudioForConditionalGeneration(c).float().eval()
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    toks = list(range(30, 60))
    mel = torch.randn(80, 100)
    with torch.no_grad():
        want = hf(input_ids=torch.tensor([toks])).logits[0, -1].numpy()
        rows = hf.multi_modal_projector(hf.audio_tower(mel[None]).last_hidden_state)[0]
    toml = f'[auth]\nenabled = false\n[[model]]\nname = "a"\npath = "{tmp_path}"\n[model.driver]\ntype = "cpu"\naudio = "checkpoint"\n'
    with Server.from_text(toml) as srv:
        entry = srv.engine.models["a"]
        caps, drv = entry.caps[0], entry.drivers[0]
        assert caps.arch_name == "qwen2" and tuple(caps.media) == ("audio",)
        assert caps.media_spec["delimiters"] == {"audio": ["<|audio_bos|>", "<|audio_eos|>"]}
        assert drv.put_media(0, "audio", mel.numpy(), [(100,)]) == 25
        assert (drv.media[0] - rows).abs().max() < 1e-5
        req = fold([PendingRequest(0, toks, list(range(30)), [0, 1], 0, [(29, SamplerSpec(SamplerKind.RAW_LOGITS))])], 16)
        got = np.frombuffer(drv.fire_batch(req).slots[0].logits, dtype=np.float32)
    assert np.abs(got - want).max() < 2e-4
