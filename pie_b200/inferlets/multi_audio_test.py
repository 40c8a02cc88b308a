"""multi-audio-test: several audio clips interleaved with text in one context; the same clip appended twice is
encoded once. Counterpart of inferlets/multi-audio-test/src/lib.rs."""
import base64
import json

from pie_b200.sdk import Context, Model, media, runtime

from .text_completion import make_sampler

NAME = "multi-audio-test"


async def main(args):
    args = args or {}
    model = Model.load(args.get("model") or runtime.models()[0])
    if "audio" not in media.supported(model):
        return json.dumps({"ok": False, "error": f"model {model.name} has no audio encoder"})
    clips = [media.Audio.from_wav(base64.b64decode(b), n_mels=int(args.get("n_mels", 80))) for b in args.get("audios_b64", [])]
    if not clips:
        return json.dumps({"ok": False, "error": "audios_b64 is empty"})
    tok = model.tokenizer()
    ctx = Context(model)
    for i, c in enumerate(clips):
        ctx.append(tok.encode(f"Clip {i + 1}: ")).append_audio(c)
    ctx.append(tok.encode(args.get("question", "Which clip is louder?")))
    tokens = await ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 8))).collect_tokens()
    stats = model._entry.media.stats()
    ctx.release()
    return json.dumps({"ok": True, "audio_tokens": [c.num_tokens for c in clips], "tokens": tokens, "media": stats})
