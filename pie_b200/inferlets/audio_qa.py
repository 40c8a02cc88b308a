"""audio-qa: answer a question about an audio clip (PCM WAV, any sample rate; mixed down and resampled to 16 kHz).

The clip becomes a log-mel spectrogram on the host, is encoded by the model's audio tower on the driver (one row per
40 ms) and spliced into the context before the question. Needs a model whose driver declares an audio encoder.
Counterpart of inferlets/audio-qa/src/lib.rs.
"""
import base64
import json

from pie_b200.sdk import Context, Model, media, runtime

from .text_completion import make_sampler

NAME = "audio-qa"


async def main(args):
    args = args or {}
    model = Model.load(args.get("model") or runtime.models()[0])
    if "audio" not in media.supported(model):
        return json.dumps({"ok": False, "error": f"model {model.name} has no audio encoder"})
    clip = media.Audio.from_wav(base64.b64decode(args["audio_b64"]), n_mels=int(args.get("n_mels", 80)))
    ctx = Context(model)
    ctx.append_audio(clip)
    ctx.append(model.tokenizer().encode(args.get("question", "What do you hear?")))
    tokens = await ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 32))).collect_tokens()
    ctx.release()
    return json.dumps({"ok": True, "audio_tokens": clip.num_tokens, "frames": int(clip.mel.shape[1]), "tokens": tokens})
