"""video-qa: answer a question about a short clip (an animated GIF / multi-frame image).

Frames are sampled evenly, grouped in temporal pairs and encoded by the model's vision tower like an image
with a time axis. Counterpart of inferlets/video-qa/src/lib.rs.
"""
import base64
import json

from pie_b200.sdk import Context, Model, media, runtime

from .text_completion import make_sampler

NAME = "video-qa"


async def main(args):
    args = args or {}
    model = Model.load(args.get("model") or runtime.models()[0])
    if "video" not in media.supported(model):
        return json.dumps({"ok": False, "error": f"model {model.name} has no video encoder"})
    clip = media.Video.for_model(model, base64.b64decode(args["video_b64"]), max_frames=int(args.get("max_frames", 8)),
                                  **(args.get("resize") or {}))
    ctx = Context(model)
    ctx.append_video(clip)
    ctx.append(model.tokenizer().encode(args.get("question", "What happens in this clip?")))
    tokens = await ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 32))).collect_tokens()
    ctx.release()
    return json.dumps({"ok": True, "video_tokens": clip.num_tokens, "grid": list(clip.features.grid), "tokens": tokens})
