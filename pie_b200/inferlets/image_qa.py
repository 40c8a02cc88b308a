"""image-qa: answer a question about an image.

The image comes from `image_b64` (base64 of an encoded image file), `image_path` inside the process' scratch
directory, or `image_url` (fetched over HTTP, subject to the engine's network allow-list). It is decoded, resized
and cut into patches on the host, encoded by the model's vision tower on the driver, and spliced into the user
turn; generation is ordinary text generation. Needs a model whose driver declares an image encoder.
Counterpart of inferlets/image-qa/src/lib.rs.
"""
import base64
import json

from pie_b200.sdk import Context, Model, io, media, runtime

from .text_completion import make_sampler

NAME = "image-qa"


async def load_image_bytes(args: dict) -> bytes:
    if args.get("image_b64"):
        return base64.b64decode(args["image_b64"])
    if args.get("image_path"):
        return io.read_bytes(args["image_path"])
    r = await io.http_fetch(args.get("image_url", "http://127.0.0.1:8080/image.png"), timeout=float(args.get("timeout", 10)))
    return r.body


async def main(args):
    args = args or {}
    model = Model.load(args.get("model") or runtime.models()[0])
    if "image" not in media.supported(model):
        return json.dumps({"ok": False, "error": f"model {model.name} has no image encoder"})
    image = media.Image.for_model(model, await load_image_bytes(args), **(args.get("resize") or {}))
    ctx = Context(model)
    if model.instruct is not None:
        ctx.system(args.get("system", "You are a helpful visual assistant.")).user("Here is an image:")
    ctx.append_image(image)
    if model.instruct is not None:
        ctx.user(args.get("question", "What is in this image? Answer in one sentence.")).cue()
    else:
        ctx.append(model.tokenizer().encode(args.get("question", "What is in this image?")))
    gen = ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 64)))
    tokens = await gen.collect_tokens()
    ctx.release()
    return json.dumps({"ok": True, "image_tokens": image.num_tokens, "grid": list(image.features.grid), "tokens": tokens,
                       "text": model.tokenizer().decode(tokens)})
