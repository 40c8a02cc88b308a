"""multi-image-test: several images in one context, then the same images again in a second context.

Reports the soft-token count of every image and how the runtime shared work: a repeated image is encoded
once (same content, same media slot) and a repeated prefix of text + images commits to the same KV pages.
Counterpart of inferlets/multi-image-test/src/lib.rs.
"""
import base64
import json

from pie_b200.sdk import Context, Model, media, runtime

from .text_completion import make_sampler

NAME = "multi-image-test"


async def main(args):
    args = args or {}
    model = Model.load(args.get("model") or runtime.models()[0])
    if "image" not in media.supported(model):
        return json.dumps({"ok": False, "error": f"model {model.name} has no image encoder"})
    images = [media.Image.for_model(model, base64.b64decode(b), **(args.get("resize") or {})) for b in args.get("images_b64", [])]
    if not images:
        return json.dumps({"ok": False, "error": "images_b64 is empty"})
    sep = model.tokenizer().encode(args.get("separator", "\n"))
    outs, live = [], []
    for _ in range(int(args.get("rounds", 2))):
        ctx = Context(model)
        live.append(ctx)            # the clips stay encoded while a context that holds them lives
        for im in images:
            ctx.append_image(im).append(sep)
        ctx.append(model.tokenizer().encode(args.get("question", "Compare the images.")))
        outs.append(await ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 8))).collect_tokens())
    reg = model._entry.media.stats()
    for ctx in live:
        ctx.release()
    return json.dumps({"ok": True, "image_tokens": [im.num_tokens for im in images], "outputs": outs,
                       "same_output": all(o == outs[0] for o in outs), "media": reg})
