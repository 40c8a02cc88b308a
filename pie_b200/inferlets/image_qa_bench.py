"""image-qa-bench: the benchmark sibling of image-qa. The image arrives as base64 in the input, so the timed path is
decode + resize + patch rows + vision encoder + prefill + decode, never a network fetch. Reports the prompt length
(text tokens + image rows, read from the context) and the output length, with per-token timestamps. Single mode:
`image_b64` + `question`; batch mode: `images_b64` / `questions` driven concurrently in one process. An optional
start gate (a session message) lets a harness release many instances at once.
Counterpart of inferlets/image-qa-bench/src/lib.rs."""
import asyncio
import base64
import json
import time

from pie_b200.sdk import Context, Model, media, runtime, session

from .text_completion import make_sampler

NAME = "image-qa-bench"


async def one(model, image_b64: str, question: str, args: dict) -> dict:
    t0 = time.perf_counter()
    image = media.Image.for_model(model, base64.b64decode(image_b64), **(args.get("resize") or {}))
    t_pre = time.perf_counter()
    ctx = Context(model)
    if model.instruct is not None:
        ctx.system(args.get("system", "You are a helpful visual assistant.")).user("Here is an image:")
    ctx.append_image(image)
    if model.instruct is not None:
        ctx.user(question).cue()
    else:
        ctx.append(model.tokenizer().encode(question))
    gen = ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 64)))
    if args.get("ignore_eos", True):
        gen.stop([])                    # every request uses its whole token budget
    stamps, n = [], 0
    async for step in gen:
        out = await step.execute()
        n += len(out.tokens)
        stamps.append(time.perf_counter())
    n_prompt = ctx.seq_len - n + (1 if n else 0)          # the last sampled token is pending, not in the context yet
    text = model.tokenizer().decode(list(gen._generated)) if args.get("return_text") else None
    ctx.release()
    return {"t0": t0, "t_preprocess": t_pre - t0, "stamps": stamps, "num_prompt_tokens": n_prompt, "num_image_tokens": image.num_tokens,
            "num_output_tokens": n, "text": text}


async def main(args):
    args = args or {}
    model = Model.load(args.get("model") or runtime.models()[0])
    if "image" not in media.supported(model):
        return json.dumps({"ok": False, "error": f"model {model.name} has no image encoder"})
    if args.get("gate"):
        await session.receive()
    images = args.get("images_b64") or [args.get("image_b64", "")]
    questions = args.get("questions") or []
    default_q = args.get("question", "What is in this image?")
    jobs = [one(model, im or args.get("image_b64", ""), questions[i] if i < len(questions) else default_q, args)
            for i, im in enumerate(images)]
    results = await asyncio.gather(*jobs)
    return json.dumps({"ok": True, "results": results})
