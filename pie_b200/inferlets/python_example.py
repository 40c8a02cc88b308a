"""python-example: the walk-through inferlet. Loads a model, fills a chat context, generates step by step and routes the
tokens through the chat decoder (printable text, stop at the template's end marker) and the reasoning decoder (what is
inside the think tags is streamed apart from the answer). On a model without a chat template the prompt is fed as text.
Counterpart of inferlets/python-example/main.py."""
from pie_b200.sdk import Context, Model, Sampler, chat, runtime, session

NAME = "python-example"


async def main(args):
    args = args or {}
    model = Model.load(args.get("model") or runtime.models()[0])
    question = args.get("prompt", "What is the capital of France? Tell me a joke.")
    ctx = Context(model)
    if model.instruct is not None:
        ctx.system("You are a helpful assistant.").user(question).cue()
        chat_dec, think = chat.decoder(model), chat.reasoning_decoder(model)
    else:
        ctx.append(model.tokenizer().encode(question))
        chat_dec = think = None
    answer, thoughts = "", ""
    gen = ctx.generate(Sampler.top_p(0.6, 0.95), max_tokens=int(args.get("max_tokens", 64)))
    async for step in gen:
        out = await step.execute()
        if chat_dec is None:
            piece = model.tokenizer().decode(out.tokens)
            session.send(piece)
            answer += piece
            continue
        done = False
        for ev in chat_dec.feed(out.tokens):
            if ev.kind == "done":
                done = True
                break
            for part in think.feed(ev.text):            # text deltas: reasoning and answer come apart here
                if part.kind == "thinking":
                    thoughts += part.text
                else:
                    session.send(part.text)
                    answer += part.text
        if done:
            break
    if think is not None:
        for part in think.flush():          # the tail the decoder held back in case it was the start of a tag
            if part.kind != "thinking":
                session.send(part.text)
                answer += part.text
    session.send("\n[done]")
    ctx.release()
    return answer
