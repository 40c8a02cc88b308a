"""Inferlet SDK (native Python form of the WIT world `pie:inferlet/inferlet`).

    from pie_b200.sdk import Context, Model, Sampler, runtime

    async def main(input):
        model = Model.load(runtime.models()[0])
        ctx = Context(model)
        ctx.system("You are helpful.").user(input["prompt"]).cue()
        return await ctx.generate(Sampler.top_p(0.6, 0.95), max_tokens=64).collect_text()
"""
from .core import Context, Forward, GenStep, Generator, Model, Output, ProbeHandle, SampleHandle, Tokenizer
from .sample import Distribution, Entropy, Logits, Logprob, Logprobs, Sampler
from .spec import NGramSpeculator, Speculator
from .adapter import Adapter
from .grammar import AnyJson, Ebnf, Grammar, GrammarConstraint, JsonSchema, Matcher, Regex
from . import chat, io, mcp, media, messaging, runtime, scheduling, session

__all__ = ["Context", "Forward", "GenStep", "Generator", "Model", "Output", "ProbeHandle", "SampleHandle",
           "Tokenizer", "Distribution", "Entropy", "Logits", "Logprob", "Logprobs", "Sampler", "Speculator",
           "NGramSpeculator", "Adapter", "AnyJson", "Ebnf", "Grammar", "GrammarConstraint", "JsonSchema", "Matcher", "Regex",
           "chat", "io", "mcp", "media", "messaging", "runtime", "scheduling", "session"]
