"""Chat, reasoning and tool-use helpers for inferlets (WIT `pie:instruct/{chat,reasoning,tool-use}`):
stream decoders that turn generated text into events, the tool prompt / answer formatting of the
model's family, and the grammar that constrains a tool call.

    dec = chat.decoder(model)                 # events: delta / done
    tools_prompt = chat.equip(model, tools)   # text to put in the system turn
    g = chat.tool_call_constraint(model, tools)
    ctx.generate(sampler, constrain=g)

Counterpart of sdk/python/src/inferlet/{chat,reasoning,tools}.py.
"""
from __future__ import annotations

from typing import List, Sequence

from ..runtime.instruct import ChatDecoder, ReasoningDecoder, ToolDecoder
from .grammar import Ebnf


def _ins(model):
    ins = model.instruct
    if ins is None:
        raise RuntimeError(f"model {model.name} has no chat template")
    return ins


def decoder(model) -> ChatDecoder:
    return ChatDecoder(model.tokenizer()._t, _ins(model))


def reasoning_decoder(model) -> ReasoningDecoder:
    return ReasoningDecoder(_ins(model))


def tool_decoder(model) -> ToolDecoder:
    return ToolDecoder(_ins(model))


def equip(model, tools: Sequence[dict]) -> str:
    """System-prompt text that declares `tools` in the model family's format."""
    return _ins(model).equip(tools)


def answer(model, name: str, result: str) -> str:
    """Text of a tool-result turn."""
    return _ins(model).answer(name, result)


def tool_call_constraint(model, tools: Sequence[dict]) -> Ebnf:
    """Constraint that makes the model emit exactly one well-formed call of one of `tools`."""
    return Ebnf(_ins(model).tool_grammar(tools))


def parse_tool_calls(model, text: str) -> List[dict]:
    return [e.call for e in tool_decoder(model).feed(text) if e.kind == "tool_call"]
