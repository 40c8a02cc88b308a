"""Constrained decoding for inferlets: Grammar / Matcher handles, the Constraint protocol
(`step(accepted) -> BRLE mask`), GrammarConstraint, and the schema wrappers accepted by
`ctx.generate(..., constrain=...)`: JsonSchema, AnyJson, Regex, Ebnf. Any object with a
`build_constraint(model)` method plugs in the same way.
Counterpart of sdk/python/src/inferlet/grammar.py:45-300 and sdk/rust/inferlet/src/inference/structured.rs.
"""
from __future__ import annotations

import json
from typing import List, Sequence

from ..runtime import brle
from ..runtime.structured import Grammar, GrammarError, Matcher as _Matcher


class Matcher(_Matcher):
    """`Matcher(grammar, tokenizer)`; the tokenizer may be the SDK wrapper or the runtime object."""

    def __init__(self, grammar: Grammar, tokenizer, stop_tokens=None):
        super().__init__(grammar, getattr(tokenizer, "_t", tokenizer), stop_tokens)


class GrammarConstraint:
    def __init__(self, matcher: Matcher):
        self.matcher = matcher

    @classmethod
    def from_grammar(cls, grammar: Grammar, model) -> "GrammarConstraint":
        return cls(Matcher(grammar, model.tokenizer()))

    @classmethod
    def from_json_schema(cls, schema, model) -> "GrammarConstraint":
        return cls.from_grammar(Grammar.from_json_schema(schema), model)

    @classmethod
    def json(cls, model) -> "GrammarConstraint":
        return cls.from_grammar(Grammar.json(), model)

    @classmethod
    def from_regex(cls, pattern: str, model) -> "GrammarConstraint":
        return cls.from_grammar(Grammar.from_regex(pattern), model)

    @classmethod
    def from_ebnf(cls, ebnf: str, model) -> "GrammarConstraint":
        return cls.from_grammar(Grammar.from_ebnf(ebnf), model)

    def accept(self, tokens: Sequence[int]) -> None:
        self.matcher.accept_tokens(tokens)

    def step(self, accepted: Sequence[int]) -> List[int]:
        if accepted:
            self.matcher.accept_tokens(accepted)
        return self.matcher.next_token_logit_mask()

    def is_terminated(self) -> bool:
        return self.matcher.is_terminated()

    def rollback(self, n: int) -> bool:
        return self.matcher.rollback(n)


class StaticMaskConstraint:
    """The same vocabulary mask at every step (the `logit_mask=` argument of generate)."""

    def __init__(self, mask: Sequence[int]):
        self.mask = list(mask)

    def accept(self, tokens) -> None:
        pass

    def step(self, accepted) -> List[int]:
        return list(self.mask)


class JsonSchema:
    def __init__(self, schema):
        self.schema = schema if isinstance(schema, str) else json.dumps(schema)

    def build_constraint(self, model) -> GrammarConstraint:
        return GrammarConstraint.from_json_schema(self.schema, model)


class AnyJson:
    def build_constraint(self, model) -> GrammarConstraint:
        return GrammarConstraint.json(model)


class Regex:
    def __init__(self, pattern: str):
        self.pattern = pattern

    def build_constraint(self, model) -> GrammarConstraint:
        return GrammarConstraint.from_regex(self.pattern, model)


class Ebnf:
    def __init__(self, source: str):
        self.source = source

    def build_constraint(self, model) -> GrammarConstraint:
        return GrammarConstraint.from_ebnf(self.source, model)


def brle_and_many(masks: Sequence[Sequence[int]]) -> List[int]:
    out = list(masks[0])
    for m in masks[1:]:
        out = brle.logical_and(out, m)
    return out


__all__ = ["Grammar", "GrammarError", "Matcher", "GrammarConstraint", "StaticMaskConstraint", "JsonSchema",
           "AnyJson", "Regex", "Ebnf", "brle_and_many"]
