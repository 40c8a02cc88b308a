"""Structured (constrained) decoding: grammars from EBNF, regular expressions and JSON Schema,
compiled to the native byte-level pushdown matcher (csrc/host/grammar.hpp), and a token-level
`Matcher` that yields the BRLE vocabulary mask of the next step.

    g = Grammar.from_json_schema(schema)        # or .json(), .from_regex(...), .from_ebnf(...)
    m = Matcher(g, tokenizer)
    mask = m.next_token_logit_mask()            # BRLE over the vocabulary
    m.accept_tokens([tok])

EBNF dialect: `rule ::= a b | c`, "literals" with escapes, [classes] with ranges and ^ negation,
( groups ), postfix * + ? and {m,n}, `root` is the start rule. Compiled grammars are cached
(LRU 64) by source text. Counterpart of runtime/src/inference/structured.rs and structured/
{ebnf,json_schema,regex,matcher,compiled_grammar}.rs (the xgrammar-style engine of the reference).
"""
from __future__ import annotations

import json
from collections import OrderedDict
from typing import Dict, List, Optional, Sequence, Tuple


class GrammarError(ValueError):
    pass


# ------------------------------------------------------------------------------ IR builder
class _Builder:
    def __init__(self):
        self.rules: List[List[List[tuple]]] = []
        self.names: Dict[str, int] = {}

    def rule(self, name: Optional[str] = None) -> int:
        if name is not None and name in self.names:
            return self.names[name]
        self.rules.append([])
        rid = len(self.rules) - 1
        if name is not None:
            self.names[name] = rid
        return rid

    @staticmethod
    def cls(byte_set) -> tuple:
        bits = bytearray(32)
        for b in byte_set:
            bits[b >> 3] |= 1 << (b & 7)
        return (-1, bytes(bits))

    def literal(self, data: bytes) -> List[tuple]:
        return [self.cls([b]) for b in data]

    def star(self, item: List[tuple]) -> tuple:
        r = self.rule()
        self.rules[r] = [item + [(r, b"")], []]
        return (r, b"")

    def opt(self, item: List[tuple]) -> tuple:
        r = self.rule()
        self.rules[r] = [item, []]
        return (r, b"")

    def group(self, alts: List[List[tuple]]) -> tuple:
        r = self.rule()
        self.rules[r] = alts
        return (r, b"")

    def repeat(self, item: List[tuple], lo: int, hi: Optional[int]) -> List[tuple]:
        out = []
        for _ in range(lo):
            out += item
        if hi is None:
            out.append(self.star(item))
        else:
            tail: List[tuple] = []
            for _ in range(hi - lo):
                tail = [self.opt(item + tail)]
            out += tail
        return out


_ESC = {"n": 10, "t": 9, "r": 13, "\\": 92, '"': 34, "'": 39, "[": 91, "]": 93, "-": 45, "^": 94, "0": 0, "/": 47}


class _Ebnf:
    """Recursive-descent parser of the EBNF dialect into the IR."""

    def __init__(self, text: str, b: Optional[_Builder] = None):
        self.s, self.i, self.b = text, 0, b or _Builder()

    def err(self, msg):
        raise GrammarError(f"EBNF: {msg} at offset {self.i}")

    def ws(self, newlines=True):
        while self.i < len(self.s):
            c = self.s[self.i]
            if c == "#":
                while self.i < len(self.s) and self.s[self.i] != "\n":
                    self.i += 1
            elif c in " \t\r" or (newlines and c == "\n"):
                self.i += 1
            else:
                break

    def ident(self) -> str:
        j = self.i
        while j < len(self.s) and (self.s[j].isalnum() or self.s[j] in "_-."):
            j += 1
        if j == self.i:
            self.err("expected a rule name")
        name, self.i = self.s[self.i:j], j
        return name

    def parse(self) -> Tuple[List, int]:
        self.ws()
        defined = set()
        while self.i < len(self.s):
            name = self.ident()
            self.ws()
            if not self.s.startswith("::=", self.i):
                self.err("expected ::=")
            self.i += 3
            rid = self.b.rule(name)
            self.b.rules[rid] = self.alternatives()
            defined.add(name)
            self.ws()
        missing = [n for n in self.b.names if n not in defined]
        if missing:
            raise GrammarError(f"EBNF: undefined rule(s) {missing}")
        if "root" not in self.b.names:
            raise GrammarError("EBNF: no `root` rule")
        return self.b.rules, self.b.names["root"]

    def at_rule_start(self) -> bool:
        j = self.i
        while j < len(self.s) and (self.s[j].isalnum() or self.s[j] in "_-."):
            j += 1
        if j == self.i:
            return False
        while j < len(self.s) and self.s[j] in " \t":
            j += 1
        return self.s.startswith("::=", j)

    def alternatives(self) -> List[List[tuple]]:
        alts = [self.sequence()]
        while True:
            self.ws()
            if self.i < len(self.s) and self.s[self.i] == "|":
                self.i += 1
                alts.append(self.sequence())
            else:
                return alts

    def sequence(self) -> List[tuple]:
        seq: List[tuple] = []
        while True:
            self.ws()
            if self.i >= len(self.s) or self.s[self.i] in "|)" or self.at_rule_start():
                return seq
            item = self.atom()
            self.ws(newlines=False)
            while self.i < len(self.s) and self.s[self.i] in "*+?{":
                c = self.s[self.i]
                if c == "{":
                    j = self.s.index("}", self.i)
                    lo, _, hi = self.s[self.i + 1:j].partition(",")
                    item = self.b.repeat(item, int(lo), int(lo) if "," not in self.s[self.i:j] else (int(hi) if hi.strip() else None))
                    self.i = j + 1
                else:
                    self.i += 1
                    item = {"*": lambda it: [self.b.star(it)], "?": lambda it: [self.b.opt(it)],
                            "+": lambda it: it + [self.b.star(it)]}[c](item)
                self.ws(newlines=False)
            seq += item

    def char(self) -> int:
        c = self.s[self.i]
        if c == "\\":
            e = self.s[self.i + 1]
            if e == "x":
                v = int(self.s[self.i + 2:self.i + 4], 16)
                self.i += 4
                return v
            if e == "u":
                v = int(self.s[self.i + 2:self.i + 6], 16)
                self.i += 6
                return v
            self.i += 2
            return _ESC.get(e, ord(e))
        self.i += 1
        return ord(c)

    def atom(self) -> List[tuple]:
        c = self.s[self.i]
        if c == '"':
            self.i += 1
            data = bytearray()
            while self.s[self.i] != '"':
                data += chr(self.char()).encode("utf-8")
            self.i += 1
            return self.b.literal(bytes(data))
        if c == "[":
            self.i += 1
            neg = self.s[self.i] == "^"
            self.i += neg
            members, wide = set(), False
            while self.s[self.i] != "]":
                lo = self.char()
                hi = lo
                if self.s[self.i] == "-" and self.s[self.i + 1] != "]":
                    self.i += 1
                    hi = self.char()
                if hi > 127:
                    wide = True
                members.update(range(lo, min(hi, 127) + 1))
            self.i += 1
            if neg:
                return [self.b.cls([x for x in range(256) if x not in members])]   # any non-ASCII byte passes
            if wide:
                members.update(range(128, 256))
            return [self.b.cls(members)]
        if c == "(":
            self.i += 1
            alts = self.alternatives()
            self.ws()
            if self.s[self.i] != ")":
                self.err("expected )")
            self.i += 1
            return [self.b.group(alts)]
        if c == ".":
            self.i += 1
            return [self.b.cls(range(256))]
        return [(self.b.rule(self.ident()), b"")]


# ------------------------------------------------------------------------------ regex -> EBNF
def regex_to_ebnf(pattern: str) -> str:
    """Translate a regular expression (literals, ., classes, \\d \\w \\s, groups, |, * + ? {m,n})
    into the EBNF dialect; anchors are ignored (the whole output must match)."""
    out, i, n = [], 0, len(pattern)
    cls = {"d": "[0-9]", "w": "[a-zA-Z0-9_]", "s": "[ \\t\\n\\r]", "D": "[^0-9]", "W": "[^a-zA-Z0-9_]", "S": "[^ \\t\\n\\r]"}
    while i < n:
        c = pattern[i]
        if c == "\\":
            e = pattern[i + 1]
            out.append(cls[e] if e in cls else '"' + ("\\\\" if e == "\\" else '\\"' if e == '"' else
                                                       {"n": "\\n", "t": "\\t", "r": "\\r"}.get(e, e)) + '"')
            i += 2
        elif c == "[":
            j = i + 1
            if pattern[j] == "^":
                j += 1
            if pattern[j] == "]":
                j += 1
            while pattern[j] != "]":
                j += 2 if pattern[j] == "\\" else 1
            body = pattern[i:j + 1]
            for k, v in cls.items():
                body = body.replace("\\" + k, v[1:-1])
            out.append(body)
            i = j + 1
        elif c in "()|*+?":
            out.append(c)
            i += 1
        elif c == "{":
            j = pattern.index("}", i)
            out.append(pattern[i:j + 1])
            i = j + 1
        elif c in "^$":
            i += 1
        elif c == ".":
            out.append("[^\\n]")
            i += 1
        else:
            out.append('"' + ('\\"' if c == '"' else c) + '"')
            i += 1
        out.append(" ")
    return "root ::= " + "".join(out)


# ------------------------------------------------------------------------------ JSON schema -> EBNF
JSON_RULES = r'''
value ::= object | array | string | number | "true" | "false" | "null"
object ::= "{" ws ( pair ( ws "," ws pair )* )? ws "}"
pair ::= string ws ":" ws value
array ::= "[" ws ( value ( ws "," ws value )* )? ws "]"
string ::= "\"" char* "\""
char ::= [^"\\\x00-\x1f] | "\\" ( ["\\/bfnrt] | "u" hex hex hex hex )
hex ::= [0-9a-fA-F]
number ::= integer ( "." [0-9]{1,18} )? ( [eE] [+-]? [0-9]{1,3} )?
integer ::= "-"? ( "0" | [1-9] [0-9]{0,17} )
boolean ::= "true" | "false"
ws ::= [ \t\n]{0,2}
'''


def _lit(s: str) -> str:
    return '"' + s.replace("\\", "\\\\").replace('"', '\\"').replace("\n", "\\n") + '"'


def json_schema_to_ebnf(schema) -> str:
    root, rules = json_schema_rules(schema, "s")
    return f"root ::= {root}\n" + rules + JSON_RULES


def json_schema_rules(schema, prefix: str = "s"):
    """(name of the rule that matches `schema`, text of the rules it needs) with rule names
    `<prefix>0`, `<prefix>1`, ...; the shared JSON rules (value, string, ws, ...) are not included."""
    if isinstance(schema, str):
        schema = json.loads(schema)
    rules: List[str] = []
    defs = {**schema.get("definitions", {}), **schema.get("$defs", {})}
    memo: Dict[str, str] = {}

    def new(body: str) -> str:
        idx = len(rules)
        name = f"{prefix}{idx}"
        rules.append(f"{name} ::= {body}")
        return name

    def visit(s) -> str:
        if s is True or s == {}:
            return "value"
        if "$ref" in s:
            key = s["$ref"].split("/")[-1]
            if key not in memo:
                idx = len(rules)
                memo[key] = f"{prefix}{idx}"
                rules.append(None)
                body = visit(defs[key])
                rules[idx] = f"{memo[key]} ::= {body}"
            return memo[key]
        if "const" in s:
            return new(_lit(json.dumps(s["const"])))
        if "enum" in s:
            return new(" | ".join(_lit(json.dumps(v)) for v in s["enum"]))
        for k in ("anyOf", "oneOf"):
            if k in s:
                return new(" | ".join(visit(x) for x in s[k]))
        t = s.get("type")
        if isinstance(t, list):
            return new(" | ".join(visit({**s, "type": x}) for x in t))
        if t == "object" or (t is None and "properties" in s):
            props = s.get("properties", {})
            req = set(s.get("required", list(props)))
            parts, first = [], True
            for name, sub in props.items():
                item = f'{_lit(json.dumps(name))} ws ":" ws {visit(sub)}'
                sep = "" if first else 'ws "," ws '
                if name in req:
                    parts.append(f"{sep}{item}")
                    first = False
                else:
                    parts.append(f"( {sep}{item} )?" if not first else f"( {item} ws \",\" ws )?")
            # optional leading members carry their own trailing comma; keep required members last-safe
            body = '"{" ws ' + " ".join(parts) + ' ws "}"' if parts else "object"
            return new(body)
        if t == "array":
            item = visit(s.get("items", True))
            lo, hi = s.get("minItems", 0), s.get("maxItems")
            if lo == 0 and hi is None:
                return new(f'"[" ws ( {item} ( ws "," ws {item} )* )? ws "]"')
            rest = f'( ws "," ws {item} )' + ("{" + f"{max(lo - 1, 0)},{'' if hi is None else hi - 1}" + "}")
            body = f'"[" ws {item} {rest} ws "]"'
            return new(body if lo > 0 else f'"[" ws ( {item} {rest} )? ws "]"')
        if t == "string":
            if "maxLength" in s or "minLength" in s:
                lo, hi = int(s.get("minLength", 0)), s.get("maxLength")
                return new('"\\"" char{' + f"{lo},{'' if hi is None else int(hi)}" + '} "\\""')
            if "pattern" in s:
                sub = regex_to_ebnf(s["pattern"])[len("root ::= "):]
                return new('"\\"" ( ' + sub + ' ) "\\""')
            return "string"
        if t == "integer":
            return "integer"
        if t == "number":
            return "number"
        if t == "boolean":
            return "boolean"
        if t == "null":
            return new('"null"')
        return "value"

    root = visit(schema)
    return root, "\n".join(r for r in rules if r) + "\n"


# ------------------------------------------------------------------------------ public objects
_CACHE: "OrderedDict[str, Grammar]" = OrderedDict()


def optimise_rules(rules: List[List[List[tuple]]], root: int, inline_limit: int = 12):
    """Shrink a grammar without changing its language: (1) a rule with one alternative that does not call itself is
    substituted where it is referenced when it is short or referenced once (the matcher then keeps one frame less on
    its stacks for every such level: literals and sequences that the front ends wrap in helper rules); (2) rules with
    identical bodies become one; (3) rules the root no longer reaches are dropped and the rest renumbered. Returns
    (rules, root). Counterpart of the grammar optimiser of the reference
    (runtime/src/inference/structured/optimizer.rs)."""
    rules = [[list(alt) for alt in r] for r in rules]
    for _ in range(8):
        changed = False
        refs: Dict[int, int] = {}
        for r in rules:
            for alt in r:
                for sym in alt:
                    if sym[0] >= 0:
                        refs[sym[0]] = refs.get(sym[0], 0) + 1
        inlinable = {i for i, r in enumerate(rules)
                     if i != root and len(r) == 1 and all(sym[0] != i for sym in r[0])
                     and (len(r[0]) <= inline_limit or refs.get(i, 0) <= 1)}
        # never substitute a rule into a body through a cycle of inlinable rules: take those that call no inlinable rule
        leaf = {i for i in inlinable if all(sym[0] not in inlinable for sym in rules[i][0])}
        if leaf:
            for r in rules:
                for k, alt in enumerate(r):
                    if any(sym[0] in leaf for sym in alt):
                        out: List[tuple] = []
                        for sym in alt:
                            out.extend(rules[sym[0]][0] if sym[0] in leaf else [sym])
                        r[k] = out
                        changed = True
        # identical bodies (compared by value; a self-reference keeps a rule apart from its twins)
        seen: Dict[tuple, int] = {}
        alias: Dict[int, int] = {}
        for i, r in enumerate(rules):
            if any(sym[0] == i for alt in r for sym in alt):
                continue
            key = tuple(tuple(alt) for alt in r)
            if key in seen and i != root:
                alias[i] = seen[key]
            else:
                seen.setdefault(key, i)
        if alias:
            for r in rules:
                for alt in r:
                    for j, sym in enumerate(alt):
                        if sym[0] in alias:
                            alt[j] = (alias[sym[0]], sym[1])
            changed = True
        if not changed:
            break
    # reachable rules, renumbered in first-visit order
    order: List[int] = []
    index: Dict[int, int] = {}
    stack = [root]
    while stack:
        i = stack.pop()
        if i in index:
            continue
        index[i] = len(order)
        order.append(i)
        for alt in rules[i]:
            for sym in reversed(alt):
                if sym[0] >= 0 and sym[0] not in index:
                    stack.append(sym[0])
    out_rules = [[[(index[sym[0]], sym[1]) if sym[0] >= 0 else sym for sym in alt] for alt in rules[i]] for i in order]
    return out_rules, index[root]


class Grammar:
    def __init__(self, ebnf: str, optimise: bool = True):
        from .._C import pie_host
        self.source = ebnf
        rules, root = _Ebnf(ebnf).parse()
        self.rules_parsed = len(rules)
        if optimise:
            rules, root = optimise_rules(rules, root)
        self.rules_compiled = len(rules)
        self.native = pie_host.Grammar(rules, root)

    @staticmethod
    def _cached(ebnf: str) -> "Grammar":
        g = _CACHE.get(ebnf)
        if g is None:
            g = Grammar(ebnf)
            _CACHE[ebnf] = g
            while len(_CACHE) > 64:
                _CACHE.popitem(last=False)
        else:
            _CACHE.move_to_end(ebnf)
        return g

    @staticmethod
    def from_ebnf(ebnf: str) -> "Grammar":
        return Grammar._cached(ebnf)

    @staticmethod
    def from_regex(pattern: str) -> "Grammar":
        return Grammar._cached(regex_to_ebnf(pattern))

    @staticmethod
    def from_json_schema(schema) -> "Grammar":
        return Grammar._cached(json_schema_to_ebnf(schema))

    @staticmethod
    def json() -> "Grammar":
        return Grammar._cached("root ::= value\n" + JSON_RULES)

    def to_string(self) -> str:
        return self.source


_TRIES: Dict[int, object] = {}


def _trie_for(tokenizer):
    from .._C import pie_host
    key = id(tokenizer)
    if key not in _TRIES:
        ids, toks = tokenizer.vocabs()
        _TRIES[key] = pie_host.TokenTrie(list(ids), [bytes(t) for t in toks])
    return _TRIES[key]


class Matcher:
    """Walks the grammar as tokens are accepted and produces the next-step vocabulary mask."""

    def __init__(self, grammar: Grammar, tokenizer, stop_tokens: Optional[Sequence[int]] = None):
        from .._C import pie_host
        self.grammar, self.tok = grammar, tokenizer
        self.native = pie_host.GrammarMatcher(grammar.native, _trie_for(tokenizer))
        self.vocab_size = int(getattr(tokenizer, "vocab_size", 0))
        self.stop_tokens = list(stop_tokens if stop_tokens is not None else getattr(tokenizer, "eos_tokens", []))
        self._stopped = False

    def _bytes(self, tid: int) -> bytes:
        if hasattr(self.tok, "token_bytes"):
            return self.tok.token_bytes(tid)
        return bytes([tid & 0xFF])

    def accept_tokens(self, token_ids: Sequence[int]) -> None:
        for t in token_ids:
            if t in self.stop_tokens:
                if not self.native.can_terminate():
                    raise GrammarError("stop token before the grammar completed")
                self._stopped = True
                continue
            if self._stopped or not self.native.accept_bytes(self._bytes(int(t))):
                raise GrammarError(f"token {t} violates the grammar")

    def next_token_logit_mask(self) -> List[int]:
        extra = self.stop_tokens if self.native.can_terminate() else []
        return list(self.native.next_token_mask_brle(self.vocab_size, list(extra)))

    def is_terminated(self) -> bool:
        return self._stopped or self.native.is_terminated()

    def rollback(self, n: int) -> bool:
        self._stopped = False
        return self.native.rollback(n)

    def reset(self) -> None:
        self._stopped = False
        self.native.reset()
