"""Constrained decoding: grammar front ends (EBNF / regex / JSON schema), the native matcher's
token masks against Python's own `re` / `json`, rollback, and the path through the engine
(mask -> driver -> sampler) with the dummy driver and with the tiny CPU model."""
import json
import re

import numpy as np
import pytest
import torch

from pie_b200.runtime import brle
from pie_b200.runtime.structured import Grammar, GrammarError, Matcher, json_schema_to_ebnf, regex_to_ebnf
from pie_b200.runtime.tokenizer import ByteTokenizer


def allowed(m, vocab=256):
    return set(np.flatnonzero(brle.decode(m.next_token_logit_mask(), vocab)).tolist())


def feed(m, s):
    m.accept_tokens(list(s.encode()))


def test_regex_masks_match_python_re():
    pat = r"(ab|ac)+[0-9]{2,3}(x|yz)?"
    tok = ByteTokenizer(256)
    m = Matcher(Grammar.from_regex(pat), tok)
    import regex
    rx = regex.compile(pat)
    # walk a few strings; at each prefix the allowed set must equal the brute-force viable set
    alphabet = [ord(c) for c in "abc0123456789xyz!"]
    for s in ["abac123yz", "ac00x", "ab12"]:
        m.reset()
        for i, ch in enumerate(s):
            got = allowed(m) & set(alphabet)
            want = {c for c in alphabet if _viable(rx, s[:i] + chr(c))}
            assert got == want, (s[:i], got, want)
            feed(m, ch)
        assert m.native.can_terminate() == bool(rx.fullmatch(s))


def _viable(rx, prefix):
    """Can `prefix` be extended to a full match? (the regex module's partial matching)"""
    return rx.fullmatch(prefix, partial=True) is not None


def test_json_grammar_accepts_valid_rejects_invalid():
    tok = ByteTokenizer(256)
    m = Matcher(Grammar.json(), tok)
    for doc in ['{"a": [1, 2.5e3, true, null], "b": {"c": "x\\n\\u00e9"}}', "[]", '"s"', "-0.5", "[[[]]]"]:
        m.reset()
        feed(m, doc)
        assert m.native.can_terminate(), doc
        json.loads(doc)
    for bad in ['{"a" 1}', "[1,]", "01", '{"a":}', "tru e"]:
        m.reset()
        with pytest.raises(GrammarError):
            feed(m, bad)
            if not m.native.can_terminate():
                raise GrammarError("incomplete")


def test_json_schema_required_optional_enum_array():
    schema = {"type": "object",
              "properties": {"name": {"type": "string"}, "age": {"type": "integer"},
                             "tags": {"type": "array", "items": {"enum": ["a", "b"]}, "minItems": 1, "maxItems": 2}},
              "required": ["name", "age"]}
    tok = ByteTokenizer(256)
    m = Matcher(Grammar.from_json_schema(schema), tok)
    ok = ['{"name": "x", "age": 3}', '{"name":"x","age":-12,"tags":["a"]}', '{"name":"","age":0,"tags":["a","b"]}']
    bad = ['{"age": 3}', '{"name":"x","age":1.5}', '{"name":"x","age":1,"tags":[]}',
           '{"name":"x","age":1,"tags":["a","b","a"]}', '{"name":"x","age":1,"tags":["c"]}']
    for doc in ok:
        m.reset()
        feed(m, doc)
        assert m.native.can_terminate(), doc
    for doc in bad:
        m.reset()
        with pytest.raises(GrammarError):
            feed(m, doc)
            if not m.native.can_terminate():
                raise GrammarError("incomplete")


def test_schema_ref_and_anyof():
    schema = {"$defs": {"node": {"type": "object", "properties": {"v": {"type": "integer"},
                                                                   "next": {"anyOf": [{"$ref": "#/$defs/node"}, {"type": "null"}]}},
                                 "required": ["v", "next"]}},
              "$ref": "#/$defs/node"}
    m = Matcher(Grammar.from_json_schema(schema), ByteTokenizer(256))
    feed(m, '{"v":1,"next":{"v":2,"next":null}}')
    assert m.native.can_terminate()


def test_rollback_and_eos_gating():
    tok = ByteTokenizer(256, eos=0)
    m = Matcher(Grammar.from_regex(r"a[0-9]b"), tok)
    assert 0 not in allowed(m)
    feed(m, "a5")
    before = allowed(m)
    feed(m, "b")
    assert allowed(m) == {0}                 # only the stop token once the grammar is complete
    assert m.rollback(1)
    assert allowed(m) == before == {ord("b")}
    feed(m, "b")
    m.accept_tokens([0])
    assert m.is_terminated()


def test_multibyte_tokens_through_trie():
    class Tok:
        vocab_size = 6
        eos_tokens = [5]
        table = [b"{", b'"k"', b'"k":', b" ", b"}", b""]

        def vocabs(self):
            return list(range(5)), self.table[:5]

        def token_bytes(self, t):
            return self.table[t]

    m = Matcher(Grammar.from_json_schema({"type": "object", "properties": {"k": {"type": "null"}}}), Tok())
    assert allowed(m, 6) == {0}
    m.accept_tokens([0])
    # `"k":` overshoots nothing and is legal; `"k"` is legal; `}` is not (k is required)
    assert allowed(m, 6) == {1, 2, 3}


def test_ebnf_errors():
    with pytest.raises(GrammarError):
        Grammar("root ::= missing")
    with pytest.raises(GrammarError):
        Grammar("start ::= \"a\"")


def _engine(driver, tok):
    from pie_b200.inferlets import install_all
    from pie_b200.runtime.engine import Engine, EngineConfig
    eng = Engine(EngineConfig())
    eng.add_model("m", driver, tokenizer=tok)
    install_all(eng)
    return eng


def test_constrained_inferlet_with_dummy_driver():
    from pie_b200.driver.mock import DummyDriver
    eng = _engine(DummyDriver(vocab=256, page_size=16, total_pages=256), ByteTokenizer(256))
    try:
        out = eng.run("constrained-decoding", {"prompt_tokens": [1, 2, 3], "regex": r"(yes|no)-[0-9]{3}",
                                               "max_tokens": 32, "temperature": 1.0}, timeout=60)
        assert re.fullmatch(r"(yes|no)-[0-9]{3}", out), out
        schema = {"type": "object", "properties": {"ok": {"type": "boolean"}, "kind": {"enum": ["a", "b"]}}}
        out = eng.run("constrained-decoding", {"prompt_tokens": [1, 2, 3], "json_schema": schema,
                                               "max_tokens": 2000, "temperature": 1.0}, timeout=60)
        doc = json.loads(out)
        assert isinstance(doc["ok"], bool) and doc["kind"] in ("a", "b")
    finally:
        eng.shutdown()


def test_constrained_greedy_on_tiny_model_cpu():
    from pie_b200.driver.executor import TorchDriver
    from pie_b200.models.config import preset
    from pie_b200.models.weights import random_weights
    cfg = preset("tiny-llama")
    w = random_weights(cfg, "cpu", torch.float32, seed=0)
    drv = TorchDriver(cfg, device="cpu", weights=w, num_pages=64, page_size=16, max_requests=8, max_tokens=128)
    eng = _engine(drv, ByteTokenizer(cfg.vocab_size))
    try:
        out = eng.run("constrained-decoding", {"prompt_tokens": list(range(10, 30)), "regex": r"[0-9]{4}-[a-f]{2}",
                                               "max_tokens": 16}, timeout=120)
        assert re.fullmatch(r"[0-9]{4}-[a-f]{2}", out), out
    finally:
        eng.shutdown()


def test_token_mask_cache_serves_recurring_states():
    """The matcher state recurs (every character inside a string, every array item): the per-grammar
    cache must serve those masks without changing them, for every matcher of the grammar."""
    from pie_b200.runtime.structured import Grammar, Matcher
    from pie_b200.runtime.tokenizer import ByteTokenizer
    tok = ByteTokenizer(512)
    g = Grammar.from_json_schema({"type": "object", "required": ["name", "tags"], "properties": {
        "name": {"type": "string"}, "tags": {"type": "array", "items": {"type": "integer"}}}})
    text = b'{"name":"abcdefgh","tags":[12,345,6789,1]}'
    h0, m0, _ = g.native.mask_cache_stats()

    def run(capacity):
        g.native.set_mask_cache_capacity(capacity)
        m = Matcher(g, tok, stop_tokens=[])
        masks = []
        for b in text:
            masks.append(tuple(m.next_token_logit_mask()))
            m.accept_tokens([b])
        assert m.native.can_terminate()
        return masks

    cold = run(0)                                   # capacity 0: every mask is computed by the trie walk
    h1, m1, n1 = g.native.mask_cache_stats()
    assert n1 == 0 and h1 == h0
    warm = run(512)
    h2, m2, n2 = g.native.mask_cache_stats()
    again = run(512)                                # a second matcher of the same grammar: all hits
    h3, m3, n3 = g.native.mask_cache_stats()
    assert cold == warm == again
    assert h2 - h1 >= 8                             # the repeated states inside "abcdefgh" and the digits
    assert h3 - h2 == len(text) and m3 == m2 and 0 < n3 <= 512


def test_grammar_optimiser_keeps_the_language_and_shrinks_the_rule_set():
    """Helper rules of the front ends (literals, sequences, groups) are inlined, identical rules merged, unreachable ones
    dropped: fewer rules, and every vocabulary mask along valid inputs - and the step at which an invalid input dies - is
    the same as without the pass."""
    from pie_b200.runtime.structured import JSON_RULES, optimise_rules
    tok = ByteTokenizer(512)
    schema = {"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer"},
                                               "tags": {"type": "array", "items": {"enum": ["a", "b"]}},
                                               "addr": {"type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"]}},
              "required": ["name", "age"]}
    cases = [
        (json_schema_to_ebnf(schema), ['{"name": "Ada", "age": 36, "tags": ["a", "b"], "addr": {"city": "X"}}', '{"name": "", "age": -1}'],
         ['{"age": 1}', '{"name": "x", "age": "1"}']),
        ("root ::= value\n" + JSON_RULES, ['[1, {"k": [true, null]}, "s\\n"]', "-1.5e3"], ["[1,, 2]", "{'a': 1}"]),
        (regex_to_ebnf(r"(ab|cd)+[0-9]{2,4}x?"), ["abcd12", "cd9999x"], ["ab1", "abab12345"]),
        ('root ::= expr\nexpr ::= term (("+" | "-") term)*\nterm ::= [0-9]+ | "(" expr ")"\n', ["(1+2)-(3)", "42"], ["(1+", "1++2"]),
    ]
    for n, (ebnf, good, bad) in enumerate(cases):
        plain, opt = Grammar(ebnf, optimise=False), Grammar(ebnf, optimise=True)
        assert opt.rules_compiled <= plain.rules_compiled == plain.rules_parsed, ebnf[:40]
        if n < 2:           # the JSON grammars are full of helper rules: a third or more of the rules go
            assert opt.rules_compiled * 3 <= plain.rules_compiled * 2, (opt.rules_compiled, plain.rules_compiled)
        for text, valid in [(t, True) for t in good] + [(t, False) for t in bad]:
            a, b = Matcher(plain, tok), Matcher(opt, tok)
            died = None
            for i, ch in enumerate(tok.encode(text)):
                ma, mb = a.next_token_logit_mask(), b.next_token_logit_mask()
                assert ma == mb, (text, i)
                if not bool(brle.decode(ma, 512)[ch]):
                    died = i
                    break
                a.accept_tokens([ch])
                b.accept_tokens([ch])
            assert a.native.can_terminate() == b.native.can_terminate() and a.is_terminated() == b.is_terminated()
            # a bad text dies at some byte or ends before the grammar may end
            assert (died is None and a.native.can_terminate()) == valid, text
    # the pass alone: a chain of single-use wrappers collapses into the root; a recursive rule stays a rule
    cls = lambda c: (-1, bytes(bytearray([(1 << (ord(c) & 7)) if i == ord(c) >> 3 else 0 for i in range(32)])))
    rules = [[[(1, b"")]], [[(2, b""), (3, b"")]], [[cls("a")]], [[cls("b"), (3, b"")], []], [[cls("z")]]]
    out, root = optimise_rules(rules, 0)
    assert root == 0 and len(out) == 2 and out[0] == [[cls("a"), (1, b"")]] and out[1] == [[cls("b"), (1, b"")], []]
