"""Tokenizers: byte-pair encoding loaded from a Hugging Face `tokenizer.json` (byte-level GPT-2
style as in Llama-3 / Qwen, and sentencepiece-style with byte fallback as in Llama-2 / Mistral),
plus a trivial byte tokenizer for models without vocabulary files (random-init benchmarks).

Pipeline: split around added/special tokens -> normalise -> pre-tokenise with the model's split
regex -> BPE merges per piece (native engine, csrc/host/bpe.hpp) -> ids. Decoding concatenates
token bytes. Counterpart of runtime/src/model/tokenizer.rs, tokenizer/bpe.rs and
tokenizer/hf_loader.rs in the reference.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

import regex

# the split of the ByteLevel pre-tokenizer (GPT-2); newer models ship their own Split regex
GPT2_SPLIT = r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""


def _byte_unicode_map() -> Dict[int, str]:
    """GPT-2's reversible byte <-> printable unicode mapping used by byte-level vocabularies."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


_B2U = _byte_unicode_map()
_U2B = {u: b for b, u in _B2U.items()}


class ByteTokenizer:
    """ids 0..255 are bytes; for engines running random-init weights."""

    def __init__(self, vocab_size: int = 256, eos: Optional[int] = None):
        self.vocab_size = vocab_size
        self.eos_tokens = [eos] if eos is not None else []

    def encode(self, text: str) -> List[int]:
        return list(text.encode("utf-8"))

    def decode(self, tokens: Sequence[int]) -> str:
        return bytes(t & 0xFF for t in tokens).decode("utf-8", errors="replace")

    def vocabs(self) -> Tuple[List[int], List[bytes]]:
        return list(range(256)), [bytes([i]) for i in range(256)]

    def split_regex(self) -> str:
        return ""

    def special_tokens(self):
        return [], []


class BpeTokenizer:
    def __init__(self, vocab: Dict[bytes, int], merges: List[Tuple[bytes, bytes]], split_regex: str = GPT2_SPLIT,
                 special: Optional[Dict[str, int]] = None, byte_fallback: bool = False, metaspace: bool = False,
                 eos_tokens: Sequence[int] = (), unk_id: int = 0, add_prefix_space: bool = False):
        from .._C import pie_host
        toks, ids = zip(*vocab.items()) if vocab else ((), ())
        self.core = pie_host.BpeCore(list(toks), list(ids), merges, unk_id, byte_fallback)
        self.vocab = vocab
        self._split = regex.compile(split_regex) if split_regex else None
        self._split_src = split_regex
        self.special = dict(special or {})
        self._special_re = (regex.compile("|".join(regex.escape(s) for s in sorted(self.special, key=len, reverse=True)))
                            if self.special else None)
        self._id2special = {i: s for s, i in self.special.items()}
        self.metaspace, self.add_prefix_space = metaspace, add_prefix_space
        self.eos_tokens = list(eos_tokens)
        self.vocab_size = max(list(vocab.values()) + list(self.special.values()) + [0]) + 1

    # ---- encode
    def _encode_plain(self, text: str) -> List[int]:
        if not text:
            return []
        if self.metaspace:
            text = text.replace(" ", "▁")
            if self.add_prefix_space and not text.startswith("▁"):
                text = "▁" + text
            pieces = [text.encode("utf-8")]
        elif self._split is not None:
            pieces = [m.group(0).encode("utf-8") for m in self._split.finditer(text)]
        else:
            pieces = [text.encode("utf-8")]
        return self.core.encode_pieces(pieces)

    def encode(self, text: str, allow_special: bool = True) -> List[int]:
        if not allow_special or self._special_re is None:
            return self._encode_plain(text)
        out, pos = [], 0
        for m in self._special_re.finditer(text):
            out.extend(self._encode_plain(text[pos:m.start()]))
            out.append(self.special[m.group(0)])
            pos = m.end()
        out.extend(self._encode_plain(text[pos:]))
        return out

    # ---- decode
    def token_bytes(self, tid: int) -> bytes:
        if tid in self._id2special:
            return self._id2special[tid].encode("utf-8")
        try:
            return bytes(self.core.token_bytes(tid))
        except Exception:  # noqa: BLE001
            return b""

    def decode(self, tokens: Sequence[int], skip_special: bool = False) -> str:
        buf = b"".join(b"" if (skip_special and t in self._id2special) else self.token_bytes(t) for t in tokens)
        text = buf.decode("utf-8", errors="replace")
        return text.replace("▁", " ") if self.metaspace else text

    def vocabs(self) -> Tuple[List[int], List[bytes]]:
        items = sorted(self.vocab.items(), key=lambda kv: kv[1])
        return [i for _, i in items], [t for t, _ in items]

    def split_regex(self) -> str:
        return self._split_src or ""

    def special_tokens(self) -> Tuple[List[int], List[bytes]]:
        items = sorted(self.special.items(), key=lambda kv: kv[1])
        return [i for _, i in items], [s.encode("utf-8") for s, _ in items]


def _find_split_regex(pre) -> Tuple[Optional[str], bool]:
    """(split regex, byte_level) from a tokenizer.json pre_tokenizer tree."""
    if pre is None:
        return None, False
    t = pre.get("type")
    if t == "Sequence":
        rx, bl = None, False
        for p in pre.get("pretokenizers", []):
            r, b = _find_split_regex(p)
            rx, bl = rx or r, bl or b
        return rx, bl
    if t == "Split":
        pat = pre.get("pattern", {})
        return pat.get("Regex") or regex.escape(pat.get("String", "")), False
    if t == "ByteLevel":
        return (GPT2_SPLIT if pre.get("use_regex", True) else None), True
    return None, False


def load_hf_tokenizer(path) -> BpeTokenizer:
    """Build a BpeTokenizer from `tokenizer.json` (+ `tokenizer_config.json` / `generation_config.json`
    for the end-of-sequence ids) in directory `path`."""
    p = Path(path)
    tj = json.loads((p / "tokenizer.json").read_text(encoding="utf-8") if p.is_dir() else p.read_text(encoding="utf-8"))
    model = tj["model"]
    if model.get("type", "BPE") != "BPE":
        raise ValueError(f"unsupported tokenizer model {model.get('type')}")
    split, byte_level = _find_split_regex(tj.get("pre_tokenizer"))
    dec = tj.get("decoder") or {}
    byte_level = byte_level or dec.get("type") == "ByteLevel"
    byte_fallback = bool(model.get("byte_fallback", False))
    metaspace = not byte_level

    def raw(tok: str) -> bytes:
        if byte_level:
            try:
                return bytes(_U2B[c] for c in tok)
            except KeyError:
                return tok.encode("utf-8")
        if byte_fallback and len(tok) == 6 and tok.startswith("<0x") and tok.endswith(">"):
            return bytes([int(tok[3:5], 16)])
        return tok.encode("utf-8")

    vocab = {}
    for tok, i in model["vocab"].items():
        vocab.setdefault(raw(tok), i)
    merges = []
    for m in model.get("merges", []):
        a, b = m.split(" ", 1) if isinstance(m, str) else m
        merges.append((raw(a), raw(b)))
    special = {t["content"]: t["id"] for t in tj.get("added_tokens", [])}
    eos = []
    base = p if p.is_dir() else p.parent
    for fn in ("generation_config.json", "config.json"):
        f = base / fn
        if f.exists():
            e = json.loads(f.read_text()).get("eos_token_id")
            if e is not None:
                eos = e if isinstance(e, list) else [e]
                break
    if not eos:
        f = base / "tokenizer_config.json"
        if f.exists():
            name = json.loads(f.read_text()).get("eos_token")
            name = name.get("content") if isinstance(name, dict) else name
            if name in special:
                eos = [special[name]]
    unk = model.get("unk_token")
    unk_id = model["vocab"].get(unk, 0) if unk else 0
    add_prefix = bool((tj.get("normalizer") or {}).get("type") in ("Prepend", "Sequence")) and metaspace
    return BpeTokenizer(vocab, merges, split if byte_level or split else "", special, byte_fallback, metaspace, eos,
                        unk_id, add_prefix)


# split regexes of the byte-level pre-tokenizers that GGUF files name in `tokenizer.ggml.pre`
_GGUF_PRE = {
    "llama-bpe": r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+",
    "qwen2": r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+",
}
_GGUF_PRE["llama3"] = _GGUF_PRE["llama-bpe"]


def load_gguf_tokenizer(source) -> BpeTokenizer:
    """Build a BpeTokenizer from the `tokenizer.ggml.*` metadata of a GGUF file (a path or an open
    `GGUFReader`). Byte-level BPE vocabularies (`tokenizer.ggml.model = gpt2`) are covered; control
    and user-defined tokens (token types 3 and 4) become special tokens."""
    if hasattr(source, "meta"):
        meta = source.meta
    else:
        from ..models.gguf import GGUFReader
        meta = GGUFReader(source).meta
    kind = meta.get("tokenizer.ggml.model", "gpt2")
    if kind != "gpt2":
        raise ValueError(f"GGUF tokenizer model {kind!r} is not byte-level BPE")
    tokens = meta.get("tokenizer.ggml.tokens") or []
    types = meta.get("tokenizer.ggml.token_type") or [1] * len(tokens)

    def raw(tok: str) -> bytes:
        try:
            return bytes(_U2B[c] for c in tok)
        except KeyError:
            return tok.encode("utf-8")

    vocab, special = {}, {}
    for i, (tok, tt) in enumerate(zip(tokens, types)):
        if tt in (3, 4):
            special[tok] = i
        else:
            vocab.setdefault(raw(tok), i)
    merges = []
    for m in meta.get("tokenizer.ggml.merges") or []:
        a, b = m.split(" ", 1)
        merges.append((raw(a), raw(b)))
    eos = [int(meta[k]) for k in ("tokenizer.ggml.eos_token_id", "tokenizer.ggml.eot_token_id") if k in meta]
    split = _GGUF_PRE.get(str(meta.get("tokenizer.ggml.pre", "")), GPT2_SPLIT)
    return BpeTokenizer(vocab, merges, split, special, False, False, sorted(set(eos)),
                        int(meta.get("tokenizer.ggml.unknown_token_id", 0)), False)
