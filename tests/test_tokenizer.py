"""BPE tokenizer (native merge engine + tokenizer.json loader) against the Hugging Face
`tokenizers` library on vocabularies trained in-process (no files from the network)."""
import os
import tempfile

import pytest

tokenizers = pytest.importorskip("tokenizers")
from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers  # noqa: E402

from pie_b200.runtime.tokenizer import ByteTokenizer, load_hf_tokenizer  # noqa: E402

CORPUS = ["the quick brown fox jumps over the lazy dog " * 3, "hello world, hello tokenizer! 12345 café naïve über",
          "def f(x):\n    return x*2\n" * 4, "日本語のテキスト と emoji 😀"]
PROBES = CORPUS + ["unseen words: zebra <|eot|> tail", "  spaces   and\n\nnewlines", "I'm don't we've", ""]


def _train(pre):
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre
    tok.decoder = decoders.ByteLevel()
    tok.train_from_iterator(CORPUS, trainers.BpeTrainer(vocab_size=400, special_tokens=["<|eot|>"],
                                                        initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    return tok


@pytest.mark.parametrize("style", ["gpt2", "llama3"])
def test_bpe_matches_hf_tokenizers(style):
    if style == "gpt2":
        pre = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    else:
        pat = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|"
               r"\s*[\r\n]+|\s+(?!\S)|\s+")
        pre = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(pat), behavior="isolated"),
                                       pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok = _train(pre)
    d = tempfile.mkdtemp()
    tok.save(os.path.join(d, "tokenizer.json"))
    mine = load_hf_tokenizer(d)
    for text in PROBES:
        ids = mine.encode(text)
        assert ids == tok.encode(text).ids, text
        assert mine.decode(ids) == text
    sid, sb = mine.special_tokens()
    assert sb == [b"<|eot|>"] and mine.encode("<|eot|>") == sid
    vid, vb = mine.vocabs()
    assert len(vid) == len(vb) > 256


def test_byte_tokenizer_roundtrip():
    t = ByteTokenizer()
    assert t.decode(t.encode("héllo")) == "héllo"


def test_gguf_tokenizer_metadata_matches_hf_tokenizers(tmp_path):
    """The `tokenizer.ggml.*` metadata of a GGUF file (tokens in byte-unicode form, merges, token
    types, pre-tokenizer name) gives the same ids as the tokenizer it was exported from."""
    import json
    import torch
    from pie_b200.models import gguf
    from pie_b200.runtime.tokenizer import load_gguf_tokenizer
    pat = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|"
           r"\s*[\r\n]+|\s+(?!\S)|\s+")
    tok = _train(pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(pat), behavior="isolated"),
                                          pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)]))
    tj = json.loads(tok.to_str())
    vocab = tj["model"]["vocab"]
    tokens = [None] * len(vocab)
    for t, i in vocab.items():
        tokens[i] = t
    merges = [m if isinstance(m, str) else " ".join(m) for m in tj["model"]["merges"]]
    eot = vocab["<|eot|>"]
    types = [3 if i == eot else 1 for i in range(len(tokens))]
    meta = {"general.architecture": "llama", "tokenizer.ggml.model": "gpt2", "tokenizer.ggml.pre": "llama-bpe",
            "tokenizer.ggml.tokens": tokens, "tokenizer.ggml.merges": merges, "tokenizer.ggml.eos_token_id": eot}
    path = tmp_path / "tok.gguf"
    gguf.write_gguf(path, meta, {"token_embd.weight": (torch.zeros(4, 32), gguf.T_F32)})
    rd = gguf.GGUFReader(path)
    rd.meta["tokenizer.ggml.token_type"] = types        # the test writer has no integer arrays
    mine = load_gguf_tokenizer(rd)
    assert mine.eos_tokens == [eot]
    for text in PROBES:
        assert mine.encode(text) == tok.encode(text).ids, text
        assert mine.decode(mine.encode(text)) == tok.decode(tok.encode(text).ids, skip_special_tokens=False)
