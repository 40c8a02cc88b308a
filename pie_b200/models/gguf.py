"""GGUF checkpoint source: a reader that presents a ``.gguf`` file under Hugging Face tensor names,
so that the storage-program compiler and executor of :mod:`.loader` run on it unchanged.

Covers the container (header, metadata key/values, tensor table, aligned data section) and the
tensor types F32, F16, BF16, Q8_0 and Q4_0 (block formats are expanded on read; the runtime keeps
bf16). Llama-architecture files store q/k projection rows in the interleaved-rotary order of
llama.cpp; they are put back into the rotate-half order the kernels use.

The reference reads GGUF next to safetensors in its C++ loader (driver/cuda/src/loader/).
"""
from __future__ import annotations

import struct
from pathlib import Path
from typing import Dict, List, Tuple

import numpy as np
import torch

from .config import ModelConfig

GGUF_MAGIC = b"GGUF"
T_F32, T_F16, T_Q4_0, T_Q8_0, T_BF16 = 0, 1, 2, 8, 30
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_BLOCK = {T_F32: (1, 4), T_F16: (1, 2), T_BF16: (1, 2), T_Q8_0: (32, 34), T_Q4_0: (32, 18)}   # elements, bytes per block

# GGUF tensor names -> Hugging Face names ({i} = layer)
_TOP = {"token_embd.weight": "model.embed_tokens.weight", "output_norm.weight": "model.norm.weight",
        "output.weight": "lm_head.weight"}
_LAYER = {"attn_norm.weight": "input_layernorm.weight", "ffn_norm.weight": "post_attention_layernorm.weight",
          "attn_q.weight": "self_attn.q_proj.weight", "attn_k.weight": "self_attn.k_proj.weight",
          "attn_v.weight": "self_attn.v_proj.weight", "attn_output.weight": "self_attn.o_proj.weight",
          "attn_q.bias": "self_attn.q_proj.bias", "attn_k.bias": "self_attn.k_proj.bias",
          "attn_v.bias": "self_attn.v_proj.bias", "attn_q_norm.weight": "self_attn.q_norm.weight",
          "attn_k_norm.weight": "self_attn.k_norm.weight", "ffn_gate.weight": "mlp.gate_proj.weight",
          "ffn_up.weight": "mlp.up_proj.weight", "ffn_down.weight": "mlp.down_proj.weight"}


def hf_name(gguf_name: str) -> str:
    if gguf_name in _TOP:
        return _TOP[gguf_name]
    if gguf_name.startswith("blk."):
        _, li, rest = gguf_name.split(".", 2)
        if rest in _LAYER:
            return f"model.layers.{li}.{_LAYER[rest]}"
    return gguf_name


class _Cursor:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt):
        v = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += struct.calcsize(fmt)
        return v[0] if len(v) == 1 else v

    def string(self) -> str:
        n = self.take("<Q")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, vt):
        if vt in _SCALARS:
            return self.take(_SCALARS[vt])
        if vt == 8:
            return self.string()
        if vt == 9:
            et, n = self.take("<I"), self.take("<Q")
            if et in _SCALARS:      # numeric arrays in one go
                fmt = _SCALARS[et]
                arr = np.frombuffer(self.buf, dtype=np.dtype(fmt), count=n, offset=self.pos)
                self.pos += arr.nbytes
                return arr.tolist()
            return [self.value(et) for _ in range(n)]
        raise ValueError(f"unknown GGUF value type {vt}")


def dequantize(raw: np.ndarray, ggml_type: int, n: int) -> np.ndarray:
    """Bytes of `n` elements of a GGUF tensor -> float32 (F32) / float16 / bfloat16-as-uint16 stay
    zero-copy; block formats are expanded: Q8_0 = fp16 scale + 32 int8, Q4_0 = fp16 scale + 32
    nibbles (element i < 16 in the low nibble of byte i, element 16 + i in its high nibble)."""
    if ggml_type == T_F32:
        return raw.view(np.float32)
    if ggml_type == T_F16:
        return raw.view(np.float16)
    if ggml_type == T_BF16:
        return raw.view(np.uint16)
    nb = n // 32
    if ggml_type == T_Q8_0:
        blk = raw.reshape(nb, 34)
        d = blk[:, :2].copy().view(np.float16).astype(np.float32)
        q = blk[:, 2:].view(np.int8).astype(np.float32)
        return (q * d).reshape(-1)
    if ggml_type == T_Q4_0:
        blk = raw.reshape(nb, 18)
        d = blk[:, :2].copy().view(np.float16).astype(np.float32)
        b = blk[:, 2:]
        q = np.concatenate([b & 0x0F, b >> 4], axis=1).astype(np.float32) - 8.0
        return (q * d).reshape(-1)
    raise NotImplementedError(f"GGUF tensor type {ggml_type}")


class _Sliceable:
    """The slice protocol the storage-program executor uses on safetensors handles."""

    def __init__(self, reader: "GGUFReader", name: str):
        self.reader, self.name = reader, name

    def get_shape(self):
        return list(self.reader.shape(self.name))

    def __getitem__(self, idx):
        return self.reader.get(self.name)[idx]


class GGUFReader:
    def __init__(self, path):
        self.path = Path(path)
        self.buf = np.memmap(self.path, dtype=np.uint8, mode="r")
        c = _Cursor(self.buf)
        if bytes(self.buf[:4]) != GGUF_MAGIC:
            raise ValueError(f"{path} is not a GGUF file")
        c.pos = 4
        self.version = c.take("<I")
        if self.version < 2:
            raise ValueError(f"GGUF version {self.version} is not supported")
        n_tensors, n_kv = c.take("<Q"), c.take("<Q")
        self.meta: Dict[str, object] = {}
        for _ in range(n_kv):
            key = c.string()
            self.meta[key] = c.value(c.take("<I"))
        self.infos: Dict[str, Tuple[Tuple[int, ...], int, int]] = {}
        for _ in range(n_tensors):
            name = c.string()
            nd = c.take("<I")
            ne = [c.take("<Q") for _ in range(nd)]
            tt, off = c.take("<I"), c.take("<Q")
            self.infos[hf_name(name)] = (tuple(reversed(ne)), tt, off)     # ne[0] is the innermost dimension
        align = int(self.meta.get("general.alignment", 32))
        self.data_start = (c.pos + align - 1) // align * align
        self.arch = str(self.meta.get("general.architecture", "llama"))

    # ---- the reader protocol of loader.execute_program
    def names(self) -> List[str]:
        return list(self.infos)

    def shape(self, name):
        return self.infos[name][0]

    def get_slice(self, name):
        return _Sliceable(self, name)

    def get(self, name) -> torch.Tensor:
        shape, tt, off = self.infos[name]
        n = int(np.prod(shape)) if shape else 1
        per, nbytes = _BLOCK[tt]
        raw = np.asarray(self.buf[self.data_start + off: self.data_start + off + n // per * nbytes])
        arr = dequantize(raw, tt, n)
        if tt == T_BF16:
            t = torch.from_numpy(arr.copy()).view(torch.bfloat16).reshape(shape)
        else:
            t = torch.from_numpy(np.array(arr, copy=True)).reshape(shape)
        if self.arch == "llama" and name.endswith(("self_attn.q_proj.weight", "self_attn.k_proj.weight")):
            heads = self._meta_int("attention.head_count")
            if name.endswith("k_proj.weight"):
                heads = self._meta_int("attention.head_count_kv", heads)
            t = unpermute_rotary(t, heads)
        return t

    # ---- configuration
    def _meta_int(self, key, default=None):
        v = self.meta.get(f"{self.arch}.{key}", default)
        if v is None:
            raise KeyError(f"GGUF metadata has no {self.arch}.{key}")
        return int(v)

    def config(self) -> ModelConfig:
        a = self.arch
        hidden, heads = self._meta_int("embedding_length"), self._meta_int("attention.head_count")
        vocab = self.meta.get(f"{a}.vocab_size") or len(self.meta.get("tokenizer.ggml.tokens", [])) or \
            self.infos["model.embed_tokens.weight"][0][0]
        mt = {"llama": "llama", "qwen2": "qwen2", "qwen3": "qwen3", "mistral": "mistral", "phi3": "phi3"}.get(a, a)
        hf = {
            "model_type": mt, "hidden_size": hidden, "num_attention_heads": heads,
            "num_key_value_heads": self._meta_int("attention.head_count_kv", heads),
            "num_hidden_layers": self._meta_int("block_count"),
            "intermediate_size": self._meta_int("feed_forward_length"),
            "head_dim": int(self.meta.get(f"{a}.attention.key_length", hidden // heads)),
            "vocab_size": int(vocab),
            "max_position_embeddings": self._meta_int("context_length", 8192),
            "rms_norm_eps": float(self.meta.get(f"{a}.attention.layer_norm_rms_epsilon", 1e-5)),
            "rope_theta": float(self.meta.get(f"{a}.rope.freq_base", 10000.0)),
            "tie_word_embeddings": "lm_head.weight" not in self.infos,
            "torch_dtype": "bfloat16",
        }
        return ModelConfig.from_hf(hf, name=str(self.meta.get("general.name", self.path.stem)))


def unpermute_rotary(w: torch.Tensor, heads: int) -> torch.Tensor:
    """Rows of a q/k projection from llama.cpp's interleaved-pair order (x0, x_{d/2}, x1, ...)
    back to the half-split order (x0 .. x_{d/2-1}, x_{d/2} ..) of rotate-half RoPE."""
    rows = w.shape[0]
    d = rows // heads
    return w.reshape(heads, d // 2, 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


def permute_rotary(w: torch.Tensor, heads: int) -> torch.Tensor:
    """Inverse of :func:`unpermute_rotary` (what the Hugging Face -> GGUF conversion applies)."""
    rows = w.shape[0]
    d = rows // heads
    return w.reshape(heads, 2, d // 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


# ----------------------------------------------------------------------------- writer (tests, tooling)
def _w_string(out: bytearray, s: str):
    b = s.encode("utf-8")
    out += struct.pack("<Q", len(b)) + b


def quantize_q8_0(x: np.ndarray) -> bytes:
    blk = x.astype(np.float32).reshape(-1, 32)
    d = np.abs(blk).max(axis=1, keepdims=True) / 127.0
    q = np.where(d > 0, np.round(blk / np.where(d > 0, d, 1.0)), 0).astype(np.int8)
    out = np.empty((blk.shape[0], 34), dtype=np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.tobytes()


def write_gguf(path, meta: Dict[str, object], tensors: Dict[str, Tuple[torch.Tensor, int]], align: int = 32) -> None:
    """Write `tensors` ({gguf name: (tensor, ggml type)}; F32 / F16 / BF16 / Q8_0) and `meta`
    (ints, floats, strings, lists of strings) as a version-3 GGUF file."""
    out = bytearray(GGUF_MAGIC + struct.pack("<IQQ", 3, len(tensors), len(meta)))
    for k, v in meta.items():
        _w_string(out, k)
        if isinstance(v, bool):
            out += struct.pack("<I?", 7, v)
        elif isinstance(v, int):
            out += struct.pack("<II", 4, v)
        elif isinstance(v, float):
            out += struct.pack("<If", 6, v)
        elif isinstance(v, str):
            out += struct.pack("<I", 8)
            _w_string(out, v)
        elif isinstance(v, list):
            out += struct.pack("<IIQ", 9, 8, len(v))
            for s in v:
                _w_string(out, str(s))
        else:
            raise TypeError(f"metadata value of {k}")
    blobs, off = [], 0
    for name, (t, tt) in tensors.items():
        a = t.detach().cpu()
        if tt == T_F32:
            data = a.float().numpy().tobytes()
        elif tt == T_F16:
            data = a.half().numpy().tobytes()
        elif tt == T_BF16:
            data = a.bfloat16().view(torch.int16).numpy().tobytes()
        elif tt == T_Q8_0:
            data = quantize_q8_0(a.float().numpy())
        else:
            raise NotImplementedError(f"writer: GGUF tensor type {tt}")
        _w_string(out, name)
        dims = list(reversed(a.shape))
        out += struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", tt, off)
        blobs.append(data)
        off += (len(data) + align - 1) // align * align
    out += b"\0" * (-len(out) % align)
    for data in blobs:
        out += data + b"\0" * (-len(data) % align)
    Path(path).write_bytes(bytes(out))
