"""Weight loading from Hugging Face safetensors through a small storage-program compiler.

`compile_program(cfg, tensor_names, tp_size, tp_rank, ep)` turns checkpoint metadata + the runtime
layout contract (see models/weights.py) into a typed list of ops; `execute_program` runs it
against a safetensors reader, producing this rank's weight dict. Ops:

  Read(name)                      checkpoint tensor (lazily sliced)
  Shard(axis, rank, world)        contiguous shard along an axis
  Rows(start, count)              explicit row range (KV heads replicated across ranks)
  Concat(axis)                    join operands (fused QKV)
  Interleave()                    rows g0,u0,g1,u1,... (gate/up for the SwiGLU GEMM epilogue)
  Stack()                         expert stacks
  Cast(dtype) / DequantFp8Block() dtype change / 128x128 block-scaled fp8 -> bf16
  Transpose(a, b)                 swap two dimensions (GPT-OSS stores experts as [E, in, out])
  Mxfp4(blocks, scales)           e2m1 nibbles with one e8m0 scale per 32 -> values [.., rows, cols]
  Attach(path)                    store under a runtime name

The program is serialisable (`program_to_json`), so a per-rank plan can be compiled once and
cached. Counterpart of the reference's weight-loader compiler (driver/weight_loader/src/
{frontend,abi,storage_compiler}.rs: fused QKV / gate-up joins, MoE expert stacks, shard axes)
and its C++ executor (driver/cuda/src/loader/*).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .config import ModelConfig
from .weights import kv_head_range, torch_dtype


@dataclass
class Op:
    kind: str
    args: dict = field(default_factory=dict)
    inputs: List["Op"] = field(default_factory=list)

    def to_json(self):
        return {"kind": self.kind, "args": self.args, "inputs": [i.to_json() for i in self.inputs]}

    @staticmethod
    def from_json(d):
        return Op(d["kind"], d["args"], [Op.from_json(i) for i in d["inputs"]])


def Read(name): return Op("read", {"name": name})
def Shard(x, axis, rank, world): return x if world == 1 else Op("shard", {"axis": axis, "rank": rank, "world": world}, [x])
def Rows(x, start, count): return Op("rows", {"start": start, "count": count}, [x])
def Concat(xs, axis=0): return Op("concat", {"axis": axis}, list(xs))
def Interleave(a, b): return Op("interleave", {}, [a, b])
def Stack(xs): return Op("stack", {}, list(xs))
def ExpandRows(x, factor, like): return Op("expand_rows", {"factor": factor, "like": like}, [x])
def Transpose(x, a, b): return Op("transpose", {"a": a, "b": b}, [x])
def AddScalar(x, value): return Op("add_scalar", {"value": value}, [x])
def RowScales(scale, like): return Op("row_scales", {"like": like}, [scale])
def Mxfp4(blocks, scales): return Op("mxfp4", {}, [blocks, scales])

_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def dequant_mxfp4(blocks: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """blocks [..., rows, cols/32, 16] uint8 (two e2m1 values per byte, low nibble first),
    scales [..., rows, cols/32] uint8 (e8m0: 2^(s - 127)) -> float32 [..., rows, cols]."""
    lut = torch.tensor(_E2M1, dtype=torch.float32)
    b = blocks.to(torch.int64)
    vals = torch.stack([lut[b & 0x0F], lut[b >> 4]], dim=-1).reshape(*blocks.shape[:-1], 32)
    sc = torch.exp2(scales.to(torch.float32) - 127.0)
    return (vals * sc[..., None]).reshape(*blocks.shape[:-2], blocks.shape[-2] * 32)


def quant_mxfp4(w: torch.Tensor):
    """Inverse of :func:`dequant_mxfp4` for tests and tooling: nearest e2m1 value under a
    power-of-two scale per 32 columns. Returns (blocks, scales) as uint8."""
    g = w.float().reshape(*w.shape[:-1], w.shape[-1] // 32, 32)
    amax = g.abs().amax(-1).clamp_min(2.0 ** -120)
    e = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)
    q = g / torch.exp2(e)[..., None]
    lut = torch.tensor(_E2M1, dtype=torch.float32)
    idx = (q[..., None] - lut).abs().argmin(-1).to(torch.uint8)
    blocks = (idx[..., 0::2] | (idx[..., 1::2] << 4)).contiguous()
    return blocks, (e + 127).to(torch.uint8).contiguous()


class QLin:
    """A linear weight during planning: the weight expression plus, for block-scaled fp8
    checkpoints, the expression of its per-row scales ([N, K/128], the 128-row block scales
    expanded to rows). Row and column operations apply to both."""

    def __init__(self, w: Op, s: Optional[Op] = None):
        self.w, self.s = w, s

    def shard(self, axis, rank, world):
        if world == 1:
            return self
        return QLin(Shard(self.w, axis, rank, world), Shard(self.s, axis, rank, world) if self.s is not None else None)

    def rows(self, start, count):
        return QLin(Rows(self.w, start, count), Rows(self.s, start, count) if self.s is not None else None)

    @staticmethod
    def concat(xs):
        return QLin(Concat([x.w for x in xs], 0), Concat([x.s for x in xs], 0) if xs[0].s is not None else None)

    @staticmethod
    def interleave(a, b):
        return QLin(Interleave(a.w, b.w), Interleave(a.s, b.s) if a.s is not None else None)

    def attach(self, att: dict, path: str) -> None:
        att[path] = self.w
        if self.s is not None:
            att[path + "@scale"] = self.s


@dataclass
class Program:
    attach: Dict[str, Op]          # runtime path ("layers.3.wqkv") -> expression
    dtype: str
    meta: dict = field(default_factory=dict)


def program_to_json(p: Program) -> str:
    return json.dumps({"dtype": p.dtype, "meta": p.meta, "attach": {k: v.to_json() for k, v in p.attach.items()}})


def program_from_json(s: str) -> Program:
    d = json.loads(s)
    return Program({k: Op.from_json(v) for k, v in d["attach"].items()}, d["dtype"], d.get("meta", {}))


def compile_program(cfg: ModelConfig, names: Sequence[str], tp_size: int = 1, tp_rank: int = 0,
                    ep: bool = False, dtype: str = "bfloat16") -> Program:
    """Layout plan for a Llama/Qwen-family checkpoint (HF names) on rank (tp_rank of tp_size)."""
    names = set(names)
    T, r, d = tp_size, tp_rank, cfg.head_dim
    kv0, kvn = kv_head_range(cfg, r, T)
    # the language model's tensors may sit under a prefix ("model.", or a multimodal wrapper's "model.language_model.")
    pre = min((n[:-len("embed_tokens.weight")] for n in names if n.endswith("embed_tokens.weight")), key=len, default="")
    att: Dict[str, Op] = {}

    def gain(n):
        """RMSNorm gain; Gemma checkpoints store (gain - 1)."""
        return AddScalar(Op("float", {}, [w(n)]), 1.0) if cfg.norm_plus_one else w(n)

    def w(n):
        if n not in names:
            raise KeyError(f"checkpoint has no tensor {n}")
        return Read(n)

    def lin(n):
        """Linear weight `n` (+ its block scales when the checkpoint is fp8)."""
        sc = n + "_scale_inv"
        if cfg.quantization == "fp8_block" and sc in names:
            return QLin(w(n), ExpandRows(Read(sc), 128, n))
        sc = n + "_scale"
        if cfg.quantization == "fp8_block" and sc in names:
            # per-tensor (scalar) or per-output-channel ([N] / [N, 1]) scales: the same number for every 128-wide block of a row
            return QLin(w(n), RowScales(Read(sc), n))
        return QLin(w(n))

    att["embed"] = w(f"{pre}embed_tokens.weight")
    att["final_norm"] = gain(f"{pre}norm.weight")
    # an untied output projection sits beside the language model's `model.` subtree (under a wrapper's prefix too)
    head_names = ["lm_head.weight"] + ([pre[:-len("model.")] + "lm_head.weight"] if pre.endswith("model.") else [])
    head = next((w(n) for n in head_names if n in names), None) or w(f"{pre}embed_tokens.weight")
    att["lm_head"] = Shard(head, 0, r, T)
    for li in range(cfg.num_hidden_layers):
        L, P = f"{pre}layers.{li}.", f"layers.{li}."
        if cfg.is_mamba_layer(li):
            # Mamba-2 layer under the names of the Mamba-2 checkpoints (`mixer.*`); in_proj rows are already z | x B C | dt
            if T > 1:
                raise NotImplementedError("Mamba-2 layers under tensor parallelism")
            X = L + "mixer."
            att[P + "w_mamba_in"] = w(X + "in_proj.weight")
            att[P + "mamba_conv"] = Op("squeeze", {"dim": 1}, [w(X + "conv1d.weight")])
            att[P + "mamba_conv_bias"] = w(X + "conv1d.bias")
            for src, dst in (("A_log", "mamba_A_log"), ("dt_bias", "mamba_dt_bias"), ("D", "mamba_D")):
                att[P + dst] = Op("float", {}, [w(X + src)])
            att[P + "mamba_norm"], att[P + "w_mamba_out"] = w(X + "norm.weight"), w(X + "out_proj.weight")
            att[P + "ln1"], att[P + "ln2"] = w(L + "input_layernorm.weight"), w(L + "post_attention_layernorm.weight")
            QLin.interleave(lin(L + "mlp.gate_proj.weight"), lin(L + "mlp.up_proj.weight")).attach(att, P + "w_gate_up")
            lin(L + "mlp.down_proj.weight").attach(att, P + "w_down")
            continue
        if cfg.is_linear_layer(li):
            # Gated DeltaNet layer. The checkpoint groups the fused projections by key head:
            # in_proj_qkvz rows = per key head [q (dk), k (dk), v (rep * dv), z (rep * dv)], in_proj_ba rows = per
            # key head [b (rep), a (rep)]; the runtime wants q | k | v | z | b | a, each over all heads.
            if T > 1:
                raise NotImplementedError("Gated DeltaNet layers under tensor parallelism")
            X = L + "linear_attn."
            hk, hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
            dk, dv, rep = cfg.linear_key_head_dim, cfg.linear_value_head_dim, hv // hk
            G, qkvz, ba = 2 * dk + 2 * rep * dv, w(X + "in_proj_qkvz.weight"), w(X + "in_proj_ba.weight")
            parts = ([Rows(qkvz, g * G, dk) for g in range(hk)] + [Rows(qkvz, g * G + dk, dk) for g in range(hk)]
                     + [Rows(qkvz, g * G + 2 * dk, rep * dv) for g in range(hk)]
                     + [Rows(qkvz, g * G + 2 * dk + rep * dv, rep * dv) for g in range(hk)]
                     + [Rows(ba, g * 2 * rep, rep) for g in range(hk)] + [Rows(ba, g * 2 * rep + rep, rep) for g in range(hk)])
            att[P + "w_gdn_in"] = Concat(parts, 0)
            att[P + "gdn_conv"] = Op("squeeze", {"dim": 1}, [w(X + "conv1d.weight")])
            att[P + "gdn_A_log"], att[P + "gdn_dt_bias"] = Op("float", {}, [w(X + "A_log")]), Op("float", {}, [w(X + "dt_bias")])
            att[P + "gdn_norm"], att[P + "w_gdn_out"] = w(X + "norm.weight"), w(X + "out_proj.weight")
            att[P + "ln1"], att[P + "ln2"] = w(L + "input_layernorm.weight"), w(L + "post_attention_layernorm.weight")
            QLin.interleave(lin(L + "mlp.gate_proj.weight"), lin(L + "mlp.up_proj.weight")).attach(att, P + "w_gate_up")
            lin(L + "mlp.down_proj.weight").attach(att, P + "w_down")
            continue
        if cfg.sandwich_norm:   # Gemma-2/3: a norm on the way into and out of each sub-block
            att[P + "ln1"], att[P + "ln_pa"] = gain(L + "input_layernorm.weight"), gain(L + "post_attention_layernorm.weight")
            att[P + "ln2"], att[P + "ln_pf"] = gain(L + "pre_feedforward_layernorm.weight"), gain(L + "post_feedforward_layernorm.weight")
        elif cfg.post_norm:     # OLMo-2: norms follow the sub-blocks, there is no input norm
            att[P + "ln2"] = w(L + "post_attention_layernorm.weight")
            att[P + "ln3"] = w(L + "post_feedforward_layernorm.weight")
        else:
            att[P + "ln1"] = w(L + "input_layernorm.weight")
            att[P + "ln2"] = w(L + "post_attention_layernorm.weight")
        hq_d, hkv_d = cfg.num_attention_heads * d, cfg.num_key_value_heads * d
        if L + "self_attn.qkv_proj.weight" in names:          # Phi-3: q, k, v rows stored in one tensor
            fused = lin(L + "self_attn.qkv_proj.weight")
            q = fused.rows(0, hq_d).shard(0, r, T)
            k = fused.rows(hq_d + kv0 * d, kvn * d)
            v = fused.rows(hq_d + hkv_d + kv0 * d, kvn * d)
        else:
            q = lin(L + "self_attn.q_proj.weight").shard(0, r, T)
            k = lin(L + "self_attn.k_proj.weight").rows(kv0 * d, kvn * d)
            v = lin(L + "self_attn.v_proj.weight").rows(kv0 * d, kvn * d)
        QLin.concat([q, k, v]).attach(att, P + "wqkv")
        if L + "self_attn.q_proj.bias" in names:
            att[P + "bqkv"] = Concat([Shard(w(L + "self_attn.q_proj.bias"), 0, r, T),
                                      Rows(w(L + "self_attn.k_proj.bias"), kv0 * d, kvn * d),
                                      Rows(w(L + "self_attn.v_proj.bias"), kv0 * d, kvn * d)], 0)
        lin(L + "self_attn.o_proj.weight").shard(1, r, T).attach(att, P + "wo")
        if L + "self_attn.o_proj.bias" in names:
            att[P + "bo"] = w(L + "self_attn.o_proj.bias")
        if L + "self_attn.sinks" in names:
            att[P + "sinks"] = Shard(w(L + "self_attn.sinks"), 0, r, T)
        if L + "self_attn.q_norm.weight" in names and cfg.post_norm:
            # gains over all heads together (OLMo-2): a rank keeps those of its own heads
            att[P + "q_norm"] = Shard(w(L + "self_attn.q_norm.weight"), 0, r, T)
            att[P + "k_norm"] = Rows(w(L + "self_attn.k_norm.weight"), kv0 * d, kvn * d) if T > 1 \
                else w(L + "self_attn.k_norm.weight")
        elif L + "self_attn.q_norm.weight" in names:
            att[P + "q_norm"] = gain(L + "self_attn.q_norm.weight")
            att[P + "k_norm"] = gain(L + "self_attn.k_norm.weight")
        mixtral = L + "block_sparse_moe.gate.weight" in names      # Mixtral names: w1 = gate, w3 = up, w2 = down
        if cfg.is_moe and L + "mlp.router.weight" in names:
            # GPT-OSS: experts stacked in one tensor, gate/up columns already interleaved; bf16 checkpoints
            # hold [E, in, out], MXFP4 ones blocks + scales in [E, out, in/32, ...]
            if T > 1 and ep:
                raise NotImplementedError("GPT-OSS experts under expert parallelism")
            X = L + "mlp.experts."
            att[P + "router"], att[P + "router_bias"] = w(L + "mlp.router.weight"), w(L + "mlp.router.bias")
            # runtime layout [E, out, in]; under tensor parallelism the intermediate dimension is sharded:
            # rows of gate_up (interleaved pairs stay together), columns of down
            for src, dst, ax in (("gate_up_proj", "experts_gate_up", 1), ("down_proj", "experts_down", 2)):
                if X + src + "_blocks" in names:
                    full = Mxfp4(w(X + src + "_blocks"), w(X + src + "_scales"))
                else:
                    full = Transpose(w(X + src), 1, 2)
                att[P + dst] = Shard(full, ax, r, T)
            att[P + "experts_gate_up_bias"] = Shard(w(X + "gate_up_proj_bias"), 1, r, T)
            att[P + "experts_down_bias"] = w(X + "down_proj_bias") if r == 0 else Op("zeros_like", {}, [w(X + "down_proj_bias")])
        elif cfg.is_moe and (L + "mlp.gate.weight" in names or mixtral):
            att[P + "router"] = w(L + ("block_sparse_moe.gate.weight" if mixtral else "mlp.gate.weight"))
            E = cfg.num_experts
            experts = range(r * (E // T), (r + 1) * (E // T)) if (ep and T > 1) else range(E)
            gus, downs = [], []
            for e in experts:
                if mixtral:
                    X = f"{L}block_sparse_moe.experts.{e}."
                    g, u, dn = w(X + "w1.weight"), w(X + "w3.weight"), w(X + "w2.weight")
                else:
                    X = f"{L}mlp.experts.{e}."
                    g, u, dn = w(X + "gate_proj.weight"), w(X + "up_proj.weight"), w(X + "down_proj.weight")
                if not ep:
                    g, u, dn = Shard(g, 0, r, T), Shard(u, 0, r, T), Shard(dn, 1, r, T)
                gus.append(Interleave(g, u))
                downs.append(dn)
            att[P + "experts_gate_up"] = Stack(gus)
            att[P + "experts_down"] = Stack(downs)
            if L + "mlp.shared_expert.gate_proj.weight" in names:
                # the shared expert (Qwen2-MoE): a dense MLP, sharded like one; its per-token gate is replicated
                S = L + "mlp.shared_expert."
                QLin.interleave(lin(S + "gate_proj.weight").shard(0, r, T), lin(S + "up_proj.weight").shard(0, r, T)).attach(
                    att, P + "shared_gate_up")
                lin(S + "down_proj.weight").shard(1, r, T).attach(att, P + "shared_down")
                att[P + "shared_gate"] = w(L + "mlp.shared_expert_gate.weight")
        else:
            if L + "mlp.gate_up_proj.weight" in names:        # Phi-3: gate rows then up rows in one tensor
                gu = lin(L + "mlp.gate_up_proj.weight")
                gate, up = gu.rows(0, cfg.intermediate_size), gu.rows(cfg.intermediate_size, cfg.intermediate_size)
            else:
                gate, up = lin(L + "mlp.gate_proj.weight"), lin(L + "mlp.up_proj.weight")
            QLin.interleave(gate.shard(0, r, T), up.shard(0, r, T)).attach(att, P + "w_gate_up")
            lin(L + "mlp.down_proj.weight").shard(1, r, T).attach(att, P + "w_down")
    return Program(att, dtype, {"tp_size": T, "tp_rank": r, "ep": ep, "layers": cfg.num_hidden_layers,
                                "vocab_start": r * (cfg.vocab_size // T) if T > 1 else 0})


class SafetensorsReader:
    """Index over the *.safetensors shards of a checkpoint directory (lazy, sliceable reads)."""

    def __init__(self, path):
        from safetensors import safe_open
        self.path = Path(path)
        files = sorted(self.path.glob("*.safetensors")) if self.path.is_dir() else [self.path]
        if not files:
            raise FileNotFoundError(f"no .safetensors under {path}")
        self.handles = [safe_open(str(f), framework="pt", device="cpu") for f in files]
        self.where = {}
        for h in self.handles:
            for k in h.keys():
                self.where[k] = h

    def names(self) -> List[str]:
        return list(self.where)

    def get_slice(self, name):
        return self.where[name].get_slice(name)

    def get(self, name) -> torch.Tensor:
        return self.where[name].get_tensor(name)


def _eval(op: Op, reader, dtype) -> torch.Tensor:
    k = op.kind
    if k == "read":
        return reader.get(op.args["name"])
    if k in ("shard", "rows") and op.inputs[0].kind == "read":
        # slice straight out of the file: only this rank's bytes are read
        sl = reader.get_slice(op.inputs[0].args["name"])
        shape = sl.get_shape()
        if k == "rows":
            a, n = op.args["start"], op.args["count"]
            return sl[a:a + n]
        ax, r, wd = op.args["axis"], op.args["rank"], op.args["world"]
        n = shape[ax] // wd
        return sl[r * n:(r + 1) * n] if ax == 0 else sl[:, r * n:(r + 1) * n]
    xs = [_eval(i, reader, dtype) for i in op.inputs]
    if k == "shard":
        ax, r, wd = op.args["axis"], op.args["rank"], op.args["world"]
        n = xs[0].shape[ax] // wd
        return xs[0].narrow(ax, r * n, n)
    if k == "rows":
        return xs[0][op.args["start"]:op.args["start"] + op.args["count"]]
    if k == "concat":
        if xs[0].dtype == torch.float8_e4m3fn:
            return torch.cat([x.view(torch.uint8) for x in xs], dim=op.args["axis"]).view(torch.float8_e4m3fn)
        return torch.cat(xs, dim=op.args["axis"])
    if k == "interleave":
        a, b = xs
        f8 = a.dtype == torch.float8_e4m3fn
        if f8:
            a, b = a.view(torch.uint8), b.view(torch.uint8)
        y = torch.stack([a, b], dim=1).reshape(a.shape[0] * 2, *a.shape[1:])
        return y.view(torch.float8_e4m3fn) if f8 else y
    if k == "stack":
        return torch.stack(xs, dim=0)
    if k == "zeros_like":
        return torch.zeros_like(xs[0])
    if k == "squeeze":
        return xs[0].squeeze(op.args["dim"])
    if k == "float":
        return xs[0].float()
    if k == "add_scalar":
        return xs[0] + op.args["value"]
    if k == "transpose":
        return xs[0].transpose(op.args["a"], op.args["b"])
    if k == "mxfp4":
        return dequant_mxfp4(xs[0], xs[1])
    if k == "expand_rows":
        rows = reader.get_slice(op.args["like"]).get_shape()[0]       # ragged last block: cut to the weight's rows
        return xs[0].float().repeat_interleave(op.args["factor"], dim=0)[:rows]
    if k == "row_scales":
        n, kk = reader.get_slice(op.args["like"]).get_shape()
        sc = xs[0].float().reshape(-1)
        if sc.numel() not in (1, n):
            raise ValueError(f"weight scale of {sc.numel()} values for a weight of {n} rows")
        return sc.reshape(-1, 1).expand(n, -(-kk // 128)).contiguous()
    raise ValueError(f"unknown op {k}")


# ----------------------------------------------------------------------------- type check
class LoaderTypeError(ValueError):
    """The checkpoint's tensor shapes do not give the shapes the architecture needs."""


def infer_shape(op: Op, reader) -> Tuple[int, ...]:
    """Shape of an expression from the checkpoint's header alone (no tensor bytes are read)."""
    k = op.kind
    if k == "read":
        return tuple(reader.get_slice(op.args["name"]).get_shape())
    xs = [infer_shape(i, reader) for i in op.inputs]
    x = xs[0] if xs else ()
    if k == "shard":
        ax, wd = op.args["axis"], op.args["world"]
        if x[ax] % wd:
            raise LoaderTypeError(f"dimension {ax} of size {x[ax]} does not split over {wd} ranks")
        return x[:ax] + (x[ax] // wd,) + x[ax + 1:]
    if k == "rows":
        a, n = op.args["start"], op.args["count"]
        if a < 0 or a + n > x[0]:
            raise LoaderTypeError(f"rows {a}:{a + n} of a tensor with {x[0]} rows")
        return (n,) + x[1:]
    if k == "concat":
        ax = op.args["axis"]
        for y in xs[1:]:
            if len(y) != len(x) or any(y[d] != x[d] for d in range(len(x)) if d != ax):
                raise LoaderTypeError(f"concat of shapes {xs} along {ax}")
        return x[:ax] + (sum(y[ax] for y in xs),) + x[ax + 1:]
    if k == "interleave":
        if xs[0] != xs[1]:
            raise LoaderTypeError(f"interleave of shapes {xs[0]} and {xs[1]}")
        return (2 * x[0],) + x[1:]
    if k == "stack":
        if any(y != x for y in xs):
            raise LoaderTypeError(f"stack of unequal shapes {sorted(set(xs))}")
        return (len(xs),) + x
    if k in ("zeros_like", "float", "add_scalar"):
        return x
    if k == "squeeze":
        d = op.args["dim"]
        if x[d] != 1:
            raise LoaderTypeError(f"squeeze of dimension {d} with size {x[d]}")
        return x[:d] + x[d + 1:]
    if k == "transpose":
        a, b = op.args["a"], op.args["b"]
        y = list(x)
        y[a], y[b] = y[b], y[a]
        return tuple(y)
    if k == "mxfp4":                    # blocks [..., G, 16] packed nibbles -> [..., G * 32]
        return x[:-2] + (x[-2] * x[-1] * 2,)
    if k == "expand_rows":
        rows = reader.get_slice(op.args["like"]).get_shape()[0]
        return (min(x[0] * op.args["factor"], rows),) + x[1:]
    if k == "row_scales":
        n, kk = reader.get_slice(op.args["like"]).get_shape()
        cnt = 1
        for d in x:
            cnt *= d
        if cnt not in (1, n):
            raise LoaderTypeError(f"weight scale of shape {x} for a weight of {n} rows")
        return (n, -(-kk // 128))
    raise LoaderTypeError(f"unknown op {k}")


def expected_shapes(cfg: ModelConfig, tp_size: int = 1, ep: bool = False) -> Dict[str, Tuple[int, ...]]:
    """Runtime shapes of one rank's weights, per attachment key (layer keys without the `layers.N.` prefix)."""
    T, H, d = tp_size, cfg.hidden_size, cfg.head_dim
    hq = cfg.num_attention_heads // T
    hkv = max(1, cfg.num_key_value_heads // T)
    I = (cfg.moe_intermediate_size if cfg.is_moe else cfg.intermediate_size)
    E = cfg.num_experts
    el, il = (E // T, I) if (ep and T > 1) else (E, I // T)
    out = {"embed": (cfg.vocab_size, H), "final_norm": (H,), "lm_head": (cfg.vocab_size // T, H),
           "ln1": (H,), "ln2": (H,), "ln3": (H,), "ln_pa": (H,), "ln_pf": (H,), "wqkv": ((hq + 2 * hkv) * d, H), "wo": (H, hq * d),
           "bqkv": ((hq + 2 * hkv) * d,), "bo": (H,), "sinks": (hq,),
           "w_gate_up": (2 * cfg.intermediate_size // T, H), "w_down": (H, cfg.intermediate_size // T),
           "router": (E, H), "router_bias": (E,), "experts_gate_up": (el, 2 * il, H), "experts_down": (el, H, il),
           "experts_gate_up_bias": (el, 2 * il), "experts_down_bias": (el, H),
           "shared_gate_up": (2 * cfg.shared_expert_intermediate_size // T, H),
           "shared_down": (H, cfg.shared_expert_intermediate_size // T), "shared_gate": (1, H)}
    if cfg.mamba_layers:
        hm = cfg.mamba_num_heads
        out.update({"w_mamba_in": (cfg.mamba_in_features, H), "mamba_conv": (cfg.mamba_conv_channels, 4),
                    "mamba_conv_bias": (cfg.mamba_conv_channels,), "mamba_A_log": (hm,), "mamba_dt_bias": (hm,),
                    "mamba_D": (hm,), "mamba_norm": (cfg.mamba_inner,), "w_mamba_out": (H, cfg.mamba_inner)})
    if cfg.linear_layers:
        hv, dv = cfg.linear_num_value_heads, cfg.linear_value_head_dim
        out.update({"w_gdn_in": (cfg.gdn_in_features, H), "gdn_conv": (cfg.gdn_conv_channels, cfg.linear_conv_kernel_dim),
                    "gdn_A_log": (hv,), "gdn_dt_bias": (hv,), "gdn_norm": (dv,), "w_gdn_out": (H, hv * dv)})
    return out


def typecheck_program(prog: Program, cfg: ModelConfig, reader) -> Dict[str, Tuple[int, ...]]:
    """Infer the shape of every attachment from the checkpoint's header and compare it with what the
    architecture needs on this rank; all mismatches are reported together, before any tensor is read.
    Returns the inferred shapes. Counterpart of the weight loader's type checker in the reference
    (driver/weight_loader/src/typecheck.rs)."""
    want = expected_shapes(cfg, prog.meta.get("tp_size", 1), prog.meta.get("ep", False))
    shapes, errors = {}, []
    for path, op in prog.attach.items():
        try:
            shapes[path] = infer_shape(op, reader)
        except LoaderTypeError as e:
            errors.append(f"{path}: {e}")
            continue
        key = path.split(".", 2)[2] if path.startswith("layers.") else path
        if key.endswith("@scale"):
            continue
        exp = want.get(key)
        if key in ("q_norm", "k_norm"):
            continue                               # per head or over all heads, by family
        if exp is not None and tuple(shapes[path]) != tuple(exp):
            errors.append(f"{path}: checkpoint gives {tuple(shapes[path])}, the architecture needs {tuple(exp)}")
    if errors:
        more = f" (and {len(errors) - 8} more)" if len(errors) > 8 else ""
        raise LoaderTypeError("checkpoint does not fit the configuration:\n  " + "\n  ".join(errors[:8]) + more)
    return shapes


def execute_program(prog: Program, reader, device="cpu") -> dict:
    """Materialise the runtime weight dict of this rank."""
    dtype = torch_dtype(prog.dtype)
    out = {"layers": [dict() for _ in range(prog.meta["layers"])]}
    scales = {}
    for path, op in prog.attach.items():
        t = _eval(op, reader, dtype)
        if path.endswith("@scale"):
            scales[path[:-len("@scale")]] = t.float().contiguous().to(device)
            continue
        if t.dtype != torch.float8_e4m3fn:
            t = t.to(dtype)
        t = t.contiguous().to(device)
        if path.startswith("layers."):
            _, li, key = path.split(".", 2)
            out["layers"][int(li)][key] = t
        else:
            out[path] = t
    if scales:
        from ..ops import Fp8Linear
        for path, sc in scales.items():
            _, li, key = path.split(".", 2)
            lw = out["layers"][int(li)]
            kb = (lw[key].shape[1] + 127) // 128
            # a column shard of the weight takes the matching columns of the scale grid
            lw[key] = Fp8Linear(lw[key], sc[:, :kb] if sc.shape[1] >= kb else sc)
    out["lm_head_vocab_start"] = prog.meta.get("vocab_start", 0)
    return out


# ----------------------------------------------------------------------------- materialised-weight cache
def _source_fingerprint(path: Path) -> str:
    """Identity of a checkpoint without reading its tensors: names, sizes and mtimes of its files."""
    import hashlib
    files = [path] if path.is_file() else sorted(f for f in path.iterdir()
                                                  if f.suffix in (".safetensors", ".gguf", ".json"))
    h = hashlib.blake2b(digest_size=16)
    for f in files:
        st = f.stat()
        h.update(f"{f.name}:{st.st_size}:{int(st.st_mtime_ns)};".encode())
    return h.hexdigest()


def _flatten(weights: dict) -> Tuple[dict, dict]:
    """Runtime weight dict -> (flat name -> tensor, JSON-able structure notes)."""
    from ..ops import Fp8Linear
    flat, notes = {}, {"layers": len(weights["layers"]), "scalars": {}, "fp8": []}
    def put(name, v):
        if isinstance(v, Fp8Linear):
            flat[name + "@w8"], flat[name + "@scale"] = v.w8.view(torch.uint8), v.scale
            notes["fp8"].append(name)
        elif torch.is_tensor(v):
            flat[name] = v
        else:
            notes["scalars"][name] = v
    for k, v in weights.items():
        if k != "layers":
            put(k, v)
    for li, lw in enumerate(weights["layers"]):
        for k, v in lw.items():
            put(f"layers.{li}.{k}", v)
    return flat, notes


def _unflatten(flat: dict, notes: dict, device) -> dict:
    from ..ops import Fp8Linear
    out = {"layers": [dict() for _ in range(notes["layers"])]}
    def slot(name):
        if name.startswith("layers."):
            _, li, key = name.split(".", 2)
            return out["layers"][int(li)], key
        return out, name
    fp8 = set(notes["fp8"])
    for name, t in flat.items():
        base = name.rsplit("@", 1)[0]
        if base in fp8:
            continue
        d, key = slot(name)
        d[key] = t.to(device)
    for name in fp8:
        d, key = slot(name)
        d[key] = Fp8Linear(flat[name + "@w8"].view(torch.float8_e4m3fn).to(device), flat[name + "@scale"].to(device))
    for name, v in notes["scalars"].items():
        d, key = slot(name)
        d[key] = v
    return out


def weight_cache_dir() -> Optional[Path]:
    d = os.environ.get("PIE_WEIGHT_CACHE_DIR", "")
    return Path(d).expanduser() if d else None


def _cached_load(path: Path, prog: "Program", reader, device):
    """`execute_program` through the materialised-weight cache (opt-in: PIE_WEIGHT_CACHE_DIR). The
    cache key covers the source files (names, sizes, mtimes) and the whole storage program, so a
    different shard plan, dtype or fusion gets its own entry. Entries are one safetensors file per
    rank, written to a temporary name and renamed, with the key stored inside and checked on load.
    Counterpart of the reference's weight artifact cache (driver/cuda/src/model/weight_artifact_cache.hpp:1-24,
    opt-in through PIE_CUDA_WEIGHT_CACHE_DIR there)."""
    cdir = weight_cache_dir()
    if cdir is None:
        return execute_program(prog, reader, device)
    import hashlib
    from safetensors import safe_open
    from safetensors.torch import save_file
    key = hashlib.blake2b((_source_fingerprint(path) + program_to_json(prog)).encode(), digest_size=16).hexdigest()
    entry = cdir / f"{key}.safetensors"
    if entry.exists():
        try:
            with safe_open(str(entry), framework="pt", device="cpu") as f:
                meta = f.metadata() or {}
                if meta.get("key") == key:
                    flat = {k: f.get_tensor(k) for k in f.keys()}
                    return _unflatten(flat, json.loads(meta["notes"]), device)
        except Exception:  # noqa: BLE001 - a damaged entry is rebuilt
            pass
    weights = execute_program(prog, reader, device)
    try:
        cdir.mkdir(parents=True, exist_ok=True)
        flat, notes = _flatten(weights)
        tmp = entry.with_suffix(f".tmp{os.getpid()}")
        save_file({k: v.detach().cpu().contiguous() for k, v in flat.items()}, str(tmp),
                  metadata={"key": key, "notes": json.dumps(notes)})
        os.replace(tmp, entry)
    except Exception:  # noqa: BLE001 - the cache is an optimisation: never fail a load over it
        pass
    return weights


def load_checkpoint(path, device="cpu", tp_size: int = 1, tp_rank: int = 0, ep: bool = False,
                    dtype: Optional[str] = None):
    """config.json + safetensors, or one .gguf file (or a directory holding one and no
    safetensors) -> (ModelConfig, weights of this rank)."""
    p = Path(path)
    ggufs = [p] if p.is_file() and p.suffix == ".gguf" else \
        (sorted(p.glob("*.gguf")) if p.is_dir() and not list(p.glob("*.safetensors")) else [])
    if ggufs:
        from .gguf import GGUFReader
        reader = GGUFReader(ggufs[0])
        cfg = reader.config()
        prog = compile_program(cfg, reader.names(), tp_size, tp_rank, ep, dtype or cfg.dtype)
        typecheck_program(prog, cfg, reader)
        return cfg, _cached_load(ggufs[0], prog, reader, device)
    cfg = ModelConfig.from_path(path)
    reader = SafetensorsReader(path)
    prog = compile_program(cfg, reader.names(), tp_size, tp_rank, ep, dtype or cfg.dtype)
    typecheck_program(prog, cfg, reader)
    return cfg, _cached_load(p, prog, reader, device)


def export_hf_checkpoint(cfg: ModelConfig, weights: dict, path) -> None:
    """Write unsharded runtime weights back out under Hugging Face names (tests, tooling)."""
    from safetensors.torch import save_file
    p = Path(path)
    p.mkdir(parents=True, exist_ok=True)
    d, hq, hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    ungain = (lambda g: g.float() - 1.0) if cfg.norm_plus_one else (lambda g: g)      # Gemma stores (gain - 1)
    t: Dict[str, torch.Tensor] = {"model.embed_tokens.weight": weights["embed"], "model.norm.weight": ungain(weights["final_norm"])}
    if not cfg.tie_word_embeddings:
        t["lm_head.weight"] = weights["lm_head"]
    for li, lw in enumerate(weights["layers"]):
        L = f"model.layers.{li}."
        if "w_mamba_in" in lw:
            X = L + "mixer."
            t[X + "in_proj.weight"], t[X + "conv1d.weight"] = lw["w_mamba_in"], lw["mamba_conv"].unsqueeze(1)
            t[X + "conv1d.bias"], t[X + "A_log"], t[X + "dt_bias"], t[X + "D"] = (
                lw["mamba_conv_bias"], lw["mamba_A_log"], lw["mamba_dt_bias"], lw["mamba_D"])
            t[X + "norm.weight"], t[X + "out_proj.weight"] = lw["mamba_norm"], lw["w_mamba_out"]
            t[L + "input_layernorm.weight"], t[L + "post_attention_layernorm.weight"] = lw["ln1"], lw["ln2"]
            t[L + "mlp.gate_proj.weight"], t[L + "mlp.up_proj.weight"] = lw["w_gate_up"][0::2], lw["w_gate_up"][1::2]
            t[L + "mlp.down_proj.weight"] = lw["w_down"]
            continue
        if "w_gdn_in" in lw:
            X = L + "linear_attn."
            hk, hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
            dk, dv, rep = cfg.linear_key_head_dim, cfg.linear_value_head_dim, hv // hk
            q, k, v, z, b, a = lw["w_gdn_in"].split([hk * dk, hk * dk, hv * dv, hv * dv, hv, hv], 0)
            grp = lambda x, n: x.reshape(hk, n, -1)
            t[X + "in_proj_qkvz.weight"] = torch.cat([grp(q, dk), grp(k, dk), grp(v, rep * dv), grp(z, rep * dv)], 1
                                                     ).reshape(-1, cfg.hidden_size)
            t[X + "in_proj_ba.weight"] = torch.cat([grp(b, rep), grp(a, rep)], 1).reshape(-1, cfg.hidden_size)
            t[X + "conv1d.weight"] = lw["gdn_conv"].unsqueeze(1)
            t[X + "A_log"], t[X + "dt_bias"] = lw["gdn_A_log"], lw["gdn_dt_bias"]
            t[X + "norm.weight"], t[X + "out_proj.weight"] = lw["gdn_norm"], lw["w_gdn_out"]
            t[L + "input_layernorm.weight"], t[L + "post_attention_layernorm.weight"] = lw["ln1"], lw["ln2"]
            t[L + "mlp.gate_proj.weight"], t[L + "mlp.up_proj.weight"] = lw["w_gate_up"][0::2], lw["w_gate_up"][1::2]
            t[L + "mlp.down_proj.weight"] = lw["w_down"]
            continue
        if "ln_pa" in lw:
            t[L + "input_layernorm.weight"], t[L + "post_attention_layernorm.weight"] = ungain(lw["ln1"]), ungain(lw["ln_pa"])
            t[L + "pre_feedforward_layernorm.weight"], t[L + "post_feedforward_layernorm.weight"] = ungain(lw["ln2"]), ungain(lw["ln_pf"])
        elif "ln3" in lw:
            t[L + "post_attention_layernorm.weight"], t[L + "post_feedforward_layernorm.weight"] = lw["ln2"], lw["ln3"]
        else:
            t[L + "input_layernorm.weight"], t[L + "post_attention_layernorm.weight"] = lw["ln1"], lw["ln2"]
        q, k, v = lw["wqkv"].split([hq * d, hkv * d, hkv * d], 0)
        if cfg.model_type == "phi3":          # Phi-3 checkpoints store q, k, v rows in one tensor
            t[L + "self_attn.qkv_proj.weight"] = lw["wqkv"]
        else:
            t[L + "self_attn.q_proj.weight"], t[L + "self_attn.k_proj.weight"], t[L + "self_attn.v_proj.weight"] = q, k, v
        t[L + "self_attn.o_proj.weight"] = lw["wo"]
        if "bqkv" in lw:
            bq, bk, bv = lw["bqkv"].split([hq * d, hkv * d, hkv * d], 0)
            t[L + "self_attn.q_proj.bias"], t[L + "self_attn.k_proj.bias"], t[L + "self_attn.v_proj.bias"] = bq, bk, bv
        if "q_norm" in lw:
            t[L + "self_attn.q_norm.weight"], t[L + "self_attn.k_norm.weight"] = ungain(lw["q_norm"]), ungain(lw["k_norm"])
        if "bo" in lw:
            t[L + "self_attn.o_proj.bias"] = lw["bo"]
        if "sinks" in lw:
            t[L + "self_attn.sinks"] = lw["sinks"]
        if "experts_gate_up_bias" in lw:
            t[L + "mlp.router.weight"], t[L + "mlp.router.bias"] = lw["router"], lw["router_bias"]
            t[L + "mlp.experts.gate_up_proj"] = lw["experts_gate_up"].transpose(1, 2)
            t[L + "mlp.experts.down_proj"] = lw["experts_down"].transpose(1, 2)
            t[L + "mlp.experts.gate_up_proj_bias"] = lw["experts_gate_up_bias"]
            t[L + "mlp.experts.down_proj_bias"] = lw["experts_down_bias"]
        elif "experts_gate_up" in lw and cfg.model_type == "mixtral":
            # Mixtral's names: block_sparse_moe.gate, experts.N.w1 (gate) / w3 (up) / w2 (down)
            t[L + "block_sparse_moe.gate.weight"] = lw["router"]
            for e in range(lw["experts_gate_up"].shape[0]):
                gu, X = lw["experts_gate_up"][e], f"{L}block_sparse_moe.experts.{e}."
                t[X + "w1.weight"], t[X + "w3.weight"], t[X + "w2.weight"] = gu[0::2], gu[1::2], lw["experts_down"][e]
        elif "experts_gate_up" in lw:
            if "shared_gate_up" in lw:
                S = L + "mlp.shared_expert."
                t[S + "gate_proj.weight"], t[S + "up_proj.weight"] = lw["shared_gate_up"][0::2], lw["shared_gate_up"][1::2]
                t[S + "down_proj.weight"], t[L + "mlp.shared_expert_gate.weight"] = lw["shared_down"], lw["shared_gate"]
            t[L + "mlp.gate.weight"] = lw["router"]
            for e in range(lw["experts_gate_up"].shape[0]):
                gu = lw["experts_gate_up"][e]
                t[f"{L}mlp.experts.{e}.gate_proj.weight"], t[f"{L}mlp.experts.{e}.up_proj.weight"] = gu[0::2], gu[1::2]
                t[f"{L}mlp.experts.{e}.down_proj.weight"] = lw["experts_down"][e]
        elif cfg.model_type == "phi3":        # gate rows then up rows in one tensor
            t[L + "mlp.gate_up_proj.weight"] = torch.cat([lw["w_gate_up"][0::2], lw["w_gate_up"][1::2]], 0)
            t[L + "mlp.down_proj.weight"] = lw["w_down"]
        else:
            t[L + "mlp.gate_proj.weight"], t[L + "mlp.up_proj.weight"] = lw["w_gate_up"][0::2], lw["w_gate_up"][1::2]
            t[L + "mlp.down_proj.weight"] = lw["w_down"]
    save_file({k: v.contiguous().cpu() for k, v in t.items()}, str(p / "model.safetensors"))
    hf = {"model_type": cfg.model_type, "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
          "num_hidden_layers": cfg.num_hidden_layers, "num_attention_heads": hq, "num_key_value_heads": hkv,
          "head_dim": d, "vocab_size": cfg.vocab_size, "rms_norm_eps": cfg.rms_norm_eps, "rope_theta": cfg.rope_theta,
          "tie_word_embeddings": cfg.tie_word_embeddings, "torch_dtype": cfg.dtype, "attention_bias": cfg.attention_bias,
          "max_position_embeddings": cfg.max_position_embeddings}
    if cfg.model_type == "phi3":
        hf.update(pad_token_id=0, bos_token_id=1, eos_token_id=2)
    if cfg.sandwich_norm:
        hf.update(layer_types=cfg.layer_types, sliding_window=cfg.sliding_window,
                  query_pre_attn_scalar=int(cfg.query_pre_attn_scalar or cfg.head_dim),
                  hidden_activation="gelu_pytorch_tanh", attn_logit_softcapping=cfg.attn_softcap or None,
                  final_logit_softcapping=cfg.final_softcap or None, rope_scaling=cfg.rope_scaling)
        if cfg.rope_local_theta:
            hf.update(rope_local_base_freq=cfg.rope_local_theta)
    if cfg.model_type == "mixtral":
        hf.update(num_local_experts=cfg.num_experts, num_experts_per_tok=cfg.num_experts_per_tok,
                  intermediate_size=cfg.moe_intermediate_size)
    elif cfg.model_type == "gpt_oss":
        hf.update(num_local_experts=cfg.num_experts, num_experts_per_tok=cfg.num_experts_per_tok,
                  sliding_window=cfg.sliding_window, layer_types=cfg.layer_types, swiglu_limit=cfg.swiglu_limit,
                  rope_scaling=cfg.rope_scaling)
    elif cfg.mamba_layers:
        hf.update(layer_types=cfg.layer_types, mamba_num_heads=cfg.mamba_num_heads, mamba_head_dim=cfg.mamba_head_dim,
                  ssm_state_size=cfg.ssm_state_size, mamba_n_groups=cfg.mamba_n_groups,
                  mamba_norm_grouped=cfg.mamba_norm_grouped)
    elif cfg.linear_layers:
        hf.update(layer_types=cfg.layer_types, linear_num_key_heads=cfg.linear_num_key_heads,
                  linear_num_value_heads=cfg.linear_num_value_heads, linear_key_head_dim=cfg.linear_key_head_dim,
                  linear_value_head_dim=cfg.linear_value_head_dim, linear_conv_kernel_dim=cfg.linear_conv_kernel_dim)
    elif cfg.is_moe:
        hf.update(num_experts=cfg.num_experts, num_experts_per_tok=cfg.num_experts_per_tok,
                  moe_intermediate_size=cfg.moe_intermediate_size, norm_topk_prob=cfg.norm_topk_prob)
        if cfg.shared_expert_intermediate_size:
            hf.update(shared_expert_intermediate_size=cfg.shared_expert_intermediate_size, decoder_sparse_step=1, mlp_only_layers=[])
    (p / "config.json").write_text(json.dumps(hf))
