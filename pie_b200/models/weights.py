"""Weight construction: random initialisation of a named architecture (benchmarks run on
random-init weights) and the runtime layout shared with the safetensors loader.

Runtime layout per layer (this rank's shard under tensor parallelism):
  wqkv       [(hq + 2*hkv) * d, H]   q, k, v rows of this rank's heads, fused
  wo         [H, hq * d]             row-parallel (input dim sharded)
  w_gate_up  [2 * I_local, H]        gate and up rows INTERLEAVED (row 2j = gate_j, 2j+1 = up_j)
                                     so that the GEMM epilogue can apply SwiGLU on adjacent columns
  w_down     [H, I_local]
  ln1, ln2   [H]; q_norm, k_norm [d] (Qwen3); bqkv (Qwen2)
  OLMo-2 (post-norm): no ln1; ln2 follows attention, ln3 follows the MLP; q_norm [hq*d], k_norm [hkv*d]
  Gemma-2/3 (sandwich norms): ln1 / ln2 before attention / MLP, ln_pa / ln_pf on their outputs before the
  residual add; gains hold the full multiplier (the loader adds the checkpoint's implicit 1)
MoE layers replace w_gate_up / w_down by router [E, H], experts_gate_up [E_local, 2*Im, H]
(interleaved) and experts_down [E_local, H, Im].

Sharding follows the reference's loader contract (q/k/v/gate/up column-parallel, o/down
row-parallel: driver/weight_loader/src/abi.rs:1901-1916; fused QKV / gate-up joins:
driver/weight_loader/src/abi.rs:718-810).
"""
from __future__ import annotations

import torch

from .config import ModelConfig


def torch_dtype(name: str):
    return {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}[
        str(name).replace("torch.", "")]


def interleave_rows(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I, H], [I, H] -> [2I, H] with rows g0, u0, g1, u1, ..."""
    return torch.stack([gate, up], dim=1).reshape(gate.shape[0] * 2, *gate.shape[1:])


def shard_rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = t.shape[0] // world
    return t[rank * n:(rank + 1) * n]


def shard_cols(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = t.shape[1] // world
    return t[:, rank * n:(rank + 1) * n]


def kv_head_range(cfg: ModelConfig, rank: int, world: int):
    """KV heads of a rank; heads are replicated when there are fewer KV heads than ranks."""
    if cfg.num_key_value_heads >= world:
        n = cfg.num_key_value_heads // world
        return rank * n, n
    return (rank * cfg.num_key_value_heads) // world, 1


class _Gen:
    """Deterministic per-tensor normal initialiser (independent of sharding)."""

    def __init__(self, seed: int, device, dtype, std: float):
        self.seed, self.device, self.dtype, self.std = seed, torch.device(device), dtype, std
        self.count = 0

    def normal(self, *shape, std=None):
        self.count += 1
        g = torch.Generator(device=self.device)
        g.manual_seed(self.seed * 1000003 + self.count)
        std = self.std if std is None else std
        n = 1
        for s in shape:
            n *= s
        if n > (1 << 28) and self.device.type == "cuda":
            out = torch.empty(shape, dtype=self.dtype, device=self.device)
            flat = out.view(-1)
            step = 1 << 27
            for i in range(0, n, step):
                m = min(step, n - i)
                flat[i:i + m] = (torch.randn(m, generator=g, device=self.device, dtype=torch.float32) * std).to(self.dtype)
            return out
        return (torch.randn(*shape, generator=g, device=self.device, dtype=torch.float32) * std).to(self.dtype)


def random_weights(cfg: ModelConfig, device="cpu", dtype=None, seed: int = 0, tp_size: int = 1,
                   tp_rank: int = 0, ep: bool = False, std: float = 0.02, router_std: float = 1.0) -> dict:
    """N(0, std) weights of architecture `cfg`, sharded for (tp_size, tp_rank).

    Every rank draws the same full tensors from the same per-tensor seeds and keeps its shard,
    so tp=1 and tp=N runs see the same model. With `ep` the experts are split whole across
    ranks (expert parallel) instead of sharded on their intermediate dimension.
    """
    dtype = dtype or torch_dtype(cfg.dtype)
    gen = _Gen(seed, device, dtype, std)
    H, d = cfg.hidden_size, cfg.head_dim
    hq, hkv = cfg.num_attention_heads, cfg.num_key_value_heads
    T, r = tp_size, tp_rank
    ones = lambda n: torch.ones(n, dtype=dtype, device=device)
    kv0, kvn = kv_head_range(cfg, r, T)
    w = {"layers": []}
    emb = gen.normal(cfg.vocab_size, H)
    w["embed"] = emb
    for li in range(cfg.num_hidden_layers):
        if cfg.is_mamba_layer(li):
            if T > 1:
                raise NotImplementedError("Mamba-2 layers under tensor parallelism")
            # Mamba-2 mixer: input projection (z | x B C | dt), depthwise short convolution with bias over x B C,
            # per-head decay (A_log), step bias (dt_bias) and skip (D), gated RMSNorm over the inner width, output projection
            Hm, C = cfg.mamba_num_heads, cfg.mamba_conv_channels
            lw = {"ln1": ones(H), "ln2": ones(H),
                  "w_mamba_in": gen.normal(cfg.mamba_in_features, H, std=0.05),
                  "mamba_conv": gen.normal(C, 4, std=0.3), "mamba_conv_bias": gen.normal(C, std=0.1),
                  "mamba_A_log": gen.normal(Hm, std=0.5).float(), "mamba_dt_bias": gen.normal(Hm, std=0.5).float(),
                  "mamba_D": (1 + gen.normal(Hm, std=0.2)).float(), "mamba_norm": 1 + gen.normal(cfg.mamba_inner, std=0.1),
                  "w_mamba_out": gen.normal(H, cfg.mamba_inner)}
            gate, up = gen.normal(cfg.intermediate_size, H), gen.normal(cfg.intermediate_size, H)
            lw["w_gate_up"] = interleave_rows(gate, up).contiguous()
            lw["w_down"] = gen.normal(H, cfg.intermediate_size)
            w["layers"].append(lw)
            continue
        if cfg.is_linear_layer(li):
            if T > 1:
                raise NotImplementedError("Gated DeltaNet layers under tensor parallelism")
            # Gated DeltaNet mixer: fused input projection (q | k | v | z | b | a), depthwise short convolution over
            # q | k | v, per-value-head decay (A_log, dt_bias), gated RMSNorm over the head dimension, output projection
            Hv, dv = cfg.linear_num_value_heads, cfg.linear_value_head_dim
            lw = {"ln1": ones(H), "ln2": ones(H),
                  "w_gdn_in": gen.normal(cfg.gdn_in_features, H, std=0.05),
                  "gdn_conv": gen.normal(cfg.gdn_conv_channels, cfg.linear_conv_kernel_dim, std=0.3),
                  "gdn_A_log": gen.normal(Hv, std=0.5).float(), "gdn_dt_bias": gen.normal(Hv, std=0.5).float(),
                  "gdn_norm": 1 + gen.normal(dv, std=0.1), "w_gdn_out": gen.normal(H, Hv * dv)}
            gate, up = gen.normal(cfg.intermediate_size, H), gen.normal(cfg.intermediate_size, H)
            lw["w_gate_up"] = interleave_rows(gate, up).contiguous()
            lw["w_down"] = gen.normal(H, cfg.intermediate_size)
            w["layers"].append(lw)
            continue
        if cfg.post_norm:
            # norm gains away from 1 so that a misplaced norm shows in the tests
            lw = {"ln2": 1 + gen.normal(H, std=0.1), "ln3": 1 + gen.normal(H, std=0.1)}
        elif cfg.sandwich_norm:
            lw = {k: 1 + gen.normal(H, std=0.1) for k in ("ln1", "ln_pa", "ln2", "ln_pf")}
        else:
            lw = {"ln1": ones(H), "ln2": ones(H)}
        wq, wk, wv = gen.normal(hq * d, H), gen.normal(hkv * d, H), gen.normal(hkv * d, H)
        lw["wqkv"] = torch.cat([shard_rows(wq, r, T), wk[kv0 * d:(kv0 + kvn) * d], wv[kv0 * d:(kv0 + kvn) * d]], 0).contiguous()
        del wq, wk, wv
        if cfg.attention_bias:
            b = gen.normal((hq + 2 * hkv) * d)
            bq, bk, bv = b[:hq * d], b[hq * d:(hq + hkv) * d], b[(hq + hkv) * d:]
            lw["bqkv"] = torch.cat([shard_rows(bq, r, T), bk[kv0 * d:(kv0 + kvn) * d], bv[kv0 * d:(kv0 + kvn) * d]]).contiguous()
        lw["wo"] = shard_cols(gen.normal(H, hq * d), r, T).contiguous()
        if cfg.o_bias:
            lw["bo"] = gen.normal(H)
        if cfg.attention_sinks:
            lw["sinks"] = shard_rows(gen.normal(hq, std=1.0), r, T).float().contiguous()
        if cfg.qk_norm and cfg.post_norm:
            # norms over all heads together: a rank keeps the gains of its own heads
            qn, kn = 1 + gen.normal(hq * d, std=0.1), 1 + gen.normal(hkv * d, std=0.1)
            lw["q_norm"], lw["k_norm"] = shard_rows(qn, r, T).contiguous(), kn[kv0 * d:(kv0 + kvn) * d].contiguous()
        elif cfg.qk_norm and cfg.sandwich_norm:
            lw["q_norm"], lw["k_norm"] = 1 + gen.normal(d, std=0.1), 1 + gen.normal(d, std=0.1)
        elif cfg.qk_norm:
            lw["q_norm"], lw["k_norm"] = ones(d), ones(d)
        if cfg.is_moe:
            E, Im = cfg.num_experts, cfg.moe_intermediate_size
            lw["router"] = gen.normal(E, H, std=router_std / H ** 0.5)
            gate, up, down = gen.normal(E, Im, H), gen.normal(E, Im, H), gen.normal(E, H, Im)
            if ep and T > 1:
                e0, en = r * (E // T), E // T
                gate, up, down = gate[e0:e0 + en], up[e0:e0 + en], down[e0:e0 + en]
            elif T > 1:
                s = Im // T
                gate, up, down = gate[:, r * s:(r + 1) * s], up[:, r * s:(r + 1) * s], down[:, :, r * s:(r + 1) * s]
            lw["experts_gate_up"] = torch.stack([gate, up], dim=2).reshape(gate.shape[0], 2 * gate.shape[1], H).contiguous()
            lw["experts_down"] = down.contiguous()
            del gate, up, down
            if cfg.shared_expert_intermediate_size:
                # the shared expert is a dense MLP: sharded like one under tensor parallelism (also with expert parallelism)
                Is = cfg.shared_expert_intermediate_size
                sg, su = shard_rows(gen.normal(Is, H), r, T), shard_rows(gen.normal(Is, H), r, T)
                lw["shared_gate_up"] = interleave_rows(sg, su).contiguous()
                lw["shared_down"] = shard_cols(gen.normal(H, Is), r, T).contiguous()
                lw["shared_gate"] = gen.normal(1, H, std=0.1)
            if cfg.moe_style == "gpt_oss":
                lw["router_bias"] = gen.normal(E, std=0.5)
                gub, db = gen.normal(E, 2 * Im, std=0.2), gen.normal(E, H, std=0.2)
                if T > 1:       # (gate, up) pairs follow their intermediate slice; the output bias lives on rank 0
                    gub = gub[:, r * 2 * (Im // T):(r + 1) * 2 * (Im // T)]
                    db = db if r == 0 else torch.zeros_like(db)
                lw["experts_gate_up_bias"], lw["experts_down_bias"] = gub.contiguous(), db
        else:
            I = cfg.intermediate_size
            gate, up = shard_rows(gen.normal(I, H), r, T), shard_rows(gen.normal(I, H), r, T)
            lw["w_gate_up"] = interleave_rows(gate, up).contiguous()
            del gate, up
            lw["w_down"] = shard_cols(gen.normal(H, I), r, T).contiguous()
        if cfg.quantization == "fp8_block":
            from ..ops import quantize_fp8_block
            for key in ("wqkv", "wo", "w_gate_up", "w_down"):
                if key in lw:
                    # interleaved gate/up rows come from two 128-row blocks: scale over 64-row pairs
                    lw[key] = quantize_fp8_block(lw[key].float(), 128)
        w["layers"].append(lw)
    w["final_norm"] = ones(H)
    if cfg.tie_word_embeddings:
        head = emb
    else:
        head = gen.normal(cfg.vocab_size, H)
    if T > 1:
        # vocabulary-sharded lm_head: every rank computes its slice of the logits
        head = shard_rows(head, r, T).contiguous()
    w["lm_head"] = head
    w["lm_head_vocab_start"] = r * (cfg.vocab_size // T) if T > 1 else 0
    return w


def weights_nbytes(w) -> int:
    total = 0
    seen = set()

    def visit(x):
        nonlocal total
        if hasattr(x, "w8"):
            visit(x.w8)
            visit(x.scale)
        elif isinstance(x, torch.Tensor):
            if x.data_ptr() not in seen:
                seen.add(x.data_ptr())
                total += x.numel() * x.element_size()
        elif isinstance(x, dict):
            for v in x.values():
                visit(v)
        elif isinstance(x, (list, tuple)):
            for v in x:
                visit(v)

    visit(w)
    return total


def dequantized(w):
    """Copy of a weight dict with every fp8 linear expanded to its float values (oracles, export)."""
    if hasattr(w, "w8"):
        return w.dequant(torch.float32)
    if isinstance(w, dict):
        return {k: dequantized(v) for k, v in w.items()}
    if isinstance(w, list):
        return [dequantized(v) for v in w]
    return w
