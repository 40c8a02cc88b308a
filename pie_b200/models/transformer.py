"""Decoder-only transformer over paged KV: Llama-2/3, Mistral, Qwen2, Qwen3 (dense) and
Qwen3-MoE / Mixtral-style mixture-of-experts, tensor-parallel (and expert-parallel) aware.

One forward = embed -> L x [RMSNorm -> fused QKV GEMM -> per-head q/k RMSNorm + RoPE + paged
KV write -> paged attention -> o_proj GEMM (+residual | +TP reduce) -> RMSNorm -> gate/up GEMM
with SwiGLU epilogue (or MoE block) -> down GEMM (+residual | +TP reduce)] -> final norm ->
lm_head on the rows that need logits.

Behavioural counterpart: the reference's `llama_like_forward_paged`
(driver/cuda/src/model/llama_like.cpp:239-851) and its MoE block
(driver/cuda/src/model/qwen3_5_moe_forward.cpp:1128-1721). The KV write slot is the tail
of the context (positions only feed RoPE), as in driver/cuda/src/kernels/kv_paged.cu:52-62.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..ops import reference
from ..driver.lora import apply_lora
from .config import ModelConfig


@dataclass
class ForwardInputs:
    """Device-resident inputs of one forward pass (one 'fire')."""
    tokens: torch.Tensor          # int32 [N]
    positions: torch.Tensor       # int32 [N]
    slots: torch.Tensor           # int32 [N]  KV slot (page*page_size+offset) of each new token
    attn: object                  # ops.DecodePlan | ops.PrefillPlan | ops.AttnBatch (CPU)
    attn_num_pages: Optional[int] = None   # page references of this batch (prefill plans; the slab segment is larger)
    logit_rows: Optional[torch.Tensor] = None   # int32 rows of the hidden state that need logits
    rs: Optional[object] = None   # driver.recurrent.RecurrentInputs for models with Gated DeltaNet layers
    is_decode: bool = False
    lora: Optional[list] = None   # [(LoraAdapter, int64 token rows)] for requests bound to an adapter
    media: Optional[list] = None  # [(encoder output [rows, H], first source row, first token row, count)]


class ParallelContext:
    """Tensor/expert-parallel placement of this rank. Collectives live in pie_b200.parallel."""

    def __init__(self, tp_size: int = 1, tp_rank: int = 0, comm=None, ep: bool = False):
        self.tp_size, self.tp_rank, self.comm, self.ep = tp_size, tp_rank, comm, ep


class Transformer:
    def __init__(self, cfg: ModelConfig, weights: dict, device, dtype, par: Optional[ParallelContext] = None,
                 gemm_backend: str = "tcgen05"):
        self.cfg, self.w, self.device, self.dtype = cfg, weights, torch.device(device), dtype
        self.par = par or ParallelContext()
        t = self.par.tp_size
        self.hq = cfg.num_attention_heads // t
        self.hkv = max(1, cfg.num_key_value_heads // t)
        self.d = cfg.head_dim
        self.sm_scale = reference.rope_attention_factor(cfg.rope_scaling) ** 2 / math.sqrt(cfg.query_pre_attn_scalar or cfg.head_dim)
        self.inv_freq = reference.rope_inv_freq(cfg.head_dim, cfg.rope_theta, cfg.rope_scaling, self.device)
        # Gemma-3: sliding-window layers rotate with their own, unscaled base
        self.inv_freq_local = reference.rope_inv_freq(cfg.head_dim, cfg.rope_local_theta, None, self.device) \
            if cfg.rope_local_theta else None
        self.gemm_backend = gemm_backend if self.device.type == "cuda" else "torch"
        self.vocab_local = weights["lm_head"].shape[0] * (self.par.tp_size if self.par.comm is not None else 1)
        # fp8 KV pages: per-(token, head) scales [layers, pages, 2, hkv, page] set by the driver, else None
        self.kv_scale = None

    # ------------------------------------------------------------------ linear algebra
    def _gemm(self, x, w, residual=None, swiglu=False):
        if isinstance(w, ops.Fp8Linear):
            epi = ops.EPI_SWIGLU if swiglu else (ops.EPI_RESIDUAL if residual is not None else ops.EPI_STORE)
            if self.gemm_backend == "tcgen05" or not x.is_cuda:
                return ops.gemm_fp8w(x, w, residual=residual, epilogue=epi)
            w = w.dequant(x.dtype)      # library path: expand, then cuBLAS (the reference's scheme)
        if self.gemm_backend == "tcgen05" and x.dtype == torch.bfloat16:
            epi = ops.EPI_SWIGLU if swiglu else (ops.EPI_RESIDUAL if residual is not None else ops.EPI_STORE)
            return ops.gemm(x, w, residual=residual, epilogue=epi)
        # library path (cuBLAS through torch): the baseline the tcgen05 kernel is measured against
        y = torch.matmul(x, w.t())
        if swiglu:
            return reference.swiglu_interleaved(y) if not y.is_cuda else _swiglu_interleaved_cuda(y)
        if residual is not None:
            y = y + residual
        return y

    # ------------------------------------------------------------------ layers
    def _attention(self, q, kv_layer, fi: ForwardInputs, li: int = 0, lw: Optional[dict] = None):
        """Layer `li`'s attention: its own sliding window where layers differ (the plan then covers
        the whole range and the kernels mask), and its attention sinks where the model has them."""
        wl = self.cfg.layer_window_left(li) if self.cfg.layer_types is not None else None
        sinks = lw.get("sinks") if lw is not None else None
        cap = self.cfg.attn_softcap
        if not q.is_cuda:
            return ops.paged_attention_cpu(q, kv_layer, fi.attn, self.sm_scale, window_left=wl, sinks=sinks, softcap=cap)
        sl2 = None
        if sinks is not None:
            sl2 = lw.get("sinks_log2")
            if sl2 is None:
                sl2 = lw["sinks_log2"] = (sinks.float() * 1.4426950408889634).contiguous()
        ks = self.kv_scale[li] if self.kv_scale is not None else None
        if fi.is_decode:
            return ops.paged_decode_attention(q, kv_layer, fi.attn, self.sm_scale, window_left=wl, sinks_log2=sl2,
                                              kv_scale=ks, softcap=cap)
        if ks is not None:
            # prefill over fp8 pages: expand the pages this batch reads to bf16 and address them compactly
            from dataclasses import replace as _replace
            pages = fi.attn.page_indices[:fi.attn_num_pages] if getattr(fi, "attn_num_pages", None) else fi.attn.page_indices
            dense = ops.dequant_kv_pages(kv_layer, ks, pages)
            plan = _replace(fi.attn, page_indices=torch.arange(pages.numel(), dtype=torch.int32, device=pages.device))
            return ops.paged_prefill_attention(q, dense, plan, self.sm_scale, window_left=wl, sinks_log2=sl2)
        return ops.paged_prefill_attention(q, kv_layer, fi.attn, self.sm_scale, window_left=wl, sinks_log2=sl2, softcap=cap)

    def _glu(self, x, lw):
        """act(gate) * up of the fused, interleaved gate / up projection: SiLU in the GEMM's epilogue, GELU after it."""
        if self.cfg.hidden_act == "silu":
            return self._gemm(x, lw["w_gate_up"], swiglu=True)
        return ops.glu_interleaved(self._gemm(x, lw["w_gate_up"]), self.cfg.hidden_act)

    def _mlp(self, x, lw, h):
        return self._row_parallel(self._glu(x, lw), lw["w_down"], h)

    def _rope_table(self, li: int):
        if self.inv_freq_local is not None and self.cfg.layer_window_left(li) >= 0:
            return self.inv_freq_local
        return self.inv_freq

    def _row_parallel(self, a, w, h):
        """h + a @ w.T (a @ w.T when h is None), summed over the tensor-parallel group."""
        if self.par.tp_size == 1:
            return self._gemm(a, w, residual=h)
        y = self.par.comm.gemm_allreduce(a, w, self)
        return y if h is None else y.add_(h)

    def _moe(self, x, lw, h):
        from .moe import moe_block
        h = moe_block(self, x, lw, h)
        if "shared_gate_up" in lw:
            # shared expert: a dense SwiGLU MLP for every token, scaled per token by sigmoid(x . shared_gate)
            sh = self._row_parallel(self._gemm(x, lw["shared_gate_up"], swiglu=True), lw["shared_down"], None)
            gate = torch.sigmoid(torch.matmul(x, lw["shared_gate"].t()).float())
            h = h + (sh.float() * gate).to(h.dtype)
        return h

    def _fused_tp(self) -> bool:
        return self.par.tp_size > 1 and self.par.comm is not None and getattr(self.par.comm, "fused", False) \
            and self.device.type == "cuda" and not self.cfg.post_norm and not self.cfg.sandwich_norm \
            and self.cfg.model_type != "gpt_oss" and not self.cfg.shared_expert_intermediate_size

    def _forward_hidden_tp(self, fi: ForwardInputs, kv_cache) -> torch.Tensor:
        """Tensor-parallel forward over the fused kernels: the residual stream is row-sharded,
        every row-parallel GEMM scatters its partial rows to their owners from its epilogue, the
        owner reduces + normalises + pushes, and the next column-parallel GEMM gates its loads
        on the push flags. Returns the final-normalised hidden states of all rows."""
        cfg, w, comm = self.cfg, self.w, self.par.comm
        page_size = kv_cache.shape[4]
        n = fi.tokens.shape[0]
        layers = w["layers"]
        comm.embed_norm_push(fi.tokens, w["embed"], layers[0]["ln1"], cfg.rms_norm_eps, n)
        for li, lw in enumerate(layers):
            qkv = comm.gemm_gated(lw["wqkv"], n)
            q = ops.qk_norm_rope_kvwrite(qkv, fi.positions, fi.slots, self.inv_freq, lw.get("q_norm"),
                                         lw.get("k_norm"), kv_cache[li], self.hq, self.hkv, self.d,
                                         page_size, cfg.rms_norm_eps,
                                         kv_scale=self.kv_scale[li] if self.kv_scale is not None else None,
                                         bias=lw.get("bqkv"))
            a = self._attention(q, kv_cache[li], fi, li)
            comm.gemm_rs(a.reshape(n, self.hq * self.d), lw["wo"], n)
            comm.reduce_norm_push(lw["ln2"], cfg.rms_norm_eps, n)
            if "experts_gate_up" in lw:
                from .moe import moe_block_tp
                moe_block_tp(self, lw, n)
            else:
                act = comm.gemm_gated(lw["w_gate_up"], n, swiglu=True)
                comm.gemm_rs(act, lw["w_down"], n)
            nxt = layers[li + 1]["ln1"] if li + 1 < len(layers) else w["final_norm"]
            comm.reduce_norm_push(nxt, cfg.rms_norm_eps, n)
        return comm.wait_gathered(n)

    def forward_hidden(self, fi: ForwardInputs, kv_cache) -> torch.Tensor:
        if fi.media and self.par.tp_size > 1:
            raise NotImplementedError("media inputs under tensor parallelism")
        if self._fused_tp():
            return self._forward_hidden_tp(fi, kv_cache)
        cfg, w = self.cfg, self.w
        page_size = kv_cache.shape[4]
        if self.par.tp_size > 1 and w.get("embed_sharded", False):
            h = ops.embed(fi.tokens, w["embed"], vocab_start=w["embed_vocab_start"])
            h = self.par.comm.all_reduce(h)
        else:
            h = ops.embed(fi.tokens, w["embed"])
        if cfg.embed_scale != 1.0:
            # the factor is rounded to the activation dtype first, as the checkpoints' own code does
            h = h * torch.tensor(cfg.embed_scale, dtype=h.dtype).item()
        for feats, src, dst, cnt in fi.media or ():
            # rows of an encoded image / video take the place of their placeholder tokens' embeddings
            h[dst:dst + cnt] = feats[src:src + cnt].to(h.dtype)
        n = h.shape[0]
        for li in range(cfg.num_hidden_layers):
            lw = w["layers"][li]
            post = cfg.post_norm
            if "w_mamba_in" in lw:
                # Mamba-2 layer: state-space mixer, state in the recurrent-state cache
                x = ops.rmsnorm(h, lw["ln1"], cfg.rms_norm_eps)
                mix = self._gemm(x, lw["w_mamba_in"])
                o = ops.mamba2_mixer(mix, lw, cfg, fi.rs, fi.rs.layer_index[li])
                h = self._gemm(o, lw["w_mamba_out"], residual=h)
                h = self._mlp(ops.rmsnorm(h, lw["ln2"], cfg.rms_norm_eps), lw, h)
                continue
            if "w_gdn_in" in lw:
                # Gated DeltaNet layer: the mixer replaces attention, its state lives in the recurrent-state cache
                x = ops.rmsnorm(h, lw["ln1"], cfg.rms_norm_eps)
                mix = self._gemm(x, lw["w_gdn_in"])
                o = ops.gdn_mixer(mix, lw, cfg, fi.rs, fi.rs.layer_index[li])
                h = self._gemm(o, lw["w_gdn_out"], residual=h)
                h = self._mlp(ops.rmsnorm(h, lw["ln2"], cfg.rms_norm_eps), lw, h)
                continue
            x = h if post else ops.rmsnorm(h, lw["ln1"], cfg.rms_norm_eps)
            qkv = self._gemm(x, lw["wqkv"])
            qn, kn = lw.get("q_norm"), lw.get("k_norm")
            # the projection's bias rides in the RoPE / KV-write kernel unless something reads the packed rows before it
            bias = lw.get("bqkv")
            if bias is not None and (fi.lora or (qn is not None and qn.numel() != self.d)):
                qkv, bias = qkv + bias, None
            if fi.lora:
                qkv = apply_lora(fi.lora, li, "qkv", x, qkv)
            if qn is not None and qn.numel() != self.d:
                # OLMo-2: RMSNorm over the whole q and k projections (all heads together)
                qs, ks = self.hq * self.d, self.hkv * self.d
                if self.par.tp_size > 1:
                    # a rank holds some of the heads: the mean of squares needs every rank's share
                    if cfg.num_key_value_heads < self.par.tp_size:
                        raise NotImplementedError("q/k norms over all heads with replicated KV heads")
                    qf, kf = qkv[:, :qs].float(), qkv[:, qs:qs + ks].float()
                    ss = torch.stack([qf.pow(2).sum(-1), kf.pow(2).sum(-1)], dim=1)
                    ss = self.par.comm.all_reduce(ss)
                    rq = torch.rsqrt(ss[:, 0:1] / cfg.q_size + cfg.rms_norm_eps)
                    rk = torch.rsqrt(ss[:, 1:2] / cfg.kv_size + cfg.rms_norm_eps)
                    qkv[:, :qs] = (qf * rq * qn.float()).to(qkv.dtype)
                    qkv[:, qs:qs + ks] = (kf * rk * kn.float()).to(qkv.dtype)
                else:
                    qkv[:, :qs] = ops.rmsnorm(qkv[:, :qs].contiguous(), qn, cfg.rms_norm_eps)
                    qkv[:, qs:qs + ks] = ops.rmsnorm(qkv[:, qs:qs + ks].contiguous(), kn, cfg.rms_norm_eps)
                qn = kn = None
            q = ops.qk_norm_rope_kvwrite(qkv, fi.positions, fi.slots, self._rope_table(li), qn, kn, kv_cache[li],
                                         self.hq, self.hkv, self.d, page_size, cfg.rms_norm_eps,
                                         kv_scale=self.kv_scale[li] if self.kv_scale is not None else None, bias=bias)
            a = self._attention(q, kv_cache[li], fi, li, lw).reshape(n, self.hq * self.d)
            if cfg.sandwich_norm:
                # Gemma-2/3: both sublayers are normalised on the way in and on the way out
                o = self._row_parallel(a, lw["wo"], None)
                if fi.lora:
                    o = apply_lora(fi.lora, li, "o", a, o)
                h = h + ops.rmsnorm(o, lw["ln_pa"], cfg.rms_norm_eps)
                m = self._row_parallel(self._glu(ops.rmsnorm(h, lw["ln2"], cfg.rms_norm_eps), lw), lw["w_down"], None)
                h = h + ops.rmsnorm(m, lw["ln_pf"], cfg.rms_norm_eps)
                continue
            if post:
                if "experts_gate_up" in lw:
                    raise NotImplementedError("post-norm blocks with experts")
                o = self._row_parallel(a, lw["wo"], None)
                if fi.lora:
                    o = apply_lora(fi.lora, li, "o", a, o)
                h = h + ops.rmsnorm(o, lw["ln2"], cfg.rms_norm_eps)
                h = h + ops.rmsnorm(self._row_parallel(self._glu(h, lw), lw["w_down"], None), lw["ln3"], cfg.rms_norm_eps)
                continue
            h = self._row_parallel(a, lw["wo"], h)
            if "bo" in lw:
                h = h + lw["bo"]
            if fi.lora:
                h = apply_lora(fi.lora, li, "o", a, h)
            x = ops.rmsnorm(h, lw["ln2"], cfg.rms_norm_eps)
            if "experts_gate_up" in lw:
                h = self._moe(x, lw, h)
            else:
                h = self._mlp(x, lw, h)
        return h

    def logits(self, h: torch.Tensor, fi: ForwardInputs) -> torch.Tensor:
        """lm_head on the requested rows only ('compact logit rows')."""
        rows = h if fi.logit_rows is None else ops.gather_rows(h, fi.logit_rows)
        if self._fused_tp():
            # h is already final-normalised and gathered; every rank computes its vocabulary slice and
            # keeps it: token samplers run sharded (TPComm.sample_sharded), only probes gather
            return self.par.comm.gemm_gated(self.w["lm_head"], rows.shape[0], x=rows)
        x = ops.rmsnorm(rows, self.w["final_norm"], self.cfg.rms_norm_eps)
        y = self._gemm(x, self.w["lm_head"])
        if self.par.tp_size > 1 and self.par.comm is not None:
            y = self.par.comm.all_gather_logits(y)
        if self.cfg.final_softcap:
            y = (torch.tanh(y.float() / self.cfg.final_softcap) * self.cfg.final_softcap).to(y.dtype)
        return y

    @property
    def sharded_logits(self) -> bool:
        """True when `logits` returns this rank's vocabulary slice [rows, V / tp] instead of [rows, V]."""
        return self._fused_tp()

    def forward(self, fi: ForwardInputs, kv_cache) -> torch.Tensor:
        return self.logits(self.forward_hidden(fi, kv_cache), fi)


def _swiglu_interleaved_cuda(y):
    g, u = y[..., 0::2], y[..., 1::2]
    return torch.nn.functional.silu(g) * u


def _dense_mamba2(cfg: ModelConfig, lw: dict, xn: torch.Tensor) -> torch.Tensor:
    """Mamba-2 mixer over one whole sequence from an empty state, head by head and token by token
    (independent of the cached, batched implementation it checks)."""
    hm, p, ns, g = cfg.mamba_num_heads, cfg.mamba_head_dim, cfg.ssm_state_size, cfg.mamba_n_groups
    inner, c = cfg.mamba_inner, cfg.mamba_conv_channels
    mix = xn @ lw["w_mamba_in"].float().t()
    t = mix.shape[0]
    pad = torch.cat([torch.zeros(3, c), mix[:, inner:inner + c]], 0)
    cw = lw["mamba_conv"].float()
    conv = torch.stack([(pad[i:i + 4] * cw.t()).sum(0) for i in range(t)]) + lw["mamba_conv_bias"].float()
    conv = conv * torch.sigmoid(conv)
    y = torch.zeros(t, inner)
    for h in range(hm):
        grp = h // (hm // g)
        a = -torch.exp(lw["mamba_A_log"].float()[h])
        state = torch.zeros(p, ns)
        for i in range(t):
            xv = conv[i, h * p:(h + 1) * p]
            bv = conv[i, inner + grp * ns:inner + (grp + 1) * ns]
            cv = conv[i, inner + g * ns + grp * ns:inner + g * ns + (grp + 1) * ns]
            dt = torch.nn.functional.softplus(mix[i, inner + c + h] + lw["mamba_dt_bias"].float()[h])
            state = state * torch.exp(dt * a) + dt * torch.outer(xv, bv)
            y[i, h * p:(h + 1) * p] = state @ cv + lw["mamba_D"].float()[h] * xv
    z = mix[:, :inner]
    y = y * (z * torch.sigmoid(z))
    ng = g if cfg.mamba_norm_grouped else 1
    yg = y.reshape(t, ng, inner // ng)
    yg = yg / torch.sqrt((yg * yg).mean(-1, keepdim=True) + cfg.rms_norm_eps)
    return yg.reshape(t, inner) * lw["mamba_norm"].float()


def _dense_gdn(cfg: ModelConfig, lw: dict, xn: torch.Tensor) -> torch.Tensor:
    """Gated DeltaNet over one whole sequence from an empty state, written token by token with explicit
    head loops (independent of the cached, batched implementation it checks)."""
    hk, hv, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    kk, c = cfg.linear_conv_kernel_dim, cfg.gdn_conv_channels
    mix = xn @ lw["w_gdn_in"].float().t()
    t = mix.shape[0]
    pad = torch.cat([torch.zeros(kk - 1, c), mix[:, :c]], 0)
    cw = lw["gdn_conv"].float()
    conv = torch.stack([(pad[i:i + kk] * cw.t()).sum(0) for i in range(t)])
    conv = conv * torch.sigmoid(conv)
    out = torch.zeros(t, hv * dv)
    for h in range(hv):
        kh = h // (hv // hk)
        state = torch.zeros(dk, dv)
        for i in range(t):
            q = conv[i, kh * dk:(kh + 1) * dk]
            k = conv[i, hk * dk + kh * dk:hk * dk + (kh + 1) * dk]
            v = conv[i, 2 * hk * dk + h * dv:2 * hk * dk + (h + 1) * dv]
            z = mix[i, c + h * dv:c + (h + 1) * dv]
            beta = torch.sigmoid(mix[i, c + hv * dv + h])
            g = -torch.exp(lw["gdn_A_log"].float()[h]) * torch.nn.functional.softplus(
                mix[i, c + hv * dv + hv + h] + lw["gdn_dt_bias"].float()[h])
            q = q / torch.sqrt((q * q).sum() + 1e-6) / math.sqrt(dk)
            k = k / torch.sqrt((k * k).sum() + 1e-6)
            state = state * torch.exp(g)
            delta = (v - k @ state) * beta
            state = state + torch.outer(k, delta)
            o = q @ state
            o = o / torch.sqrt((o * o).mean() + cfg.rms_norm_eps) * lw["gdn_norm"].float()
            out[i, h * dv:(h + 1) * dv] = o * z * torch.sigmoid(z)
    return out


def dense_reference_forward(cfg: ModelConfig, w: dict, tokens: torch.Tensor, embeds: Optional[dict] = None,
                            spans: Optional[list] = None) -> torch.Tensor:
    """Independent dense (non-paged) fp32 forward of the same weights for one sequence:
    RMSNorm -> QKV -> rotate-half RoPE -> causal attention -> SwiGLU. Returns logits [T, V].
    This is the token-for-token oracle of the paged engine path."""
    x = w["embed"].float()[tokens.long()] * cfg.embed_scale
    for row, vec in (embeds or {}).items():        # {token row: embedding} of media rows
        x[row] = vec.float()
    t = x.shape[0]
    pos = torch.arange(t)
    inv_global = reference.rope_inv_freq(cfg.head_dim, cfg.rope_theta, cfg.rope_scaling)
    inv_local = reference.rope_inv_freq(cfg.head_dim, cfg.rope_local_theta, None) if cfg.rope_local_theta else inv_global
    act = (lambda g: torch.nn.functional.gelu(g, approximate="tanh")) if cfg.hidden_act == "gelu_tanh" else torch.nn.functional.silu
    hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim

    def norm(v, g):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * g.float()

    for li, lw in enumerate(w["layers"]):
        if "w_mamba_in" in lw:
            x = x + _dense_mamba2(cfg, lw, norm(x, lw["ln1"])) @ lw["w_mamba_out"].float().t()
            gu = norm(x, lw["ln2"]) @ lw["w_gate_up"].float().t()
            x = x + (torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]) @ lw["w_down"].float().t()
            continue
        if "w_gdn_in" in lw:
            x = x + _dense_gdn(cfg, lw, norm(x, lw["ln1"])) @ lw["w_gdn_out"].float().t()
            gu = norm(x, lw["ln2"]) @ lw["w_gate_up"].float().t()
            x = x + (torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]) @ lw["w_down"].float().t()
            continue
        xn = x if cfg.post_norm else norm(x, lw["ln1"])
        qkv = xn @ lw["wqkv"].float().t()
        if "bqkv" in lw:
            qkv = qkv + lw["bqkv"].float()
        q = qkv[:, : hq * d].reshape(t, hq, d)
        k = qkv[:, hq * d:(hq + hkv) * d].reshape(t, hkv, d)
        v = qkv[:, (hq + hkv) * d:].reshape(t, hkv, d)
        if "q_norm" in lw and lw["q_norm"].numel() != d:       # over all heads together
            q = norm(q.reshape(t, hq * d), lw["q_norm"]).reshape(t, hq, d)
            k = norm(k.reshape(t, hkv * d), lw["k_norm"]).reshape(t, hkv, d)
        elif "q_norm" in lw:
            q, k = norm(q, lw["q_norm"]), norm(k, lw["k_norm"])
        inv = inv_local if cfg.layer_window_left(li) >= 0 else inv_global
        q, k = reference._rope(q, pos, inv), reference._rope(k, pos, inv)
        k = k.repeat_interleave(hq // hkv, dim=1)
        v = v.repeat_interleave(hq // hkv, dim=1)
        s = torch.einsum("qhd,khd->hqk", q, k) * (reference.rope_attention_factor(cfg.rope_scaling) ** 2
                                                  / math.sqrt(cfg.query_pre_attn_scalar or d))
        if cfg.attn_softcap:
            s = torch.tanh(s / cfg.attn_softcap) * cfg.attn_softcap
        future = torch.triu(torch.ones(t, t, dtype=torch.bool), 1)
        for a0, n0 in spans or ():          # [(first row, rows)]: rows of a span see every key up to the span's end
            future[a0:a0 + n0, :a0 + n0] = False
        s = s.masked_fill(future[None], float("-inf"))
        if cfg.layer_window_left(li) >= 0:       # a query sees itself and the sliding_window - 1 keys before it
            s = s.masked_fill(torch.tril(torch.ones(t, t, dtype=torch.bool), -cfg.sliding_window)[None], float("-inf"))
        if "sinks" in lw:       # a per-head extra logit that only takes probability mass
            s = torch.cat([s, lw["sinks"].float()[:, None, None].expand(hq, t, 1)], dim=-1)
            a = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1)[..., :t], v).reshape(t, hq * d)
        else:
            a = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(t, hq * d)
        if cfg.sandwich_norm:
            x = x + norm(a @ lw["wo"].float().t(), lw["ln_pa"])
            gu = norm(x, lw["ln2"]) @ lw["w_gate_up"].float().t()
            x = x + norm((act(gu[:, 0::2]) * gu[:, 1::2]) @ lw["w_down"].float().t(), lw["ln_pf"])
            continue
        if cfg.post_norm:
            x = x + norm(a @ lw["wo"].float().t(), lw["ln2"])
            gu = x @ lw["w_gate_up"].float().t()
            x = x + norm((act(gu[:, 0::2]) * gu[:, 1::2]) @ lw["w_down"].float().t(), lw["ln3"])
            continue
        x = x + a @ lw["wo"].float().t()
        if "bo" in lw:
            x = x + lw["bo"].float()
        xn = norm(x, lw["ln2"])
        if "experts_gate_up" in lw:
            from .moe import moe_reference
            x = x + moe_reference(cfg, xn, lw)
        else:
            gu = xn @ lw["w_gate_up"].float().t()
            x = x + (act(gu[:, 0::2]) * gu[:, 1::2]) @ lw["w_down"].float().t()
    y = norm(x, w["final_norm"]) @ w["lm_head"].float().t()
    return torch.tanh(y / cfg.final_softcap) * cfg.final_softcap if cfg.final_softcap else y
