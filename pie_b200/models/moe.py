"""Mixture-of-experts block (Qwen3-MoE / Mixtral style: softmax router, top-k, SwiGLU experts).

`moe_block` is the runtime path. On one GPU (or with experts sharded on their intermediate
dimension under tensor parallelism, the reference's scheme:
driver/cuda/src/model/qwen3_5_moe_forward.cpp:1144-1153) tokens are sorted by expert and each
expert's segment goes through the GEMM kernels; with expert parallelism the dispatch/combine
all-to-all of :mod:`pie_b200.parallel` moves token rows between ranks.
Router semantics (softmax over all experts, top-k, optional renormalisation) follow
driver/cuda/src/kernels/topk_softmax.cu:19.
"""
from __future__ import annotations

import torch

from .. import ops
from .config import ModelConfig


def route(cfg: ModelConfig, logits: torch.Tensor):
    """Router: softmax over experts, top-k, renormalise. Returns (weights fp32 [N,k], ids [N,k])."""
    probs = torch.softmax(logits.float(), dim=-1)
    w, ids = torch.topk(probs, cfg.num_experts_per_tok, dim=-1)
    if cfg.norm_topk_prob:
        w = w / w.sum(-1, keepdim=True)
    return w, ids


def moe_reference(cfg: ModelConfig, x: torch.Tensor, lw: dict) -> torch.Tensor:
    """Dense fp32 oracle: every token through its top-k experts (full, unsharded experts)."""
    xf = x.float()
    w, ids = route(cfg, xf @ lw["router"].float().t())
    out = torch.zeros_like(xf)
    for e in range(lw["experts_gate_up"].shape[0]):
        sel = (ids == e)
        tok = sel.any(-1).nonzero()[:, 0]
        if tok.numel() == 0:
            continue
        gu = xf[tok] @ lw["experts_gate_up"][e].float().t()
        act = torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]
        y = act @ lw["experts_down"][e].float().t()
        out[tok] += y * (w[tok] * sel[tok]).sum(-1, keepdim=True)
    return out


def moe_block(model, x: torch.Tensor, lw: dict, h: torch.Tensor) -> torch.Tensor:
    """h + MoE(x). x is the normalised hidden state [N, H]."""
    cfg, par = model.cfg, model.par
    if par.tp_size > 1 and par.ep:
        return par.comm.moe_expert_parallel(model, x, lw, h)
    logits = model._gemm(x, lw["router"]) if x.is_cuda and lw["router"].shape[0] % 8 == 0 \
        else torch.matmul(x, lw["router"].t())
    w, ids = route(cfg, logits)
    n, k = ids.shape
    flat = ids.reshape(-1)
    order = torch.argsort(flat, stable=True)
    tok = (order // k).to(torch.int32)
    counts = torch.bincount(flat, minlength=lw["experts_gate_up"].shape[0])
    xs = ops.gather_rows(x, tok) if x.is_cuda else x[tok.long()]
    ys = torch.empty(xs.shape[0], x.shape[1], dtype=x.dtype, device=x.device)
    if x.is_cuda and hasattr(ops, "grouped_gemm"):
        ops.grouped_expert_mlp(xs, counts, lw["experts_gate_up"], lw["experts_down"], ys)
    else:
        start = 0
        for e, c in enumerate(counts.tolist()):
            if c:
                act = model._gemm(xs[start:start + c], lw["experts_gate_up"][e], swiglu=True)
                ys[start:start + c] = model._gemm(act, lw["experts_down"][e])
            start += c
    wflat = w.reshape(-1)[order].to(torch.float32)
    out = torch.zeros(n, x.shape[1], dtype=torch.float32, device=x.device)
    out.index_add_(0, tok.long(), ys.float() * wflat[:, None])
    out = out.to(x.dtype)
    if par.tp_size > 1:
        out = par.comm.all_reduce(out)
    return h + out
