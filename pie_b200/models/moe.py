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


def gpt_oss_glu(gu: torch.Tensor, limit: float) -> torch.Tensor:
    """GPT-OSS expert activation on interleaved (gate, up) columns: gate clamped from above, up
    clamped to +-limit, (up + 1) * gate * sigmoid(1.702 * gate)
    (the reference's gpt_oss_glu kernel: driver/cuda/src/kernels/swiglu.cu)."""
    gate = gu[..., 0::2].float().clamp(max=limit)
    up = gu[..., 1::2].float().clamp(-limit, limit)
    return (up + 1.0) * gate * torch.sigmoid(1.702 * gate)


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
    logits = xf @ lw["router"].float().t()
    biased = "experts_gate_up_bias" in lw
    if "router_bias" in lw:
        logits = logits + lw["router_bias"].float()
    w, ids = route(cfg, logits)
    out = torch.zeros_like(xf)
    for e in range(lw["experts_gate_up"].shape[0]):
        sel = (ids == e)
        tok = sel.any(-1).nonzero()[:, 0]
        if tok.numel() == 0:
            continue
        gu = xf[tok] @ lw["experts_gate_up"][e].float().t()
        if biased:
            act = gpt_oss_glu(gu + lw["experts_gate_up_bias"][e].float(), cfg.swiglu_limit)
            y = act @ lw["experts_down"][e].float().t() + lw["experts_down_bias"][e].float()
        else:
            act = torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]
            y = act @ lw["experts_down"][e].float().t()
        out[tok] += y * (w[tok] * sel[tok]).sum(-1, keepdim=True)
    if "shared_gate_up" in lw:
        gu = xf @ lw["shared_gate_up"].float().t()
        sh = (torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]) @ lw["shared_down"].float().t()
        out = out + torch.sigmoid(xf @ lw["shared_gate"].float().t()) * sh
    return out


def _buffers(model, n: int, lw: dict, device) -> "ops.MoeBuffers":
    """Scratch for up to n tokens, grown in powers of two and kept on the model (fixed addresses
    let the block be captured in CUDA graphs)."""
    cap = 1 << max(0, (max(n, 1) - 1).bit_length())
    buf = getattr(model, "_moe_buf", None)
    e, n2, hdim = lw["experts_gate_up"].shape
    if buf is None or buf.n < cap or buf.I != n2 // 2 or buf.E != e:
        buf = ops.MoeBuffers(cap, hdim, n2 // 2, e, model.cfg.num_experts_per_tok, device)
        model._moe_buf = buf
    return buf


def moe_block(model, x: torch.Tensor, lw: dict, h: torch.Tensor) -> torch.Tensor:
    """h + MoE(x). x is the normalised hidden state [N, H].

    GPU: router GEMM -> route/align/permute kernels -> grouped tcgen05 GEMMs (SwiGLU fused into the
    first) -> weighted combine with the residual; no host synchronisation, graph-safe.
    Under tensor parallelism without EP the experts are sharded on their intermediate dimension
    (the reference's scheme) and the partial outputs are summed across ranks."""
    cfg, par = model.cfg, model.par
    if cfg.moe_style == "gpt_oss":
        return _moe_block_biased(model, x, lw, h)
    if par.tp_size > 1 and par.ep:
        # NCCL baseline of expert parallelism: every rank evaluates its own experts on all tokens
        logits = model._gemm(x, lw["router"]) if x.is_cuda else torch.matmul(x, lw["router"].t())
        e_local = lw["experts_gate_up"].shape[0]
        buf = _buffers(model, x.shape[0], lw, x.device)
        part = ops.moe_experts(x, logits, lw["experts_gate_up"], lw["experts_down"], cfg.num_experts_per_tok,
                               cfg.norm_topk_prob, buf, e_lo=par.tp_rank * e_local)
        return h + par.comm.all_reduce(part)
    if x.is_cuda:
        logits = model._gemm(x, lw["router"]) if lw["router"].shape[0] % 8 == 0 \
            else torch.matmul(x, lw["router"].t())
        buf = _buffers(model, x.shape[0], lw, x.device)
        if par.tp_size > 1:
            part = ops.moe_experts(x, logits, lw["experts_gate_up"], lw["experts_down"], cfg.num_experts_per_tok,
                                   cfg.norm_topk_prob, buf)
            return h + par.comm.all_reduce(part)
        return ops.moe_experts(x, logits, lw["experts_gate_up"], lw["experts_down"], cfg.num_experts_per_tok,
                               cfg.norm_topk_prob, buf, residual=h)
    w, ids = route(cfg, torch.matmul(x, lw["router"].t()))
    n, k = ids.shape
    flat = ids.reshape(-1)
    order = torch.argsort(flat, stable=True)
    tok = order // k
    counts = torch.bincount(flat, minlength=lw["experts_gate_up"].shape[0])
    xs = x[tok]
    ys = torch.empty(xs.shape[0], x.shape[1], dtype=x.dtype, device=x.device)
    start = 0
    for e, c in enumerate(counts.tolist()):
        if c:
            act = model._gemm(xs[start:start + c], lw["experts_gate_up"][e], swiglu=True)
            ys[start:start + c] = model._gemm(act, lw["experts_down"][e])
        start += c
    wflat = w.reshape(-1)[order].to(torch.float32)
    out = torch.zeros(n, x.shape[1], dtype=torch.float32, device=x.device)
    out.index_add_(0, tok, ys.float() * wflat[:, None])
    return h + out.to(x.dtype)


def _moe_block_biased(model, x: torch.Tensor, lw: dict, h: torch.Tensor) -> torch.Tensor:
    """GPT-OSS experts: router bias, per-expert biases on both projections and the clamped GLU.
    GPU: the same route / align / permute / grouped tcgen05 GEMM / combine kernels as the SwiGLU
    block, with the first GEMM storing gate and up unactivated and the biases and the activation
    applied to the expert-sorted rows in between (row -> expert through the tile table); static
    shapes, no host synchronisation. CPU: the dense formula."""
    cfg, par = model.cfg, model.par
    if par.tp_size > 1 and par.ep:
        raise NotImplementedError("GPT-OSS experts under expert parallelism")
    if not x.is_cuda:
        if par.tp_size > 1:
            raise NotImplementedError("GPT-OSS experts under tensor parallelism on the CPU path")
        return h + moe_reference(cfg, x, lw).to(x.dtype)
    k = cfg.num_experts_per_tok
    n = x.shape[0]
    logits = torch.matmul(x, lw["router"].t()) + lw["router_bias"]
    buf = _buffers(model, n, lw, x.device)
    mt = ops.moe_max_mtiles(n, k, buf.E)
    ops.moe_route(logits, k, cfg.norm_topk_prob, buf, 0)
    ops.moe_align(buf, mt)
    ops.moe_permute(x, buf)
    rows = mt * 128
    gu = getattr(model, "_moe_gu", None)
    if gu is None or gu.shape[0] < rows or gu.shape[1] != 2 * buf.I:
        gu = torch.empty(max(rows, buf.xs.shape[0]), 2 * buf.I, dtype=x.dtype, device=x.device)
        model._moe_gu = gu
    ops.grouped_gemm(buf.xs, lw["experts_gate_up"], buf.tile_expert, gu, mt, ops.EPI_STORE)
    if x.dtype == torch.bfloat16 and gu.is_contiguous() and buf.act.is_contiguous():
        ops.moe_bias_glu(gu, lw["experts_gate_up_bias"], buf.tile_expert, buf.act, mt, cfg.swiglu_limit)
        ops.grouped_gemm(buf.act, lw["experts_down"], buf.tile_expert, buf.ys, mt, ops.EPI_STORE)
        ops.moe_row_bias(buf.ys, lw["experts_down_bias"], buf.tile_expert, mt)
    else:
        row_expert = buf.tile_expert[:mt].clamp(min=0).long().repeat_interleave(128)       # unused tiles: any expert
        act = gpt_oss_glu(gu[:rows] + lw["experts_gate_up_bias"][row_expert], cfg.swiglu_limit)
        buf.act[:rows] = act.to(x.dtype)
        ops.grouped_gemm(buf.act, lw["experts_down"], buf.tile_expert, buf.ys, mt, ops.EPI_STORE)
        buf.ys[:rows] += lw["experts_down_bias"][row_expert]
    if par.tp_size > 1:
        # experts sharded on their intermediate dimension: partial sums over ranks, then the residual
        return h + par.comm.all_reduce(ops.moe_combine(buf, n, None))
    return ops.moe_combine(buf, n, h)


def moe_block_tp(model, lw: dict, n: int) -> None:
    """MoE block of the fused tensor-parallel forward. The normalised activations of all n tokens
    are already on every rank (the all-gather push is the dispatch); each rank routes all tokens,
    runs its own experts (expert parallelism) or its intermediate-dimension slice of every expert,
    and scatters its partial output rows to the row owners by peer stores (the combine), where the
    following reduce+norm kernel sums them with the residual."""
    cfg, par = model.cfg, model.par
    comm = par.comm
    x = comm.wait_gathered(n)
    logits = model._gemm(x, lw["router"])
    buf = _buffers(model, n, lw, x.device)
    e_local = lw["experts_gate_up"].shape[0]
    e_lo = par.tp_rank * e_local if par.ep else 0
    ops.moe_experts(x, logits, lw["experts_gate_up"], lw["experts_down"], cfg.num_experts_per_tok,
                    cfg.norm_topk_prob, buf, e_lo=e_lo, rs=(comm.tp_blob, comm.rows_per_rank(n)))
