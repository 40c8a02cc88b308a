"""Plain PyTorch implementations of every op in :mod:`pie_b200.ops`.

They serve two purposes: the CPU path of the engine (the tiny fp32 plumbing model runs on
them) and the fp32 oracle that the numerics tests compare each CUDA kernel against.
All math is done in fp32 regardless of the storage dtype.
"""
from __future__ import annotations

import math

import torch


def embed(tokens, table, vocab_start=0):
    idx = tokens.long() - vocab_start
    ok = (idx >= 0) & (idx < table.shape[0])
    out = table[idx.clamp(0, table.shape[0] - 1)]
    return torch.where(ok[:, None], out, torch.zeros_like(out))


def rmsnorm(x, w, eps, w_offset=0.0):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + w_offset)
    return y.to(x.dtype)


def add_rmsnorm(delta, residual, w, eps, w_offset=0.0):
    """residual += delta (in place, rounded to the storage dtype); returns norm(residual)."""
    residual.copy_((residual.float() + delta.float()).to(residual.dtype))
    return rmsnorm(residual, w, eps, w_offset)


def swiglu(gate_up):
    inter = gate_up.shape[-1] // 2
    g, u = gate_up[..., :inter].float(), gate_up[..., inter:].float()
    return (torch.nn.functional.silu(g) * u).to(gate_up.dtype)


def swiglu_interleaved(gate_up):
    g, u = gate_up[..., 0::2].float(), gate_up[..., 1::2].float()
    return (torch.nn.functional.silu(g) * u).to(gate_up.dtype)


def rope_inv_freq(head_dim, theta, scaling=None, device="cpu"):
    """Inverse frequencies of rotate-half RoPE, with optional Llama-3, linear or YaRN frequency
    scaling (`rope_scaling` of a Hugging Face config).

    Mirrors the frequency tables of the reference (driver/cuda/src/kernels/rope.cu:55-160).
    """
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    kind = (scaling or {}).get("rope_type", (scaling or {}).get("type"))
    if kind == "linear":
        inv = inv / float(scaling.get("factor", 1.0))
    elif kind == "yarn":
        factor = float(scaling.get("factor", 1.0))
        orig = float(scaling.get("original_max_position_embeddings", 4096))
        fast, slow = float(scaling.get("beta_fast", 32.0)), float(scaling.get("beta_slow", 1.0))

        def corr_dim(rot):      # dimension whose wavelength makes `rot` turns over the original context
            return head_dim * math.log(orig / (rot * 2 * math.pi)) / (2 * math.log(theta))

        low, high = corr_dim(fast), corr_dim(slow)
        if scaling.get("truncate", True):       # GPT-OSS keeps the fractional bounds
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, head_dim - 1)
        ramp = ((torch.arange(head_dim // 2, dtype=torch.float64) - low) / max(high - low, 1e-3)).clamp(0, 1)
        keep = 1.0 - ramp       # 1: high-frequency dimensions keep their frequency, 0: interpolated by `factor`
        inv = inv / factor * (1 - keep) + inv * keep
    if kind == "llama3":
        factor = scaling.get("factor", 8.0)
        lo = scaling.get("low_freq_factor", 1.0)
        hi = scaling.get("high_freq_factor", 4.0)
        old = scaling.get("original_max_position_embeddings", 8192)
        wavelen = 2 * math.pi / inv
        smooth = ((old / wavelen) - lo) / (hi - lo)
        scaled = torch.where(wavelen > old / lo, inv / factor, inv)
        mid = (wavelen <= old / lo) & (wavelen >= old / hi)
        inv = torch.where(mid, (1 - smooth) * inv / factor + smooth * inv, scaled)
    return inv.float().to(device)


def rope_attention_factor(scaling=None) -> float:
    """YaRN scales cos and sin by a factor (0.1 ln(factor) + 1 unless the config names one): the
    attention logits grow by its square, which callers fold into the softmax scale."""
    if not scaling or scaling.get("rope_type", scaling.get("type")) != "yarn":
        return 1.0
    if scaling.get("attention_factor"):
        return float(scaling["attention_factor"])
    f = float(scaling.get("factor", 1.0))
    return 0.1 * math.log(f) + 1.0 if f > 1 else 1.0


def _rope(x, positions, inv_freq):
    # x [N, H, D] fp32; rotate-half convention
    d = x.shape[-1]
    ang = positions.float()[:, None] * inv_freq.float()[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    lo, hi = x[..., : d // 2], x[..., d // 2:]
    return torch.cat([lo * cos - hi * sin, hi * cos + lo * sin], dim=-1)


def qk_norm_rope_kvwrite(qkv, positions, slots, inv_freq, q_norm_w, k_norm_w, kv_layer, hq, hkv,
                         head_dim, page_size, eps):
    """Split packed qkv, per-head RMSNorm (optional) + RoPE on q and k, scatter k/v into pages.

    kv_layer is [pages, 2, hkv, page_size, head_dim]; slots[t] = page*page_size + offset
    (negative: skip the write). Returns q [N, hq, head_dim].
    """
    n = qkv.shape[0]
    dt = qkv.dtype
    q = qkv[:, : hq * head_dim].reshape(n, hq, head_dim).float()
    k = qkv[:, hq * head_dim:(hq + hkv) * head_dim].reshape(n, hkv, head_dim).float()
    v = qkv[:, (hq + hkv) * head_dim:(hq + 2 * hkv) * head_dim].reshape(n, hkv, head_dim)
    if q_norm_w is not None:
        q = (q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_norm_w.float()).to(dt).float()
    if k_norm_w is not None:
        k = (k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_norm_w.float()).to(dt).float()
    q = _rope(q, positions, inv_freq).to(dt)
    k = _rope(k, positions, inv_freq).to(dt)
    ok = slots >= 0
    s = slots[ok].long()
    page, off = s // page_size, s % page_size
    kv_layer[page, 0, :, off, :] = k[ok]
    kv_layer[page, 1, :, off, :] = v[ok]
    return q


def gather_kv(kv_layer, pages, kv_len):
    """K, V of one request as [hkv, kv_len, D] from its page list."""
    blk = kv_layer[pages.long()]  # [np, 2, hkv, page, D]
    np_, _, hkv, page, d = blk.shape
    k = blk[:, 0].permute(1, 0, 2, 3).reshape(hkv, np_ * page, d)[:, :kv_len]
    v = blk[:, 1].permute(1, 0, 2, 3).reshape(hkv, np_ * page, d)[:, :kv_len]
    return k, v


def paged_attention(q, kv_layer, qo_indptr, kv_page_indptr, page_indices, kv_lens, sm_scale,
                    masks=None, window_left=-1, return_lse=False, sinks=None):
    """Ragged paged attention. q [N, hq, D]; masks: optional list (per request) of bool
    [qo_len, kv_len] tensors or None (causal: query i sees kv < kv_len - qo_len + i + 1).
    sinks [hq]: per-head logits that join the softmax denominator without a value row."""
    n, hq, d = q.shape
    hkv = kv_layer.shape[2]
    g = hq // hkv
    out = torch.zeros_like(q)
    lse = torch.full((n, hq), float("-inf"), dtype=torch.float32, device=q.device)
    nreq = len(kv_lens)
    for r in range(nreq):
        q0, q1 = int(qo_indptr[r]), int(qo_indptr[r + 1])
        ql = q1 - q0
        kl = int(kv_lens[r])
        if ql == 0:
            continue
        pages = page_indices[int(kv_page_indptr[r]):int(kv_page_indptr[r + 1])]
        k, v = gather_kv(kv_layer, pages, kl)
        kf = k.float().repeat_interleave(g, dim=0)  # [hq, kl, D]
        vf = v.float().repeat_interleave(g, dim=0)
        qf = q[q0:q1].float().permute(1, 0, 2)      # [hq, ql, D]
        s = torch.einsum("hqd,hkd->hqk", qf, kf) * sm_scale
        if masks is not None and masks[r] is not None:
            allow = masks[r].to(q.device)[:, :kl]
        else:
            qi = torch.arange(ql, device=q.device)[:, None]
            kj = torch.arange(kl, device=q.device)[None, :]
            allow = kj < (kl - ql + qi + 1)
            if window_left >= 0:
                allow = allow & (kj >= (kl - ql + qi - window_left))
        s = s.masked_fill(~allow[None], float("-inf"))
        m = s.amax(-1, keepdim=True)
        m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
        p = (s - m).exp()
        l = p.sum(-1, keepdim=True)
        if sinks is not None:
            l = torch.where(l > 0, l + (sinks.float().to(q.device)[:, None, None] - m).exp(), l)
        o = torch.einsum("hqk,hkd->hqd", p, vf) / l.clamp_min(1e-30)
        o = torch.where(l > 0, o, torch.zeros_like(o))
        out[q0:q1] = o.permute(1, 0, 2).to(q.dtype)
        lse[q0:q1] = torch.where(l > 0, m + l.log(), torch.full_like(l, float("-inf")))[..., 0].T
    return (out, lse) if return_lse else out


def kept_set(logits_row, temperature, top_k, top_p, min_p, allowed=None):
    """Boolean mask of the tokens a (top-k AND top-p AND min-p) filter keeps; fp32 math."""
    x = logits_row.float()
    if allowed is not None:
        x = x.masked_fill(~allowed, float("-inf"))
    probs = torch.softmax(x / max(temperature, 1e-6), dim=-1)
    keep = torch.isfinite(x)
    order = torch.argsort(probs, descending=True, stable=True)
    sp = probs[order]
    if 0 < top_k < x.numel():
        kth = sp[top_k - 1]
        keep &= probs >= kth
    if top_p < 1.0:
        cum = torch.cumsum(sp, 0)
        # smallest prefix whose mass reaches top_p
        npfx = int((cum < top_p).sum().item()) + 1
        thr = sp[min(npfx, sp.numel()) - 1]
        keep &= probs >= thr
    if min_p > 0:
        keep &= probs >= min_p * probs.max()
    return keep


def sample(logits, temperature, top_k, top_p, min_p, seeds, masks=None, generator=None):
    """Reference sampler: exact filters, then a multinomial draw (torch RNG, so only the
    distribution, not the stream, matches the CUDA kernel). temperature<=0 -> arg-max."""
    rows = logits.shape[0]
    out = torch.empty(rows, dtype=torch.int32)
    for r in range(rows):
        allowed = None if masks is None or masks[r] is None else masks[r]
        x = logits[r].float()
        if allowed is not None:
            x = x.masked_fill(~allowed, float("-inf"))
        t = float(temperature[r])
        if t <= 0:
            out[r] = int(torch.argmax(x))
            continue
        keep = kept_set(logits[r], t, int(top_k[r]), float(top_p[r]), float(min_p[r]), allowed)
        p = torch.softmax(x / t, -1) * keep
        g = generator or torch.Generator().manual_seed(int(seeds[r]) & 0x7FFFFFFF)
        out[r] = int(torch.multinomial(p / p.sum(), 1, generator=g))
    return out


def row_stats(logits):
    x = logits.float()
    m = x.amax(-1)
    lse = torch.logsumexp(x, -1)
    p = torch.softmax(x, -1)
    ent = -(p * torch.log_softmax(x, -1)).sum(-1)
    return torch.stack([m, lse, ent], dim=-1)


def brle_to_bool(runs, nbits, tail_value=False):
    """Decode one BRLE vector (even entries = run of False, odd = run of True)."""
    out = torch.full((nbits,), bool(tail_value), dtype=torch.bool)
    pos = 0
    for i, n in enumerate(runs):
        if pos >= nbits:
            break
        end = min(nbits, pos + int(n))
        out[pos:end] = bool(i & 1)
        pos = end
    return out


def gemm(x, w, residual=None):
    y = x.float() @ w.float().t()
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)
