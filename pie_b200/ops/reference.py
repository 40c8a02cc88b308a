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


def glu_interleaved(gate_up, act: str = "silu"):
    g, u = gate_up[..., 0::2].float(), gate_up[..., 1::2].float()
    a = torch.nn.functional.gelu(g, approximate="tanh") if act == "gelu_tanh" else torch.nn.functional.silu(g)
    return (a * u).to(gate_up.dtype)


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
                    masks=None, window_left=-1, return_lse=False, sinks=None, softcap=0.0):
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
        if softcap:         # Gemma-2: scores squashed into (-cap, cap) before masking
            s = torch.tanh(s / softcap) * softcap
        qi = torch.arange(ql, device=q.device)[:, None]
        kj = torch.arange(kl, device=q.device)[None, :]
        if masks is not None and masks[r] is not None:
            allow = masks[r].to(q.device)[:, :kl]
        else:
            allow = kj < (kl - ql + qi + 1)
        if window_left >= 0:        # a layer's window bounds the keys on the left under a custom mask too, as in the kernels
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


# ------------------------------------------------------------------ Gated DeltaNet (linear attention)
def gdn_mixer(mix, conv_w, a_log, dt_bias, norm_w, eps, hk, hv, dk, dv, qo_indptr, conv_state, rec_state, slots, reset):
    """Gated DeltaNet mixer over a ragged batch, state carried in per-slot caches (updated in place).

    `mix` [N, 2*hk*dk + 2*hv*dv + 2*hv] is the fused input projection q | k | v | z | b | a. Per request
    (rows qo_indptr[r]:qo_indptr[r+1], cache slot slots[r], state zeroed first when reset[r]):
      * causal depthwise convolution (kernel K) + SiLU over the q | k | v channels, continuing from the
        slot's last K-1 inputs (`conv_state` [S, C, K-1]);
      * per value head: q, k L2-normalised, q scaled by dk^-1/2; beta = sigmoid(b);
        g = -exp(A_log) * softplus(a + dt_bias); S <- S * exp(g); delta = (v - k^T S) * beta;
        S <- S + k (x) delta; o = q^T S   (`rec_state` [S, hv, dk, dv], fp32);
      * out = RMSNorm(o) * norm_w * silu(z) per head.
    Math of the reference's recurrent step (driver/cuda/src/kernels/gated_delta_net.cu, recurrent_step*).
    """
    n = mix.shape[0]
    c = 2 * hk * dk + hv * dv
    kk = conv_w.shape[1]
    x = mix.float()
    out = torch.zeros(n, hv * dv, dtype=torch.float32, device=mix.device)
    cw = conv_w.float()
    decay = -torch.exp(a_log.float())
    rep = hv // hk
    for r in range(len(qo_indptr) - 1):
        a0, a1 = int(qo_indptr[r]), int(qo_indptr[r + 1])
        if a1 <= a0:
            continue
        s = int(slots[r])
        if reset[r]:
            conv_state[s].zero_()
            rec_state[s].zero_()
        hist = torch.cat([conv_state[s].float().t(), x[a0:a1, :c]], dim=0)          # [K-1 + T, C]
        t = a1 - a0
        conv = sum(hist[j:j + t] * cw[:, j] for j in range(kk))                      # causal: taps end at the token
        conv = torch.nn.functional.silu(conv)
        conv_state[s].copy_(hist[-(kk - 1):].t().to(conv_state.dtype))
        q = conv[:, :hk * dk].reshape(t, hk, dk)
        k = conv[:, hk * dk:2 * hk * dk].reshape(t, hk, dk)
        v = conv[:, 2 * hk * dk:].reshape(t, hv, dv)
        z = x[a0:a1, c:c + hv * dv].reshape(t, hv, dv)
        b = x[a0:a1, c + hv * dv:c + hv * dv + hv]
        a = x[a0:a1, c + hv * dv + hv:]
        q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
        k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
        q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)      # key heads serve `rep` value heads
        beta = torch.sigmoid(b)
        g = decay * torch.nn.functional.softplus(a + dt_bias.float())
        st = rec_state[s].float()                                                     # [hv, dk, dv]
        o = torch.zeros(t, hv, dv, device=mix.device)
        for i in range(t):
            st = st * torch.exp(g[i])[:, None, None]
            kv = (st * k[i][:, :, None]).sum(1)
            delta = (v[i] - kv) * beta[i][:, None]
            st = st + k[i][:, :, None] * delta[:, None, :]
            o[i] = (st * q[i][:, :, None]).sum(1)
        rec_state[s].copy_(st)
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * norm_w.float()
        out[a0:a1] = (o * torch.nn.functional.silu(z)).reshape(t, hv * dv)
    return out.to(mix.dtype)


# ------------------------------------------------------------------ Mamba-2 (state-space duality) mixer
def mamba2_mixer(mix, conv_w, conv_b, a_log, dt_bias, d_skip, norm_w, eps, heads, head_dim, state, groups,
                 qo_indptr, conv_state, rec_state, slots, reset, norm_groups: int = 1):
    """Mamba-2 mixer over a ragged batch with per-slot state (updated in place).

    `mix` [N, z | x B C | dt]: z [heads*head_dim] gates the output, x B C go through the causal depthwise
    convolution (kernel K, bias, SiLU) continuing from the slot's last K-1 inputs, dt [heads].
    Per head h (group g = h // (heads / groups)), state S in R^{head_dim x state} (fp32):
        dt' = softplus(dt + dt_bias);  S <- S * exp(dt' * -exp(A_log)) + dt' * x (x) B_g;  y = S C_g + D * x
    out = RMSNorm(y * silu(z)) * norm_w, the norm over the whole inner width or per `norm_groups` slices of it.
    Math of the reference's Mamba-2 step kernels (driver/cuda/src/kernels/nemotron_h.cu, selective state update)."""
    n = mix.shape[0]
    inner, c = heads * head_dim, heads * head_dim + 2 * groups * state
    kk = conv_w.shape[1]
    x_all = mix.float()
    out = torch.zeros(n, inner, dtype=torch.float32, device=mix.device)
    cw, cb = conv_w.float(), conv_b.float()
    a = -torch.exp(a_log.float())
    hpg = heads // groups
    for r in range(len(qo_indptr) - 1):
        a0, a1 = int(qo_indptr[r]), int(qo_indptr[r + 1])
        if a1 <= a0:
            continue
        s = int(slots[r])
        if reset[r]:
            conv_state[s].zero_()
            rec_state[s].zero_()
        t = a1 - a0
        z = x_all[a0:a1, :inner]
        hist = torch.cat([conv_state[s].float().t(), x_all[a0:a1, inner:inner + c]], dim=0)
        conv = sum(hist[j:j + t] * cw[:, j] for j in range(kk)) + cb
        conv = torch.nn.functional.silu(conv)
        conv_state[s].copy_(hist[-(kk - 1):].t().to(conv_state.dtype))
        x = conv[:, :inner].reshape(t, heads, head_dim)
        bmat = conv[:, inner:inner + groups * state].reshape(t, groups, state).repeat_interleave(hpg, dim=1)
        cmat = conv[:, inner + groups * state:].reshape(t, groups, state).repeat_interleave(hpg, dim=1)
        dt = torch.nn.functional.softplus(x_all[a0:a1, inner + c:] + dt_bias.float())      # [t, heads]
        st = rec_state[s].float()                                                           # [heads, head_dim, state]
        y = torch.zeros(t, heads, head_dim, device=mix.device)
        for i in range(t):
            st = st * torch.exp(dt[i] * a)[:, None, None] + (dt[i][:, None] * x[i])[:, :, None] * bmat[i][:, None, :]
            y[i] = (st * cmat[i][:, None, :]).sum(-1) + d_skip.float()[:, None] * x[i]
        rec_state[s].copy_(st)
        y = y.reshape(t, inner) * torch.nn.functional.silu(z)
        yg = y.reshape(t, norm_groups, inner // norm_groups)
        yg = yg * torch.rsqrt(yg.pow(2).mean(-1, keepdim=True) + eps)
        out[a0:a1] = yg.reshape(t, inner) * norm_w.float()
    return out.to(mix.dtype)
