"""Model-forward ops. GPU tensors go to the hand-written sm_100a kernels
(``csrc/kernels``), CPU tensors to the PyTorch reference in :mod:`.reference`.

There is no silent fallback on a GPU: if the kernel library is missing, a call with CUDA
tensors raises :class:`pie_b200.ops._lib.KernelLibraryError`.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from . import _lib, reference
from ._lib import check, fn, ptr, stream_ptr

EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2

_NUM_SMS = {}


def num_sms(device=None) -> int:
    dev = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    if dev not in _NUM_SMS:
        _NUM_SMS[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _NUM_SMS[dev]


# --------------------------------------------------------------------------- status word
_STATUS = {}


def kernel_status(device=None) -> torch.Tensor:
    """Device int32 that kernels with bounded waits set when a wait runs out (0 = healthy)."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    if dev not in _STATUS:
        _STATUS[dev] = torch.zeros(8, dtype=torch.int32, device=f"cuda:{dev}")   # [0] status, [2..7] wait counters
        with torch.cuda.device(dev):       # kernels without a status argument report here too
            check(fn("pie_set_status_word")(ptr(_STATUS[dev])), "set_status_word")
    return _STATUS[dev]


BOUNDS_TABLES = ["tokens", "positions", "kv_page_indices", "kv_last_page_lens", "kv_slots", "logit_rows"]


def check_kernel_status(device=None) -> None:
    words = kernel_status(device)[:2].tolist()
    st = int(words[0])
    if st != 0:
        kernel_status(device).zero_()
        if st == 5:
            code, pos = (int(words[1]) >> 24) & 0xFF, int(words[1]) & 0xFFFFFF
            name = BOUNDS_TABLES[code] if code < len(BOUNDS_TABLES) else f"table {code}"
            raise _lib.KernelLibraryError(f"index out of bounds: {name}[{pos}] (status 5)")
        raise _lib.KernelLibraryError(f"a kernel gave up on a bounded wait (status {st})")


def validate_indices(v, lo: int, hi: int, table: str) -> None:
    """Debug check (`PIE_BOUNDS=1`): every entry of the int32 table `v` lies in [lo, hi). On the device the
    first bad entry is recorded in the status block (read back by `check_kernel_status`); on the host it
    raises at once. Nothing is dereferenced through a bad index either way."""
    if v.numel() == 0:
        return
    if not v.is_cuda:
        bad = ((v < lo) | (v >= hi)).nonzero()
        if bad.numel():
            i = int(bad[0])
            raise IndexError(f"index out of bounds: {table}[{i}] = {int(v[i])}, not in [{lo}, {hi})")
        return
    check(fn("pie_validate_indices")(ptr(v), v.numel(), lo, hi, BOUNDS_TABLES.index(table),
                                     ptr(kernel_status(v.device)), stream_ptr()), "validate_indices")


# --------------------------------------------------------------------------- elementwise
def embed(tokens, table, vocab_start: int = 0, out=None):
    if not table.is_cuda:
        return reference.embed(tokens, table, vocab_start)
    n, h = tokens.numel(), table.shape[1]
    if out is None:
        out = torch.empty(n, h, dtype=table.dtype, device=table.device)
    check(fn("pie_embed_gather")(ptr(tokens), ptr(table), ptr(out), n, h, vocab_start, table.shape[0],
                                 stream_ptr()), "embed_gather")
    return out


def rmsnorm(x, w, eps: float, out=None, w_offset: float = 0.0):
    if not x.is_cuda:
        return reference.rmsnorm(x, w, eps, w_offset)
    if out is None:
        out = torch.empty_like(x)
    rows = x.numel() // x.shape[-1]
    check(fn("pie_rmsnorm")(ptr(x), None, None, ptr(w), ptr(out), rows, x.shape[-1], eps, w_offset,
                            stream_ptr()), "rmsnorm")
    return out


def add_rmsnorm(delta, residual, w, eps: float, out=None, w_offset: float = 0.0):
    """residual += delta in place; returns rmsnorm(residual) * w."""
    if not residual.is_cuda:
        return reference.add_rmsnorm(delta, residual, w, eps, w_offset)
    if out is None:
        out = torch.empty_like(residual)
    rows = residual.numel() // residual.shape[-1]
    check(fn("pie_rmsnorm")(ptr(residual), ptr(delta), ptr(residual), ptr(w), ptr(out), rows,
                            residual.shape[-1], eps, w_offset, stream_ptr()), "add_rmsnorm")
    return out


def swiglu(gate_up, out=None):
    if not gate_up.is_cuda:
        return reference.swiglu(gate_up)
    rows, two_i = gate_up.shape
    if out is None:
        out = torch.empty(rows, two_i // 2, dtype=gate_up.dtype, device=gate_up.device)
    check(fn("pie_swiglu")(ptr(gate_up), ptr(out), rows, two_i // 2, stream_ptr()), "swiglu")
    return out


GLU_ACTS = {"silu": 0, "gelu_tanh": 1}


def glu_interleaved(gate_up, act: str = "silu", out=None):
    """act(gate) * up over interleaved columns (gate_0, up_0, gate_1, ...): the layout the fused gate / up
    projection produces. `act`: "silu" or "gelu_tanh" (Gemma's GeGLU)."""
    if not gate_up.is_cuda or gate_up.dtype != torch.bfloat16:
        return reference.glu_interleaved(gate_up, act)
    rows, two_i = gate_up.shape
    gate_up = gate_up.contiguous()
    if out is None:
        out = torch.empty(rows, two_i // 2, dtype=gate_up.dtype, device=gate_up.device)
    check(fn("pie_glu_interleaved")(ptr(gate_up), ptr(out), rows, two_i // 2, GLU_ACTS[act], stream_ptr()), "glu_interleaved")
    return out


def qk_norm_rope_kvwrite(qkv, positions, slots, inv_freq, q_norm_w, k_norm_w, kv_layer, hq, hkv,
                         head_dim, page_size, eps, q_out=None, kv_scale=None, bias=None):
    """Per-head q/k RMSNorm (optional), RoPE, Q out, K/V rows appended into their page slots. With
    `kv_scale` (fp8 pages: kv_layer is a byte tensor, kv_scale [pages, 2, hkv, page] fp32) the rows are
    stored as e4m3 with one scale per (token, head). `bias` [(hq + 2 hkv) * head_dim]: the projection's bias,
    added to the packed rows first (in the kernel, instead of a pass of its own)."""
    if not qkv.is_cuda:
        if kv_scale is not None:
            raise NotImplementedError("fp8 KV pages need the CUDA kernels")
        if bias is not None:
            qkv = qkv + bias
        return reference.qk_norm_rope_kvwrite(qkv, positions, slots, inv_freq, q_norm_w, k_norm_w,
                                              kv_layer, hq, hkv, head_dim, page_size, eps)
    n = qkv.shape[0]
    if q_out is None:
        q_out = torch.empty(n, hq, head_dim, dtype=qkv.dtype, device=qkv.device)
    if bias is not None:
        check(fn("pie_qk_bias_norm_rope_kvwrite")(ptr(qkv), ptr(bias), ptr(positions), ptr(slots), ptr(inv_freq), ptr(q_norm_w),
                                                  ptr(k_norm_w), ptr(q_out), ptr(kv_layer), ptr(kv_scale), n, hq, hkv,
                                                  head_dim, page_size, eps, qkv.stride(0), stream_ptr()),
              "qk_bias_norm_rope_kvwrite")
        return q_out
    if kv_scale is not None:
        check(fn("pie_qk_norm_rope_kvwrite_kv8")(ptr(qkv), ptr(positions), ptr(slots), ptr(inv_freq), ptr(q_norm_w),
                                                 ptr(k_norm_w), ptr(q_out), ptr(kv_layer), ptr(kv_scale), n, hq, hkv,
                                                 head_dim, page_size, eps, qkv.stride(0), stream_ptr()),
              "qk_norm_rope_kvwrite_kv8")
        return q_out
    check(fn("pie_qk_norm_rope_kvwrite")(ptr(qkv), ptr(positions), ptr(slots), ptr(inv_freq),
                                         ptr(q_norm_w), ptr(k_norm_w), ptr(q_out), ptr(kv_layer), n,
                                         hq, hkv, head_dim, page_size, eps, qkv.stride(0),
                                         stream_ptr()), "qk_norm_rope_kvwrite")
    return q_out


def gather_rows(x, idx, out=None):
    if not x.is_cuda:
        return x[idx.long()]
    if out is None:
        out = torch.empty(idx.numel(), x.shape[1], dtype=x.dtype, device=x.device)
    check(fn("pie_gather_rows")(ptr(x), ptr(idx), ptr(out), idx.numel(), x.shape[1], stream_ptr()),
          "gather_rows")
    return out


def feed_tokens(tokens, src_row, prev_sampled, n: int):
    """tokens[i] = prev_sampled[src_row[i]] where src_row[i] >= 0 (device-side token feed)."""
    if not tokens.is_cuda:
        sel = src_row[:n] >= 0
        tokens[:n][sel] = prev_sampled[src_row[:n][sel].long()]
        return
    check(fn("pie_feed_tokens")(ptr(tokens), ptr(src_row), ptr(prev_sampled), n, stream_ptr()), "feed_tokens")


def copy_pages(kv, src, dst):
    """kv [layers, pages, ...]: copy page src[i] -> dst[i] in every layer."""
    if not kv.is_cuda:
        kv[:, dst.long()] = kv[:, src.long()]
        return
    layers = kv.shape[0]
    page_bytes = kv[0, 0].numel() * kv.element_size()
    layer_bytes = kv[0].numel() * kv.element_size()
    check(fn("pie_copy_pages")(ptr(kv), ptr(src), ptr(dst), src.numel(), layers, page_bytes,
                               layer_bytes, stream_ptr()), "copy_pages")


def brle_expand(rows_runs, nbits: int, device, tail_value: bool = False):
    """Expand BRLE rows (lists of run lengths, even index = zeros) to a packed bitmask
    [rows, ceil(nbits/32)] uint32 (as int32 tensor)."""
    words = (nbits + 31) // 32
    nrows = len(rows_runs)
    if torch.device(device).type != "cuda":
        out = torch.zeros(nrows, words * 32, dtype=torch.bool)
        for r, runs in enumerate(rows_runs):
            out[r, :nbits] = reference.brle_to_bool(runs, nbits, tail_value)
        w = out.view(nrows, words, 32).to(torch.int64)
        packed = (w << torch.arange(32, dtype=torch.int64)).sum(-1)
        return _to_i32(packed)
    ends = [np.cumsum(np.asarray(r, dtype=np.int64)).clip(max=2**32 - 1).astype(np.uint32) for r in rows_runs]
    indptr = np.zeros(nrows + 1, dtype=np.int32)
    indptr[1:] = np.cumsum([len(e) for e in ends])
    flat = np.concatenate(ends) if ends and indptr[-1] > 0 else np.zeros(1, dtype=np.uint32)
    d_ends = torch.from_numpy(flat.view(np.int32)).to(device)
    d_indptr = torch.from_numpy(indptr).to(device)
    out = torch.empty(nrows, words, dtype=torch.int32, device=device)
    check(fn("pie_brle_expand")(ptr(d_ends), ptr(d_indptr), ptr(out), nrows, nbits, int(tail_value),
                                stream_ptr()), "brle_expand")
    return out


def brle_expand_ragged(rows_runs, row_nbits, device, tail_value: bool = False):
    """BRLE rows of different lengths in one launch: row r expands to ceil(row_nbits[r] / 32) words. Returns the words
    of all rows back to back (int32 tensor) and the word offset of every row (int64 numpy [rows + 1])."""
    nrows = len(rows_runs)
    nbits = np.asarray(row_nbits, dtype=np.int32)
    words = (nbits.astype(np.int64) + 31) // 32
    offs = np.zeros(nrows + 1, dtype=np.int64)
    offs[1:] = np.cumsum(words)
    if torch.device(device).type != "cuda":
        parts = [brle_expand([r], int(n), device, tail_value).reshape(-1) for r, n in zip(rows_runs, nbits)]
        return (torch.cat(parts) if parts else torch.zeros(0, dtype=torch.int32)), offs
    ends = [np.cumsum(np.asarray(r, dtype=np.int64)).clip(max=2**32 - 1).astype(np.uint32) for r in rows_runs]
    indptr = np.zeros(nrows + 1, dtype=np.int32)
    indptr[1:] = np.cumsum([len(e) for e in ends])
    flat = np.concatenate(ends) if ends and indptr[-1] > 0 else np.zeros(1, dtype=np.uint32)
    out = torch.empty(max(1, int(offs[-1])), dtype=torch.int32, device=device)
    if nrows:
        d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
        d_ends, d_indptr, d_offs, d_bits = d(flat.view(np.int32)), d(indptr), d(offs[:-1]), d(nbits)
        check(fn("pie_brle_expand_ragged")(ptr(d_ends), ptr(d_indptr), ptr(out), ptr(d_offs), ptr(d_bits), nrows,
                                           int(words.max()) if nrows else 0, int(tail_value), stream_ptr()), "brle_expand_ragged")
    return out[:int(offs[-1])], offs


def _to_i32(packed_i64):
    p = packed_i64 & 0xFFFFFFFF
    p = torch.where(p >= 2**31, p - 2**32, p)
    return p.to(torch.int32)


# --------------------------------------------------------------------------- GEMM
_GEMM_WS = {}


def ensure_gemm_workspace(device) -> None:
    """Register the stream-K scratch of `device` with the kernel library (once per device):
    fp32 space for the partial tiles of split output tiles and their arrival counters."""
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx in _GEMM_WS:
        return
    sms = num_sms(idx)
    ws = torch.empty(3 * sms * 128 * 256, dtype=torch.float32, device=f"cuda:{idx}")
    cnt = torch.zeros(2 * sms * 4, dtype=torch.int32, device=f"cuda:{idx}")
    check(fn("pie_gemm_set_workspace")(idx, ptr(ws), ws.numel(), ptr(cnt), cnt.numel()), "gemm_set_workspace")
    _GEMM_WS[idx] = (ws, cnt)
    import os
    if os.environ.get("PIE_GEMM_PAIRS", "1") == "0":
        set_gemm_pairs(False)
    set_pdl(os.environ.get("PIE_PDL", "1") != "0")
    if "PIE_GEMM_SWAP" in os.environ:
        set_gemm_swap(int(os.environ["PIE_GEMM_SWAP"]))


def set_pdl(enabled: bool) -> None:
    """Programmatic dependent launch for the library's kernels: a kernel's prologue and weight
    prefetch overlap the tail of its predecessor in the stream (also inside CUDA graphs).
    On unless PIE_PDL=0: measured 3.5 % of a 64-request decode step, 2 % at 128, neutral at 512."""
    check(fn("pie_set_pdl")(1 if enabled else 0), "set_pdl")


def set_gemm_swap(max_m: int) -> None:
    """Batches of up to max_m rows (default and at most 128) may run the single-CTA GEMM with swapped
    operands (weights on the 128-row side of the MMA, transposed epilogue) where the launcher's rule
    expects a gain; 0 turns that off, 1000 swaps every batch of up to 128 rows (tests)."""
    fn("pie_gemm_set_swap")(int(max_m))


def set_gemm_pairs(enabled: bool) -> None:
    """Use CTA-pair (cta_group::2, 256-row) tiles where the shape allows, or single-CTA tiles only."""
    check(fn("pie_gemm_set_pairs")(1 if enabled else 0), "gemm_set_pairs")


def gemm(x, w, residual=None, epilogue: int = EPI_STORE, out=None, force_bn: int = 0):
    """y = x @ w.T (+ residual | SwiGLU over interleaved gate/up columns). x [M,K], w [N,K]."""
    if not x.is_cuda:
        y = reference.gemm(x, w, residual if epilogue == EPI_RESIDUAL else None)
        return reference.swiglu_interleaved(y) if epilogue == EPI_SWIGLU else y
    m, k = x.shape
    n = w.shape[0]
    n_out = n // 2 if epilogue == EPI_SWIGLU else n
    if out is None:
        out = torch.empty(m, n_out, dtype=x.dtype, device=x.device)
    if m == 0:
        return out
    ensure_gemm_workspace(x.device)
    check(fn("pie_gemm_bf16")(ptr(x), ptr(w), ptr(out), ptr(residual), m, n, k, x.stride(0), w.stride(0),
                              out.stride(0), residual.stride(0) if residual is not None else 0, epilogue,
                              force_bn, ptr(kernel_status(x.device)), num_sms(x.device), stream_ptr()),
          "gemm_bf16")
    return out


# --------------------------------------------------------------------------- fp8 weights
FP8_BLOCK = 128


class Fp8Linear:
    """Weight [N, K] in fp8 e4m3 with one fp32 scale per (row, 128 columns). Checkpoints with
    128 x 128 block scales expand each block's scale to its rows when loaded, which keeps row
    permutations (interleaved gate/up) exact."""

    def __init__(self, w8: torch.Tensor, scale: torch.Tensor):
        assert w8.dtype == torch.float8_e4m3fn and scale.dtype == torch.float32
        assert scale.shape == (w8.shape[0], (w8.shape[1] + FP8_BLOCK - 1) // FP8_BLOCK)
        self.w8, self.scale = w8.contiguous(), scale.contiguous()

    @property
    def shape(self):
        return self.w8.shape

    @property
    def device(self):
        return self.w8.device

    def nbytes(self) -> int:
        return self.w8.numel() + self.scale.numel() * 4

    def dequant(self, dtype=torch.bfloat16, out=None) -> torch.Tensor:
        return dequant_fp8(self, dtype, out)


def quantize_fp8_block(w: torch.Tensor, block_rows: int = FP8_BLOCK) -> "Fp8Linear":
    """Block-scaled fp8 quantisation (scale = absmax / 448 per block_rows x 128 block)."""
    n, k = w.shape
    wf = w.float()
    kb = (k + FP8_BLOCK - 1) // FP8_BLOCK
    nb = (n + block_rows - 1) // block_rows
    pad = torch.zeros(nb * block_rows, kb * FP8_BLOCK, dtype=torch.float32, device=w.device)
    pad[:n, :k] = wf
    blocks = pad.view(nb, block_rows, kb, FP8_BLOCK)
    scale = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12) / 448.0          # [nb, kb]
    q = (blocks / scale[:, None, :, None]).view(nb * block_rows, kb * FP8_BLOCK)[:n, :k]
    row_scale = scale.repeat_interleave(block_rows, dim=0)[:n].contiguous()
    return Fp8Linear(q.to(torch.float8_e4m3fn), row_scale)


_FP8_SCRATCH = {}


def dequant_fp8(q: "Fp8Linear", dtype=torch.bfloat16, out=None) -> torch.Tensor:
    n, k = q.shape
    if not q.w8.is_cuda:
        kb = q.scale.shape[1]
        s = q.scale.repeat_interleave(FP8_BLOCK, dim=1)[:, :k]
        return (q.w8.float() * s).to(dtype)
    if out is None:
        out = torch.empty(n, k, dtype=torch.bfloat16, device=q.device)
    check(fn("pie_dequant_fp8_rowblock")(ptr(q.w8), ptr(q.scale), ptr(out), n, k, stream_ptr()), "dequant_fp8")
    return out


def quant_act_fp8(x: torch.Tensor):
    """1 x 128 activation quantisation: (x8 e4m3 [M, K], scales fp32 [M, ceil(K/128)])."""
    m, k = x.shape
    kb = (k + FP8_BLOCK - 1) // FP8_BLOCK
    if not x.is_cuda:
        pad = torch.zeros(m, kb * FP8_BLOCK, dtype=torch.float32)
        pad[:, :k] = x.float()
        blocks = pad.view(m, kb, FP8_BLOCK)
        sc = blocks.abs().amax(dim=2).clamp_min(1e-12) / 448.0
        return (blocks / sc[:, :, None]).view(m, -1)[:, :k].to(torch.float8_e4m3fn), sc
    x8 = torch.empty(m, k, dtype=torch.float8_e4m3fn, device=x.device)
    sx = torch.empty(m, kb, dtype=torch.float32, device=x.device)
    check(fn("pie_quant_act_fp8")(ptr(x), x.stride(0), ptr(x8), ptr(sx), m, k, stream_ptr()), "quant_act_fp8")
    return x8, sx


def gemm_fp8_reference(x8, sx, q: "Fp8Linear") -> torch.Tensor:
    """fp32 evaluation of the block-scaled product (the oracle of the fused kernel)."""
    k = x8.shape[1]
    xs = x8.float() * sx.repeat_interleave(FP8_BLOCK, dim=1)[:, :k]
    ws = q.w8.float() * q.scale.repeat_interleave(FP8_BLOCK, dim=1)[:, :k]
    return xs @ ws.t()


_FP8_MODE = None


def fp8_mode() -> str:
    """"fused": fp8 x fp8 tcgen05 GEMM with block scales folded per 128-deep K block (activations
    quantised 1 x 128 on the fly); "dequant": expand the weight to bf16 first (the reference's scheme)."""
    global _FP8_MODE
    if _FP8_MODE is None:
        import os
        _FP8_MODE = os.environ.get("PIE_FP8_MODE", "fused")
    return _FP8_MODE


def gemm_fp8w(x, q: "Fp8Linear", residual=None, epilogue: int = EPI_STORE, mode: Optional[str] = None):
    """y = x @ W.T for a block-scaled fp8 weight, with the usual epilogues."""
    if not x.is_cuda:
        w = dequant_fp8(q, x.dtype)
        y = reference.gemm(x, w, residual if epilogue == EPI_RESIDUAL else None)
        return reference.swiglu_interleaved(y) if epilogue == EPI_SWIGLU else y
    n, k = q.shape
    m = x.shape[0]
    if mode is None:
        # measured cross-over on B200: the per-block rescale caps the fused kernel at ~0.55 PFLOP/s,
        # so prefill-sized M runs faster through one expansion and the bf16 pair kernel
        mode = fp8_mode() if m <= 1024 else "dequant"
    if mode == "fused" and k % 16 == 0 and n % 16 == 0:
        x8, sx = quant_act_fp8(x)
        out = torch.empty(m, n // 2 if epilogue == EPI_SWIGLU else n, dtype=torch.bfloat16, device=x.device)
        check(fn("pie_gemm_fp8_blockscaled")(ptr(x8), ptr(sx), ptr(q.w8), ptr(q.scale), ptr(out), ptr(residual), m, n, k,
                                             out.stride(0), residual.stride(0) if residual is not None else 0,
                                             epilogue, ptr(kernel_status(x.device)), num_sms(x.device), stream_ptr()),
              "gemm_fp8_blockscaled")
        return out
    key = (q.device.index, tuple(q.shape))
    buf = _FP8_SCRATCH.get(key)
    if buf is None:
        buf = _FP8_SCRATCH[key] = torch.empty(*q.shape, dtype=torch.bfloat16, device=q.device)
    dequant_fp8(q, out=buf)
    return gemm(x, buf, residual=residual, epilogue=epilogue)


# --------------------------------------------------------------------------- mixture of experts
MOE_TILE = 128


def moe_max_mtiles(n_tokens: int, k: int, num_experts: int) -> int:
    """Upper bound of 128-row tiles after padding every expert's segment."""
    return (n_tokens * k + MOE_TILE - 1) // MOE_TILE + num_experts


class MoeBuffers:
    """Device scratch of one MoE block evaluation for up to `n` tokens (graph-safe: fixed addresses)."""

    def __init__(self, n: int, hidden: int, inter: int, num_experts: int, k: int, device, dtype=torch.bfloat16):
        self.n, self.k, self.E, self.H, self.I = n, k, num_experts, hidden, inter
        self.max_mtiles = moe_max_mtiles(n, k, num_experts)
        rows = self.max_mtiles * MOE_TILE
        i32 = dict(dtype=torch.int32, device=device)
        self.ids = torch.empty(n, k, **i32)
        self.pos = torch.empty(n, k, **i32)
        self.slot_of = torch.empty(n, k, **i32)
        self.w = torch.empty(n, k, dtype=torch.float32, device=device)
        self.counts = torch.zeros(num_experts, **i32)
        self.counts_out = torch.zeros(num_experts, **i32)
        self.seg_start = torch.empty(num_experts, **i32)
        self.tile_expert = torch.empty(self.max_mtiles, **i32)
        self.xs = torch.zeros(rows, hidden, dtype=dtype, device=device)
        self.act = torch.zeros(rows, inter, dtype=dtype, device=device)
        self.ys = torch.zeros(rows, hidden, dtype=dtype, device=device)


def moe_route(logits, k: int, renorm: bool, buf: "MoeBuffers", e_lo: int = 0):
    """Top-k routing over all experts; only experts [e_lo, e_lo + buf.E) take slots here."""
    n, e = logits.shape
    check(fn("pie_moe_route")(ptr(logits), 1 if logits.dtype == torch.float32 else 0, logits.stride(0), n, e, k,
                              1 if renorm else 0, e_lo, buf.E, ptr(buf.ids), ptr(buf.w), ptr(buf.pos),
                              ptr(buf.counts), stream_ptr()), "moe_route")
    return buf.ids[:n], buf.w[:n]


def moe_align(buf: "MoeBuffers", max_mtiles: int = 0):
    check(fn("pie_moe_align")(ptr(buf.counts), buf.E, max_mtiles or buf.max_mtiles, ptr(buf.seg_start),
                              ptr(buf.tile_expert), ptr(buf.counts_out), stream_ptr()), "moe_align")


def moe_permute(x, buf: "MoeBuffers"):
    n, h = x.shape
    check(fn("pie_moe_permute")(ptr(x), x.stride(0), ptr(buf.ids), ptr(buf.pos), ptr(buf.seg_start), n, h, buf.k,
                                ptr(buf.xs), ptr(buf.slot_of), stream_ptr()), "moe_permute")


def grouped_gemm(a, w, tile_expert, out, max_mtiles: int, epilogue: int = EPI_STORE):
    """out[tile rows] = a[tile rows] @ w[tile_expert[tile]].T for every used 128-row tile. w [E,N,K]."""
    e, n, k = w.shape
    assert w.is_contiguous() and a.shape[1] == k and a.shape[0] >= max_mtiles * MOE_TILE
    check(fn("pie_grouped_gemm_bf16")(ptr(a), ptr(w), ptr(out), ptr(tile_expert), max_mtiles, e, n, k, a.stride(0),
                                      out.stride(0), epilogue, ptr(kernel_status(a.device)), num_sms(a.device),
                                      stream_ptr()), "grouped_gemm_bf16")
    return out


def moe_bias_glu(gu, bias, tile_expert, act, mtiles: int, limit: float):
    """act = clamped GLU of (gu + bias[expert of row]) on expert-sorted rows (GPT-OSS experts)."""
    check(fn("pie_moe_bias_glu")(ptr(gu), ptr(bias), ptr(tile_expert), ptr(act), mtiles, act.shape[1], limit,
                                 stream_ptr()), "moe_bias_glu")
    return act


def moe_row_bias(y, bias, tile_expert, mtiles: int):
    """y[row] += bias[expert of row] on expert-sorted rows."""
    check(fn("pie_moe_row_bias")(ptr(y), ptr(bias), ptr(tile_expert), mtiles, y.shape[1], stream_ptr()), "moe_row_bias")
    return y


def moe_combine(buf: "MoeBuffers", n: int, residual=None, out=None):
    if out is None:
        out = torch.empty(n, buf.H, dtype=buf.ys.dtype, device=buf.ys.device)
    check(fn("pie_moe_combine")(ptr(buf.ys), ptr(buf.slot_of), ptr(buf.w), ptr(residual),
                                residual.stride(0) if residual is not None else 0, n, buf.H, buf.k, ptr(out),
                                out.stride(0), stream_ptr()), "moe_combine")
    return out


def moe_experts(x, logits, w_gate_up, w_down, k: int, renorm: bool, buf: "MoeBuffers", residual=None,
                e_lo: int = 0, rs=None):
    """residual + sum_j w_j * down_e(swiglu(gate_up_e(x))) over each token's top-k experts e.

    w_gate_up / w_down hold experts [e_lo, e_lo + E_local) (all of them on one GPU). With
    rs=(tp_blob, rows_per_rank) the partial sums go to the row owners' receive buffers by peer
    stores instead of `out` (tensor / expert parallelism)."""
    n = x.shape[0]
    mt = moe_max_mtiles(n, k, buf.E)
    moe_route(logits, k, renorm, buf, e_lo)
    moe_align(buf, mt)
    moe_permute(x, buf)
    grouped_gemm(buf.xs, w_gate_up, buf.tile_expert, buf.act, mt, EPI_SWIGLU)
    grouped_gemm(buf.act, w_down, buf.tile_expert, buf.ys, mt, EPI_STORE)
    if rs is not None:
        check(fn("pie_moe_combine_rs")(ptr(buf.ys), ptr(buf.slot_of), ptr(buf.w), n, buf.H, k, rs[0], rs[1],
                                       stream_ptr()), "moe_combine_rs")
        return None
    return moe_combine(buf, n, residual)


# --------------------------------------------------------------------------- attention
@dataclass
class AttnBatch:
    """Host description of one fire's attention work (CSR arrays as numpy int32)."""
    qo_indptr: np.ndarray
    kv_page_indptr: np.ndarray
    page_indices: np.ndarray
    kv_lens: np.ndarray            # total kv length per request, new tokens included
    masks: Optional[list] = None   # per request: None (causal) or bool [qo_len, kv_len] array
    window_left: int = -1

    @property
    def num_requests(self) -> int:
        return len(self.kv_lens)

    @property
    def is_decode(self) -> bool:
        q = np.diff(self.qo_indptr)
        return bool(len(q) > 0 and (q == 1).all() and self.masks is None)


# work units (KV chunk x KV head) each persistent decode-attention CTA should get: more units balance the
# tail of the launch better, fewer keep the merge pass short
_DECODE_UNITS_PER_CTA = int(os.environ.get("PIE_DECODE_UNITS", "4"))


def plan_decode_items(kv_lens: np.ndarray, hkv: int, target_ctas: int, max_items: int = 0,
                      min_chunk: int = 256, window_left: int = -1):
    """Split each request's KV range into chunks so that items*hkv fills the machine. With a
    sliding window only the last window_left + 1 keys are covered, from the 16-token boundary
    at or below the first visible key (the kernel masks the keys below it).

    Returns (item_req, item_start, item_end, req_item_indptr) as int32 arrays.
    """
    full_lens = np.asarray(kv_lens, dtype=np.int64)
    lo = np.zeros_like(full_lens)
    if window_left >= 0:
        lo = np.maximum(0, full_lens - 1 - window_left) // 16 * 16
    kv_lens = full_lens - lo
    total = int(kv_lens.sum())
    chunk = max(min_chunk, -(-total * hkv // max(1, target_ctas * _DECODE_UNITS_PER_CTA)))
    chunk = -(-chunk // 16) * 16
    while True:
        n_items = np.maximum(1, -(-kv_lens // chunk))
        if max_items <= 0 or int(n_items.sum()) <= max_items:
            break
        chunk *= 2
    indptr = np.zeros(len(kv_lens) + 1, dtype=np.int32)
    indptr[1:] = np.cumsum(n_items)
    tot = int(indptr[-1])
    item_req = np.repeat(np.arange(len(kv_lens), dtype=np.int32), n_items)
    within = np.arange(tot, dtype=np.int64) - np.repeat(indptr[:-1].astype(np.int64), n_items)
    start = within * chunk
    end = np.minimum(start + chunk, kv_lens[item_req])
    start, end = start + lo[item_req], end + lo[item_req]
    return item_req, start.astype(np.int32), end.astype(np.int32), indptr


@dataclass
class CascadePlan:
    """Host side of a decode plan with shared-prefix items (see `plan_decode_cascade`)."""
    item_req: np.ndarray
    item_start: np.ndarray
    item_end: np.ndarray
    item_slot: np.ndarray
    item_tile: np.ndarray
    tile_members: np.ndarray      # [tiles, 16]
    req_slot_indptr: np.ndarray
    shared_tokens: int            # KV tokens that are read once instead of once per member
    groups: int


def find_shared_prefixes(kv_lens: np.ndarray, page_indptr: np.ndarray, page_indices: np.ndarray, page_size: int,
                         min_shared_tokens: int = 256, cache: Optional[dict] = None):
    """Groups of requests whose leading KV pages are the same physical pages (forks of one context).
    Returns [(members int32 array, shared_tokens)] for groups of two or more requests that share at
    least `min_shared_tokens`; shared_tokens is a multiple of the page size.

    `cache` (a dict the caller keeps between steps) remembers the groups and their common page count
    for a batch with the same rows in the same order: page lists only grow at their private tail from
    one decode step to the next, so a step then only re-checks the lengths."""
    r = len(kv_lens)
    if r < 2:
        return []
    kv = np.asarray(kv_lens, dtype=np.int64)
    indptr = np.asarray(page_indptr, dtype=np.int64)
    npages = np.diff(indptr)
    pages = np.asarray(page_indices)
    first = np.where(npages > 0, pages[np.minimum(indptr[:-1], max(0, len(pages) - 1))], -1 - np.arange(r))
    key = (r, first.tobytes())
    found = cache.get(key) if cache is not None else None
    if found is not None:
        # still valid if every member still holds at least the remembered common pages
        if any(int(npages[mem].min()) < lcp for mem, lcp in found):
            found = None
    if found is None:
        order = np.argsort(first, kind="stable")
        sf = first[order]
        cut = np.flatnonzero(np.diff(sf)) + 1
        found = []
        for a, b in zip(np.concatenate([[0], cut]), np.concatenate([cut, [r]])):
            if b - a < 2 or sf[a] < 0:
                continue
            mem = order[a:b]
            n = int(npages[mem].min())
            if n * page_size < min_shared_tokens:
                continue
            block = pages[indptr[mem][:, None] + np.arange(n)[None, :]]          # [members, n]
            differ = (block != block[0:1]).any(axis=0)
            lcp = int(np.argmax(differ)) if differ.any() else n
            if lcp * page_size >= min_shared_tokens:
                found.append((np.sort(mem).astype(np.int32), lcp))
        if cache is not None:
            if len(cache) > 64:
                cache.clear()
            cache[key] = found
    out = []
    for mem, lcp in found:
        # the page that receives this step's token is private, and so is everything after it
        n = min(lcp, int(((kv[mem] - 1) // page_size).min()))
        if n * page_size >= min_shared_tokens:
            out.append((mem, n * page_size))
    return out


def plan_decode_cascade(kv_lens: np.ndarray, groups, hkv: int, group_size: int, target_ctas: int, max_items: int,
                        min_chunk: int = 256) -> Optional[CascadePlan]:
    """Decode plan in which every group of `groups` (from `find_shared_prefixes`) reads its shared
    prefix once: per group and per tile of 16 // group_size members, shared items over the prefix in
    chunks; per request, unshared items over the rest. A request's partial results occupy consecutive
    slots (shared chunks first). Returns None when there is nothing to share or the plan would not
    fit `max_items` slots / items."""
    memb = max(1, 16 // group_size)
    if not groups or memb < 2:        # 16 query heads per KV head fill the tile: nothing to pack
        return None
    kv = np.asarray(kv_lens, dtype=np.int64)
    r = len(kv)
    shared = np.zeros(r, np.int64)
    for mem, st in groups:
        shared[mem] = st
    own = kv - shared
    tiles_of = [-(-len(mem) // memb) for mem, _ in groups]
    work = int(own.sum()) + sum(st * t for (_, st), t in zip(groups, tiles_of))
    chunk = max(min_chunk, -(-work * hkv // max(1, target_ctas * _DECODE_UNITS_PER_CTA)))
    chunk = -(-chunk // 16) * 16
    while True:
        n_sh = -(-shared // chunk)
        n_own = np.maximum(1, -(-own // chunk))
        n_items = int(n_own.sum()) + sum(int(-(-st // chunk)) * t for (_, st), t in zip(groups, tiles_of))
        if int((n_sh + n_own).sum()) <= max_items and n_items <= max_items:
            break
        chunk *= 2
        if chunk > (1 << 22):
            return None
    indptr = np.zeros(r + 1, np.int32)
    indptr[1:] = np.cumsum(n_sh + n_own)
    i_req, i_st, i_en, i_slot, i_tile, members = [], [], [], [], [], []
    for (mem, st), nt in zip(groups, tiles_of):
        nch = int(-(-st // chunk))
        for t in range(nt):
            row = np.full(16, -1, np.int32)
            part = mem[t * memb:(t + 1) * memb]
            row[:len(part)] = part
            tid = len(members)
            members.append(row)
            c = np.arange(nch, dtype=np.int64)
            i_req.append(np.full(nch, part[0], np.int32))
            i_st.append(c * chunk)
            i_en.append(np.minimum((c + 1) * chunk, st))
            i_slot.append(c)
            i_tile.append(np.full(nch, tid, np.int32))
    req = np.repeat(np.arange(r, dtype=np.int32), n_own)
    base = np.zeros(r + 1, np.int64)
    base[1:] = np.cumsum(n_own)
    within = np.arange(int(base[-1]), dtype=np.int64) - np.repeat(base[:-1], n_own)
    st_own = shared[req] + within * chunk
    i_req.append(req)
    i_st.append(st_own)
    i_en.append(np.minimum(st_own + chunk, kv[req]))
    i_slot.append(indptr[:-1].astype(np.int64)[req] + n_sh[req] + within)
    i_tile.append(np.full(len(req), -1, np.int32))
    cat = lambda xs: np.concatenate(xs).astype(np.int32)
    return CascadePlan(cat(i_req), cat(i_st), cat(i_en), cat(i_slot), cat(i_tile), np.stack(members).astype(np.int32),
                       indptr, int(sum(st * (len(mem) - t) for (mem, st), t in zip(groups, tiles_of))), len(groups))


def prefill_tile_rows(hq: int, hkv: int, head_dim: int, page_size: int, softcap: bool = False) -> int:
    """Packed (token, head) rows per prefill tile: 256 (two MMA tiles per CTA; ``PIE_PREFILL_TC=128``
    for one) where the tcgen05 kernel covers the shape (head_dim 64 or 128, 16-token pages, group size
    dividing 128), else - or with ``PIE_PREFILL_TC=0`` - the 64 rows of the mma.sync kernel."""
    want = os.environ.get("PIE_PREFILL_TC", "256")
    if want == "0" or not fn("pie_prefill_attn_tc_supported")(hq, hkv, head_dim, page_size):
        return 64
    return 128 if want == "128" and not softcap else 256          # a soft cap is built for the two-tile variant only


def plan_prefill_tiles(qo_indptr: np.ndarray, group: int, rows: int = 64, kv_lens=None):
    """Tiles of rows/group query tokens per request: (tile_req, tile_qstart). With `kv_lens` the
    tiles are ordered by falling causal work (keys visible to the tile's last token), so that the
    long tiles start first and the short ones fill the tail of the grid."""
    tq = max(1, rows // group)
    qlens = np.diff(qo_indptr).astype(np.int64)
    ntiles = -(-qlens // tq)
    tile_req = np.repeat(np.arange(len(qlens), dtype=np.int32), ntiles)
    base = np.zeros(len(qlens) + 1, dtype=np.int64)
    base[1:] = np.cumsum(ntiles)
    within = np.arange(int(base[-1]), dtype=np.int64) - np.repeat(base[:-1], ntiles)
    qstart = within * tq
    if kv_lens is not None and len(tile_req) > 1:
        kl = np.asarray(kv_lens, dtype=np.int64)[tile_req]
        work = kl - qlens[tile_req] + np.minimum(qstart + tq, qlens[tile_req])
        order = np.argsort(-work, kind="stable")
        tile_req, qstart = tile_req[order], qstart[order]
    return tile_req, qstart.astype(np.int32)


@dataclass
class DecodePlan:
    """Device-side arguments of the split-KV decode kernel (static addresses: graph safe)."""
    page_indices: torch.Tensor
    kv_page_indptr: torch.Tensor
    item_req: torch.Tensor
    item_start: torch.Tensor
    item_end: torch.Tensor
    req_item_indptr: torch.Tensor
    num_items: torch.Tensor       # int32[1] on device
    scratch: torch.Tensor         # fp32 partial outputs + lse
    max_items: int
    num_reqs: int
    num_ctas: int
    page_size: int
    window_left: int = -1
    # shared-prefix plans (`plan_decode_cascade`): slot / tile of every item and the members of every tile
    item_slot: Optional[torch.Tensor] = None
    item_tile: Optional[torch.Tensor] = None
    tile_members: Optional[torch.Tensor] = None


def decode_scratch_floats(max_items: int, hq: int, head_dim: int) -> int:
    return max_items * hq * head_dim + max_items * hq


def dequant_kv_pages(kv8_layer, scale_layer, pages: torch.Tensor, pad_zero_page: bool = True) -> torch.Tensor:
    """fp8 pages `pages` (int32, device) of one layer expanded to a compact bf16 tensor
    [len(pages) (+ 1 zero page), 2, hkv, page, d]; page j of the result is source page pages[j]."""
    n = pages.numel()
    _, two, hkv, page, d = kv8_layer.shape
    out = torch.empty(n + (1 if pad_zero_page else 0), two, hkv, page, d, dtype=torch.bfloat16, device=kv8_layer.device)
    if pad_zero_page:
        out[n].zero_()
    check(fn("pie_dequant_kv_pages")(ptr(kv8_layer), ptr(scale_layer), ptr(pages), ptr(out), n, hkv, page, d,
                                     stream_ptr()), "dequant_kv_pages")
    return out


def paged_decode_attention(q, kv_layer, plan: DecodePlan, sm_scale: float, out=None, window_left=None,
                           sinks_log2=None, kv_scale=None, softcap: float = 0.0):
    """q [R, hq, D] (one token per request) against paged KV; split-KV + merge. `window_left`
    overrides the plan's window for this call (a layer with its own window; the plan's items
    must then cover at least that window), `sinks_log2` [hq] fp32 = sink logits * log2(e)."""
    if out is None:
        out = torch.empty_like(q)
    wl = plan.window_left if window_left is None else window_left
    r, hq, d = q.shape
    hkv = kv_layer.shape[2]
    if softcap:                     # softmax over softcap * tanh(score / softcap) (Gemma-2)
        if kv_scale is not None or plan.item_tile is not None:
            raise NotImplementedError("soft-capped scores over fp8 KV pages or shared-prefix plans")
        check(fn("pie_paged_decode_attn_softcap")(
            ptr(q), ptr(kv_layer), ptr(plan.page_indices), ptr(plan.kv_page_indptr), ptr(plan.item_req),
            ptr(plan.item_start), ptr(plan.item_end), ptr(plan.req_item_indptr), ptr(plan.num_items),
            ptr(out), ptr(plan.scratch), plan.max_items, plan.num_reqs, hq, hkv, d, plan.page_size,
            sm_scale, plan.num_ctas, 1, wl, ptr(sinks_log2), float(softcap), stream_ptr()), "paged_decode_attn_softcap")
        return out
    if kv_scale is not None:        # fp8 pages with per-(token, head) scales
        if plan.item_tile is not None:
            raise NotImplementedError("shared-prefix plans over fp8 KV pages")
        check(fn("pie_paged_decode_attn_kv8")(
            ptr(q), ptr(kv_layer), ptr(kv_scale), ptr(plan.page_indices), ptr(plan.kv_page_indptr), ptr(plan.item_req),
            ptr(plan.item_start), ptr(plan.item_end), ptr(plan.req_item_indptr), ptr(plan.num_items),
            ptr(out), ptr(plan.scratch), plan.max_items, plan.num_reqs, hq, hkv, d, plan.page_size,
            sm_scale, plan.num_ctas, wl, ptr(sinks_log2), stream_ptr()), "paged_decode_attn_kv8")
        return out
    if plan.item_tile is not None:
        check(fn("pie_paged_decode_attn_cascade")(
            ptr(q), ptr(kv_layer), ptr(plan.page_indices), ptr(plan.kv_page_indptr), ptr(plan.item_req),
            ptr(plan.item_start), ptr(plan.item_end), ptr(plan.req_item_indptr), ptr(plan.num_items),
            ptr(out), ptr(plan.scratch), plan.max_items, plan.num_reqs, hq, hkv, d, plan.page_size,
            sm_scale, plan.num_ctas, ptr(sinks_log2), ptr(plan.item_slot), ptr(plan.item_tile),
            ptr(plan.tile_members), stream_ptr()), "paged_decode_attn_cascade")
        return out
    check(fn("pie_paged_decode_attn_window")(
        ptr(q), ptr(kv_layer), ptr(plan.page_indices), ptr(plan.kv_page_indptr), ptr(plan.item_req),
        ptr(plan.item_start), ptr(plan.item_end), ptr(plan.req_item_indptr), ptr(plan.num_items),
        ptr(out), ptr(plan.scratch), plan.max_items, plan.num_reqs, hq, hkv, d, plan.page_size,
        sm_scale, plan.num_ctas, 1, wl, ptr(sinks_log2), stream_ptr()), "paged_decode_attn")
    return out


@dataclass
class PrefillPlan:
    page_indices: torch.Tensor
    kv_page_indptr: torch.Tensor
    qo_indptr: torch.Tensor
    kv_lens: torch.Tensor
    tile_req: torch.Tensor
    tile_qstart: torch.Tensor
    num_tiles: int
    page_size: int
    mask_bits: Optional[torch.Tensor] = None
    mask_word_indptr: Optional[torch.Tensor] = None
    window_left: int = -1
    tile_rows: int = 64           # 128 / 256: tiles planned for the tcgen05 kernel


def paged_prefill_attention(q, kv_layer, plan: PrefillPlan, sm_scale: float, out=None, lse_out=None,
                            window_left=None, sinks_log2=None, softcap: float = 0.0):
    if out is None:
        out = torch.empty_like(q)
    wl = plan.window_left if window_left is None else window_left
    n, hq, d = q.shape
    hkv = kv_layer.shape[2]
    if softcap and plan.tile_rows > 64:
        if plan.tile_rows != 256:
            raise ValueError("soft-capped scores on the tcgen05 kernel need 256-row tiles: plan with prefill_tile_rows(..., softcap=True)")
        check(fn("pie_paged_prefill_attn_tc_softcap")(
            ptr(q), ptr(kv_layer), ptr(plan.page_indices), ptr(plan.kv_page_indptr), ptr(plan.qo_indptr),
            ptr(plan.kv_lens), ptr(plan.tile_req), ptr(plan.tile_qstart), plan.num_tiles,
            ptr(plan.mask_bits), ptr(plan.mask_word_indptr), ptr(out), ptr(lse_out), n, hq, hkv, d,
            kv_layer.shape[0], sm_scale, wl, plan.tile_rows, ptr(sinks_log2), ptr(kernel_status(q.device)),
            float(softcap), stream_ptr()), "paged_prefill_attn_tc_softcap")
        return out
    if softcap:
        check(fn("pie_paged_prefill_attn_softcap")(
            ptr(q), ptr(kv_layer), ptr(plan.page_indices), ptr(plan.kv_page_indptr), ptr(plan.qo_indptr),
            ptr(plan.kv_lens), ptr(plan.tile_req), ptr(plan.tile_qstart), plan.num_tiles,
            ptr(plan.mask_bits), ptr(plan.mask_word_indptr), ptr(out), ptr(lse_out), hq, hkv, d,
            plan.page_size, sm_scale, wl, ptr(sinks_log2), float(softcap), stream_ptr()), "paged_prefill_attn_softcap")
        return out
    if plan.tile_rows > 64:
        # kv_layer is [pages + 1, 2, hkv, page, d]; its last page is the zero pad page
        check(fn("pie_paged_prefill_attn_tc")(
            ptr(q), ptr(kv_layer), ptr(plan.page_indices), ptr(plan.kv_page_indptr), ptr(plan.qo_indptr),
            ptr(plan.kv_lens), ptr(plan.tile_req), ptr(plan.tile_qstart), plan.num_tiles,
            ptr(plan.mask_bits), ptr(plan.mask_word_indptr), ptr(out), ptr(lse_out), n, hq, hkv, d,
            kv_layer.shape[0], sm_scale, wl, plan.tile_rows, ptr(sinks_log2), ptr(kernel_status(q.device)),
            stream_ptr()),
            "paged_prefill_attn_tc")
        return out
    check(fn("pie_paged_prefill_attn")(
        ptr(q), ptr(kv_layer), ptr(plan.page_indices), ptr(plan.kv_page_indptr), ptr(plan.qo_indptr),
        ptr(plan.kv_lens), ptr(plan.tile_req), ptr(plan.tile_qstart), plan.num_tiles,
        ptr(plan.mask_bits), ptr(plan.mask_word_indptr), ptr(out), ptr(lse_out), hq, hkv, d,
        plan.page_size, sm_scale, wl, ptr(sinks_log2), stream_ptr()), "paged_prefill_attn")
    return out


def pack_masks(masks, kv_lens, device):
    """Pack per-request bool [qo_len, kv_len] masks into the word layout the prefill kernel
    reads: request r starts at word mask_word_indptr[r], row stride ceil(kv_len/32) words.
    Requests without a mask get an all-causal mask synthesised by the caller beforehand."""
    chunks, indptr = [], [0]
    for m, kl in zip(masks, kv_lens):
        words = (int(kl) + 31) // 32
        mm = np.zeros((m.shape[0], words * 32), dtype=bool)
        mm[:, : m.shape[1]] = np.asarray(m, dtype=bool)[:, : words * 32]
        bits = np.packbits(mm.reshape(m.shape[0], words, 32), axis=-1, bitorder="little")
        chunks.append(bits.reshape(-1).view(np.uint32))
        indptr.append(indptr[-1] + m.shape[0] * words)
    flat = np.concatenate(chunks) if chunks else np.zeros(1, dtype=np.uint32)
    return (torch.from_numpy(flat.view(np.int32)).to(device),
            torch.from_numpy(np.asarray(indptr, dtype=np.int64)).to(device))


def build_prefill_plan(batch: AttnBatch, group: int, page_size: int, device, tile_rows: int = 64) -> PrefillPlan:
    tile_req, tile_qstart = plan_prefill_tiles(batch.qo_indptr, group, tile_rows, batch.kv_lens)
    mask_bits = mask_indptr = None
    if batch.masks is not None:
        masks = []
        qlens = np.diff(batch.qo_indptr)
        for r, m in enumerate(batch.masks):
            kl, ql = int(batch.kv_lens[r]), int(qlens[r])
            if m is None:
                qi = np.arange(ql)[:, None]
                m = np.arange(kl)[None, :] < (kl - ql + qi + 1)
            masks.append(np.asarray(m, dtype=bool))
        mask_bits, mask_indptr = pack_masks(masks, batch.kv_lens, device)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(device)
    return PrefillPlan(t(batch.page_indices), t(batch.kv_page_indptr), t(batch.qo_indptr),
                       t(batch.kv_lens), t(tile_req), t(tile_qstart), len(tile_req), page_size,
                       mask_bits, mask_indptr, batch.window_left, tile_rows)


def paged_attention_cpu(q, kv_layer, batch: AttnBatch, sm_scale: float, window_left=None, sinks=None, softcap=0.0):
    masks = None
    if batch.masks is not None:
        masks = [None if m is None else torch.as_tensor(np.asarray(m, dtype=bool)) for m in batch.masks]
    return reference.paged_attention(q, kv_layer, batch.qo_indptr, batch.kv_page_indptr,
                                     torch.as_tensor(batch.page_indices), batch.kv_lens, sm_scale,
                                     masks=masks, window_left=batch.window_left if window_left is None else window_left,
                                     sinks=sinks, softcap=softcap)


# --------------------------------------------------------------------------- sampling
def sample(logits, temperature, top_k, top_p, min_p, seeds, mask_bits=None, mask_row=None, out=None):
    """Draw one token per row of bf16 logits on the device. All parameter tensors are per row
    (float32 / int32 / float32 / float32 / int64 seeds)."""
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    mask_words = mask_bits.shape[1] if mask_bits is not None else 0
    check(fn("pie_sample")(ptr(logits), logits.stride(0), rows, vocab, ptr(temperature), ptr(top_k),
                           ptr(top_p), ptr(min_p), ptr(seeds), ptr(mask_bits), ptr(mask_row),
                           mask_words, ptr(out), stream_ptr()), "sample")
    return out


def row_stats(logits):
    """[rows, 3] fp32: max, log-sum-exp and entropy of the unscaled next-token distribution."""
    if not logits.is_cuda:
        return reference.row_stats(logits)
    rows, vocab = logits.shape
    out = torch.empty(rows, 3, dtype=torch.float32, device=logits.device)
    check(fn("pie_row_stats")(ptr(logits), logits.stride(0), rows, vocab, ptr(out), stream_ptr()),
          "row_stats")
    return out


# --------------------------------------------------------------------------- Gated DeltaNet
def gdn_mixer(mix, lw: dict, cfg, rs, layer: int):
    """The linear-attention mixer of one layer over a ragged batch (see `reference.gdn_mixer` for the math).
    `mix` is the fused input projection [N, q | k | v | z | b | a]; `rs` a `driver.recurrent.RecurrentInputs`;
    the layer's slot states are advanced in place. Returns [N, Hv * dv]."""
    hk, hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
    dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
    if rs is None:
        raise ValueError("a model with Gated DeltaNet layers needs recurrent-state inputs")
    conv_state, rec_state = rs.conv_state[layer], rs.rec_state[layer]
    if not mix.is_cuda:
        return reference.gdn_mixer(mix, lw["gdn_conv"], lw["gdn_A_log"], lw["gdn_dt_bias"], lw["gdn_norm"],
                                   cfg.rms_norm_eps, hk, hv, dk, dv, rs.qo_host, conv_state, rec_state,
                                   rs.slots_host, rs.reset_host)
    n, r = mix.shape[0], len(rs.slots_host)
    out = torch.empty(n, hv * dv, dtype=torch.bfloat16, device=mix.device)
    check(fn("pie_gdn_mixer")(ptr(mix), mix.stride(0), ptr(lw["gdn_conv"]), ptr(lw["gdn_A_log"]), ptr(lw["gdn_dt_bias"]),
                              ptr(lw["gdn_norm"]), ptr(conv_state), ptr(rec_state), ptr(rs.qo_indptr), ptr(rs.tok_req),
                              ptr(rs.slots), ptr(rs.reset), ptr(rs.scratch), ptr(out), n, r, hk, hv, dk, dv,
                              cfg.linear_conv_kernel_dim, cfg.rms_norm_eps, stream_ptr()), "gdn_mixer")
    return out


def gdn_copy_slot(buf, src: int, dst: int) -> None:
    """buf[:, dst] <- buf[:, src] for a [layers, slots, ...] fp32 state cache on the device."""
    layers, slots = buf.shape[0], buf.shape[1]
    slot_elems = buf[0, 0].numel()
    check(fn("pie_gdn_copy_slot")(ptr(buf), slots * slot_elems, slot_elems, layers, src, dst, stream_ptr()), "gdn_copy_slot")


# --------------------------------------------------------------------------- Mamba-2
def mamba2_mixer(mix, lw: dict, cfg, rs, layer: int):
    """The Mamba-2 mixer of one layer over a ragged batch (see `reference.mamba2_mixer`). `mix` is the input
    projection [N, z | x B C | dt]; the layer's slot states are advanced in place. Returns [N, heads * head_dim]."""
    hm, p, ns, g = cfg.mamba_num_heads, cfg.mamba_head_dim, cfg.ssm_state_size, cfg.mamba_n_groups
    if rs is None:
        raise ValueError("a model with Mamba-2 layers needs recurrent-state inputs")
    conv_state, rec_state = rs.conv_state[layer], rs.rec_state[layer]
    if not mix.is_cuda:
        return reference.mamba2_mixer(mix, lw["mamba_conv"], lw["mamba_conv_bias"], lw["mamba_A_log"], lw["mamba_dt_bias"],
                                      lw["mamba_D"], lw["mamba_norm"], cfg.rms_norm_eps, hm, p, ns, g, rs.qo_host,
                                      conv_state, rec_state, rs.slots_host, rs.reset_host,
                                      norm_groups=g if cfg.mamba_norm_grouped else 1)
    n, r, inner = mix.shape[0], len(rs.slots_host), hm * p
    y = torch.empty(n, inner, dtype=torch.float32, device=mix.device)
    check(fn("pie_mamba2_mixer")(ptr(mix), mix.stride(0), ptr(lw["mamba_conv"]), ptr(lw["mamba_conv_bias"]),
                                 ptr(lw["mamba_A_log"]), ptr(lw["mamba_dt_bias"]), ptr(lw["mamba_D"]), ptr(conv_state),
                                 ptr(rec_state), ptr(rs.qo_indptr), ptr(rs.tok_req), ptr(rs.slots), ptr(rs.reset),
                                 ptr(rs.scratch), ptr(y), n, r, hm, p, ns, g, stream_ptr()), "mamba2_mixer")
    # gate and per-group RMSNorm over the inner width (one pass over [N, inner]; the state update above is the cost)
    z = mix[:, :inner].float()
    y = y * torch.nn.functional.silu(z)
    ng = g if cfg.mamba_norm_grouped else 1
    yg = y.view(n, ng, inner // ng)
    yg = yg * torch.rsqrt(yg.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps)
    return (yg.view(n, inner) * lw["mamba_norm"].float()).to(torch.bfloat16)
