"""The library comparator of the headline benchmark: the same decode workload served the way the
reference's CUDA driver serves it, built ONLY from library kernels and none of this repository's:

* GEMMs: cuBLAS through `torch.matmul` (reference: cuBLASLt / cuBLAS, driver/cuda/src/ops/gemm.cpp:326-415)
* attention: FlashInfer FA2 paged decode from the installed `flashinfer` wheel, planned once per step
  on the host and run inside the CUDA graph (reference: driver/cuda/src/ops/attention_flashinfer.cu:714,
  plan :301-312; the tensor-core "prefill-decode" plan of entry.cpp:1032-1039 is used when the GQA
  group is >= 4, as it is the faster of the two)
* RMSNorm / fused add+RMSNorm, Llama-3.1 RoPE, paged KV append, SiLU*up, softmax and top-p sampling:
  FlashInfer's kernels (the reference has its own SIMT kernels for these)
* tensor parallelism: NCCL all-reduce after o_proj and after down_proj
  (driver/cuda/src/model/llama_like.cpp:633-657, 706-742), rank 0 alone holds lm_head, computes the
  full logits and samples (entry.cpp:961), and the sampled tokens are broadcast over NCCL as the next
  step's inputs (executor.cpp:1305-1360)
* the whole step (all-reduces and broadcast included) is one CUDA graph per batch size
  (executor/forward_graph.hpp)

Every rank runs the same loop on the same synthetic plan (SPMD), so no control plane is needed. NCCL
moves all data between GPUs; no library kernel is handed another GPU's memory. The KV content of
the synthetic contexts is random (the timed region is the decode steps, which are complete: KV
append, attention over the true lengths, sampling).

FlashInfer compiles its kernels on first use; `prebuild()` compiles them ahead of time (it works on
a machine without a GPU) into a cache directory that `configure_cache()` selects.
"""
from __future__ import annotations

import math
import os
from pathlib import Path
from typing import List, Optional

import numpy as np
import torch

CACHE_ENV = "FLASHINFER_WORKSPACE_BASE"


def configure_cache(base: Optional[str] = None) -> str:
    """Point FlashInfer's JIT cache at `base` (default: baseline/_ref/fi beside the package's
    repository, which is where `prebuild` puts it) and pin the target architecture. Call before
    importing flashinfer."""
    if base is None:
        base = str(Path(__file__).resolve().parents[2] / "baseline" / "_ref" / "fi")
    os.environ.setdefault(CACHE_ENV, base)
    os.environ.setdefault("FLASHINFER_CUDA_ARCH_LIST", "10.0a")
    return os.environ[CACHE_ENV]


def prebuild(head_dim: int = 128, verbose: bool = True) -> None:
    """Compile every FlashInfer module the arm uses (needs nvcc, not a GPU)."""
    configure_cache()
    import time

    import flashinfer  # noqa: F401
    from flashinfer.activation import get_act_and_mul_module
    from flashinfer.decode import get_batch_decode_module
    from flashinfer.norm import get_norm_module
    from flashinfer.page import get_page_module
    from flashinfer.prefill import get_batch_prefill_module
    from flashinfer.rope import get_rope_module
    from flashinfer.sampling import get_sampling_module
    bf = torch.bfloat16
    jobs = [("page", get_page_module), ("rope", get_rope_module), ("norm", get_norm_module),
            ("silu_and_mul", lambda: get_act_and_mul_module("silu")), ("sampling", get_sampling_module),
            ("decode", lambda: get_batch_decode_module(bf, bf, bf, torch.int32, head_dim, head_dim, 0, False, False)),
            ("decode (tensor cores)", lambda: get_batch_prefill_module("fa2", bf, bf, bf, torch.int32, head_dim, head_dim,
                                                                       0, False, False, False))]
    for name, job in jobs:
        t0 = time.time()
        job()
        if verbose:
            print(f"[library arm] flashinfer module {name}: {time.time() - t0:.1f} s", flush=True)


class LibraryLlama:
    """Llama-architecture decoder shard of one tensor-parallel rank over library kernels."""

    def __init__(self, cfg, device, rank: int, world: int, max_batch: int, num_pages: int, page_size: int = 16,
                 seed: int = 0, tensor_cores: Optional[bool] = None):
        import flashinfer
        self.fi = flashinfer
        self.cfg, self.device, self.rank, self.world = cfg, torch.device(device), rank, world
        self.hq = cfg.num_attention_heads // world
        self.hkv = max(1, cfg.num_key_value_heads // world)
        self.d, self.h = cfg.head_dim, cfg.hidden_size
        self.inter = cfg.intermediate_size // world
        self.page_size, self.max_batch = page_size, max_batch
        g = torch.Generator(device=self.device).manual_seed(seed + 1000 * rank)
        bf = torch.bfloat16

        def w(*shape):
            return (torch.randn(*shape, generator=g, device=self.device, dtype=torch.float32) * 0.02).to(bf)

        self.embed = w(cfg.vocab_size, self.h)
        self.layers = []
        for _ in range(cfg.num_hidden_layers):
            self.layers.append(dict(
                ln1=torch.ones(self.h, dtype=bf, device=self.device), ln2=torch.ones(self.h, dtype=bf, device=self.device),
                wqkv=w((self.hq + 2 * self.hkv) * self.d, self.h), wo=w(self.h, self.hq * self.d),
                w_gate_up=w(2 * self.inter, self.h), w_down=w(self.h, self.inter)))
        self.final_norm = torch.ones(self.h, dtype=bf, device=self.device)
        self.lm_head = w(cfg.vocab_size, self.h) if rank == 0 else None     # rank 0 alone emits logits
        # paged KV, FlashInfer NHD layout: [pages, 2, page, kv heads, d] per layer
        self.kv = [torch.empty(num_pages, 2, page_size, self.hkv, self.d, dtype=bf, device=self.device)
                   for _ in range(cfg.num_hidden_layers)]
        for t in self.kv:
            t.normal_(0.0, 0.5, generator=g)
        self.workspace = torch.empty(256 << 20, dtype=torch.uint8, device=self.device)
        self.indptr_buf = torch.zeros(max_batch + 1, dtype=torch.int32, device=self.device)
        self.indices_buf = torch.zeros(num_pages, dtype=torch.int32, device=self.device)
        self.last_buf = torch.ones(max_batch, dtype=torch.int32, device=self.device)
        if tensor_cores is None:
            tensor_cores = self.hq // self.hkv >= 4
        self.wrapper = flashinfer.BatchDecodeWithPagedKVCacheWrapper(
            self.workspace, "NHD", use_cuda_graph=True, use_tensor_cores=tensor_cores,
            paged_kv_indptr_buffer=self.indptr_buf, paged_kv_indices_buffer=self.indices_buf,
            paged_kv_last_page_len_buffer=self.last_buf)
        # fixed-address step inputs
        self.tokens = torch.zeros(max_batch, dtype=torch.int32, device=self.device)
        self.positions = torch.zeros(max_batch, dtype=torch.int32, device=self.device)
        self.batch_idx = torch.arange(max_batch, dtype=torch.int32, device=self.device)
        self.append_pos = torch.zeros(max_batch, dtype=torch.int32, device=self.device)
        self.temperature = torch.ones(max_batch, dtype=torch.float32, device=self.device)
        self.top_p = torch.ones(max_batch, dtype=torch.float32, device=self.device)
        self.graph = None
        self.sm_scale = 1.0 / math.sqrt(self.d)
        rs = cfg.rope_scaling or {}
        self.rope = dict(rope_scale=float(rs.get("factor", 8.0)), rope_theta=float(cfg.rope_theta),
                         low_freq_factor=float(rs.get("low_freq_factor", 1.0)),
                         high_freq_factor=float(rs.get("high_freq_factor", 4.0)),
                         old_context_len=int(rs.get("original_max_position_embeddings", 8192)))

    # ------------------------------------------------------------------ one decode step
    def plan(self, indptr: np.ndarray, indices: np.ndarray, last_page_len: np.ndarray) -> None:
        """Host-side attention plan of the step (outside the graph, as in the reference)."""
        self.wrapper.plan(torch.from_numpy(indptr), torch.from_numpy(indices), torch.from_numpy(last_page_len),
                          self.hq, self.hkv, self.d, self.page_size, pos_encoding_mode="NONE",
                          q_data_type=torch.bfloat16, kv_data_type=torch.bfloat16, sm_scale=self.sm_scale)

    def _all_reduce(self, x):
        if self.world > 1:
            torch.distributed.all_reduce(x)
        return x

    def step_body(self) -> None:
        """embed -> L x [norm, QKV, RoPE, KV append, attention, o_proj, AR, add+norm, gate/up, SiLU*up,
        down, AR] -> final norm -> (rank 0) lm_head, softmax, top-p sample -> broadcast tokens."""
        fi, b = self.fi, self.max_batch
        qs, ks = self.hq * self.d, self.hkv * self.d
        resid = self.embed.index_select(0, self.tokens)
        x = fi.norm.rmsnorm(resid, self.layers[0]["ln1"], self.cfg.rms_norm_eps)
        for li, lw in enumerate(self.layers):
            qkv = torch.matmul(x, lw["wqkv"].t())
            q = qkv[:, :qs].view(b, self.hq, self.d)
            k = qkv[:, qs:qs + ks].view(b, self.hkv, self.d)
            v = qkv[:, qs + ks:].view(b, self.hkv, self.d)
            fi.rope.apply_llama31_rope_pos_ids_inplace(q, k, self.positions, **self.rope)
            fi.page.append_paged_kv_cache(k, v, self.batch_idx, self.append_pos, self.kv[li], self.indices_buf,
                                          self.indptr_buf, self.last_buf, kv_layout="NHD")
            a = self.wrapper.run(q, self.kv[li])
            o = self._all_reduce(torch.matmul(a.view(b, qs), lw["wo"].t()))
            fi.norm.fused_add_rmsnorm(o, resid, lw["ln2"], self.cfg.rms_norm_eps)      # resid += o; o = norm(resid)
            gu = torch.matmul(o, lw["w_gate_up"].t())
            act = fi.activation.silu_and_mul(gu)
            y = self._all_reduce(torch.matmul(act, lw["w_down"].t()))
            nxt = self.layers[li + 1]["ln1"] if li + 1 < len(self.layers) else self.final_norm
            fi.norm.fused_add_rmsnorm(y, resid, nxt, self.cfg.rms_norm_eps)
            x = y
        if self.rank == 0:
            logits = torch.matmul(x, self.lm_head.t())
            probs = fi.sampling.softmax(logits, temperature=self.temperature)
            tok = fi.sampling.top_p_sampling_from_probs(probs, self.top_p)
            self.tokens.copy_(tok.to(torch.int32))
        if self.world > 1:
            torch.distributed.broadcast(self.tokens, src=0)

    def capture(self) -> None:
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self.step_body()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(self.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.step_body()


def run(cfg, prompt_lens: List[int], out_tokens: int, warmup: int, steps: int, rank: int, world: int, device,
        temperature: float = 1.0, top_p: float = 0.9, page_size: int = 16) -> dict:
    """Device-timed decode of `len(prompt_lens)` synthetic contexts: W untimed + K timed steps,
    bracketed by synchronise (+ barrier) and CUDA events, max over ranks. Every rank calls it."""
    configure_cache()
    dev = torch.device(device)
    r = len(prompt_lens)
    plen = np.asarray(prompt_lens, dtype=np.int64)
    per = (plen + out_tokens + 1 + page_size - 1) // page_size
    num_pages = int(per.sum())
    starts = np.zeros(r + 1, np.int64)
    np.cumsum(per, out=starts[1:])
    maxp = int(per.max())
    table = np.zeros((r, maxp), np.int32)
    for i in range(r):
        table[i, :per[i]] = np.arange(starts[i], starts[i] + per[i], dtype=np.int32)
    cols = np.arange(maxp, dtype=np.int32)[None, :]
    model = LibraryLlama(cfg, dev, rank, world, r, num_pages, page_size)
    model.temperature.fill_(temperature)
    model.top_p.fill_(top_p)
    g = torch.Generator(device="cpu").manual_seed(3)
    model.tokens.copy_(torch.randint(0, cfg.vocab_size, (r,), generator=g, dtype=torch.int32))
    pos_pinned = [torch.zeros(r, dtype=torch.int32).pin_memory() for _ in range(2)]

    def prepare(step: int) -> None:
        kv_before = plen + step
        kv_after = kv_before + 1
        used = (kv_after + page_size - 1) // page_size
        indptr = np.zeros(r + 1, np.int32)
        np.cumsum(used, out=indptr[1:])
        indices = table[cols < used[:, None]]
        last = ((kv_after - 1) % page_size + 1).astype(np.int32)
        model.plan(indptr, indices, last)
        host = pos_pinned[step & 1]
        host.numpy()[:] = kv_before
        model.positions.copy_(host, non_blocking=True)
        model.append_pos.copy_(host, non_blocking=True)

    prepare(0)
    model.capture()
    barrier = torch.distributed.barrier if world > 1 else (lambda: None)
    ev0 = ev1 = None
    for s in range(warmup + steps):
        if s == warmup:
            torch.cuda.synchronize(dev)
            barrier()
            torch.cuda.synchronize(dev)
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        prepare(s)
        model.graph.replay()
    ev1.record()
    torch.cuda.synchronize(dev)
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float32, device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item())
        barrier()
    toks = model.tokens.cpu().numpy()
    ok = bool(((toks >= 0) & (toks < cfg.vocab_size)).all())
    return {"impl": "library", "ms_per_step": ms / steps, "tokens_per_s": r * steps / (ms / 1e3), "tokens_valid": ok,
            "attention": "flashinfer fa2 paged decode" + (" (tensor cores)" if model.wrapper.use_tensor_cores else ""),
            "gemm": "cublas", "collectives": f"nccl all-reduce x2/layer, rank-0 logits, token broadcast (tp{world})"
            if world > 1 else None}


def main():
    """python -m pie_b200.bench.library_arm --prebuild   (compile the FlashInfer modules, no GPU needed)"""
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--prebuild", action="store_true")
    a = ap.parse_args()
    if a.prebuild:
        prebuild()


if __name__ == "__main__":
    main()
