"""The model driver: executes batched forward requests on one GPU (or on the CPU for the
plumbing configuration) and answers with sampled tokens / probe payloads.

Per fire (`TorchDriver.fire_batch`): derive KV lengths and tail-append slots from the CSR
page tables -> fill ONE pinned host slab with every integer/float input (tokens, positions,
slots, indptrs, page ids, split-KV work items, sampler parameters) -> one or two H2D copies
into a fixed-address device slab -> forward (CUDA-graph replay for pure-decode batches padded
to a bucket of the lattice, eager otherwise) -> sampling kernel -> D2H of the sampled tokens.

Behavioural counterpart of the reference's executor
(driver/cuda/src/executor/executor.cpp:2133-2800 handle_fire_batch, :1727-1781 graph
shape decision, executor/persistent_inputs.hpp fixed-address slabs,
executor/forward_graph.hpp:63-91 bucket lattice, sampling_dispatch.cpp:49-137).
Differences by design: logit masks are consumed by the GPU sampler (no host override), all
inputs travel in one slab copy instead of six, and the decode work list is graph-safe
because its length lives in device memory.
"""
from __future__ import annotations

import os
import threading
import time
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from .. import ops
from ..models.config import ModelConfig
from ..models.transformer import ForwardInputs, ParallelContext, Transformer
from ..models.weights import random_weights, torch_dtype
from . import nvtx
from .kv_cache import KVCache
from .schema import (Capabilities, CopyRequest, ForwardRequest, ForwardResponse, SamplerKind, verify_drafts,
                     SamplerSpec, SlotOutput, position_seed)


def graph_buckets(max_requests: int) -> List[int]:
    """Request-count lattice for decode graphs: 1,2,4,8 then steps of 8 to 64, 16 to 256, 32 beyond."""
    out = [b for b in (1, 2, 4, 8) if b <= max_requests]
    b = 16
    while b <= max_requests:
        out.append(b)
        b += 8 if b < 64 else (16 if b < 256 else 32)
    if out[-1] != max_requests:
        out.append(max_requests)
    return out


class _Slab:
    """Named int32 segments in one pinned host buffer mirrored by one device buffer."""

    def __init__(self, segments: Dict[str, int], device):
        self.offsets, off = {}, 0
        for name, n in segments.items():
            off = (off + 3) & ~3  # 16-byte aligned segments
            self.offsets[name] = (off, n)
            off += n
        self.size = off
        cuda = torch.device(device).type == "cuda"
        # two pinned host copies: a pipelined decode step fills one while the H2D copy of the
        # previous step may still be reading the other
        self.hosts = [torch.zeros(self.size, dtype=torch.int32, pin_memory=cuda) for _ in range(2 if cuda else 1)]
        self.host = self.hosts[0]
        self.np = self.host.numpy()
        self.dev = torch.zeros(self.size, dtype=torch.int32, device=device) if cuda else self.host

    def select(self, parity: int) -> None:
        self.host = self.hosts[parity % len(self.hosts)]
        self.np = self.host.numpy()

    def h(self, name, dtype=np.int32):
        o, n = self.offsets[name]
        return self.np[o:o + n].view(dtype)

    def d(self, name, n=None, dtype=torch.int32):
        o, cap = self.offsets[name]
        t = self.dev[o:o + (cap if n is None else n * (2 if dtype == torch.int64 else 1))]
        return t.view(dtype) if dtype != torch.int32 else t

    def upload(self, upto_name: str, extra: Optional[tuple] = None):
        if self.dev is self.host:
            return
        o, n = self.offsets[upto_name]
        end = o + n
        self.dev[:end].copy_(self.host[:end], non_blocking=True)
        if extra is not None:
            name, used = extra
            o2, _ = self.offsets[name]
            if used:
                self.dev[o2:o2 + used].copy_(self.host[o2:o2 + used], non_blocking=True)


@dataclass
class CohortStep:
    """One pure-decode step over r rows in array form (no per-request objects)."""
    r: int
    host_tokens: np.ndarray     # int32 [r] input token when src_row < 0
    src_row: np.ndarray         # int32 [r] row of the previous pipelined step that sampled this row's input
    positions: np.ndarray       # int32 [r]
    kv_lens: np.ndarray         # int32 [r] KV length including this token
    page_indptr: np.ndarray     # int32 [r+1]
    page_indices: np.ndarray    # int32
    temperature: np.ndarray
    top_k: np.ndarray
    top_p: np.ndarray
    min_p: np.ndarray
    seeds: np.ndarray           # int64 [r]


class AsyncTokens:
    """Result handle of `decode_async`: wait() blocks until the step's tokens are on the host."""

    def __init__(self, event, host_buf, r: int, ready: Optional[np.ndarray] = None, driver=None):
        self.event, self.host_buf, self.r, self.ready, self.driver = event, host_buf, r, ready, driver

    def wait(self) -> np.ndarray:
        if self.ready is None:
            self.event.synchronize()
            self.ready = self.host_buf[:self.r].numpy().copy()
            if self.driver is not None:
                self.driver.check_status_host()
        return self.ready


@dataclass
class _Graph:
    graph: "torch.cuda.CUDAGraph"
    logits: torch.Tensor
    bucket: int
    launches: int = 0


class TorchDriver:
    """PyTorch + sm_100a-kernel model driver for one tensor-parallel rank."""

    def __init__(self, cfg: ModelConfig, device="cuda", weights: Optional[dict] = None, num_pages: int = 0,
                 page_size: int = 16, max_requests: int = 512, max_tokens: int = 8192, seed: int = 0,
                 par: Optional[ParallelContext] = None, gemm_backend: str = "tcgen05", use_graphs: bool = True,
                 swap_pages: int = 0, gpu_mem_utilization: float = 0.9, max_kv_tokens_per_request: int = 0,
                 memory_profile: str = "", kv_dtype: str = "auto", rs_slots: int = 0, vision=None, audio=None):
        self.cfg = cfg
        self.device = torch.device(device)
        if self.device.type == "cuda" and self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.cuda = self.device.type == "cuda"
        self._bound = threading.local()
        self.adapters: dict = {}
        self._lora_bindings = None
        self.dtype = torch_dtype(cfg.dtype) if not self.cuda else torch.bfloat16
        self.par = par or ParallelContext()
        if self.cuda:
            torch.cuda.set_device(self.device)
        if weights is None:
            weights = random_weights(cfg, self.device, self.dtype, seed, self.par.tp_size, self.par.tp_rank,
                                     ep=self.par.ep)
        self.model = Transformer(cfg, weights, self.device, self.dtype, self.par, gemm_backend)
        self.page_size = page_size
        hkv = self.model.hkv
        self.kv_dtype = kv_dtype
        self.memory_plan = None
        if num_pages <= 0:
            num_pages, max_requests, max_tokens = self._plan_memory(gpu_mem_utilization, memory_profile, max_requests,
                                                                    max_tokens)
            if self.par.tp_size > 1:
                # page ids are global to the replica: every rank must hold the same number of pages
                import torch.distributed as dist
                if dist.is_available() and dist.is_initialized():
                    t = torch.tensor([num_pages], dtype=torch.int64, device=self.device)
                    dist.all_reduce(t, op=dist.ReduceOp.MIN)
                    num_pages = int(t.item())
        self.kv = KVCache(cfg.num_hidden_layers, num_pages, hkv, page_size, cfg.head_dim, self.dtype,
                          self.device, swap_pages, kv_dtype=kv_dtype)
        self.model.kv_scale = self.kv.scale
        # Gated DeltaNet layers keep their state in slots of a recurrent-state cache, one per resident context
        self.rs = None
        if cfg.recurrent_layers:
            if self.par.tp_size > 1:
                raise NotImplementedError("recurrent (Gated DeltaNet / Mamba-2) layers under tensor parallelism")
            from .recurrent import RecurrentStateCache
            self.rs = RecurrentStateCache(cfg, rs_slots or max(2 * max_requests, 16), self.device)
        # media: a vision encoder (models.vision.VisionEncoder) and the clips it has encoded, by the runtime's slot
        self.vision, self.audio = vision, audio
        self.media: Dict[int, torch.Tensor] = {}
        for enc in (vision, audio):
            if enc is not None and enc.cfg.hidden_size != cfg.hidden_size:
                raise ValueError(f"media encoder output width {enc.cfg.hidden_size} != model width {cfg.hidden_size}")
        # soft-capped attention scores (Gemma-2): bf16 pages, the 64-row prefill kernel, no shared-prefix decode plans
        self.softcap = bool(cfg.attn_softcap)
        if self.softcap and kv_dtype == "fp8_e4m3":
            raise NotImplementedError("fp8 KV pages with soft-capped attention scores")
        self.max_requests, self.max_tokens = max_requests, max_tokens
        self.max_page_refs = max(4096, min(num_pages * 2, 1 << 22))
        self.num_ctas = ops.num_sms(self.device) * 2 if self.cuda else 1
        # the widest window any layer needs (-1: some layer sees everything); layers that differ mask per call
        self.window_left = self.cfg.plan_window_left
        self.max_items = max_requests + self.num_ctas * 8
        # shared-prefix decode plans: forks of one context read their common pages once per step
        import os as _os
        self._prefix_cache: dict = {}
        self.cascade = (self.cuda and _os.environ.get("PIE_CASCADE", "1") != "0" and self.window_left < 0
                        and self.cfg.layer_types is None and self.kv.scale is None and not self.softcap)
        rows = max(max_requests, 1024)
        self.max_rows = rows
        self.slab = _Slab({
            "tokens": max_tokens, "positions": max_tokens, "slots": max_tokens,
            "qo_indptr": max_requests + 1, "kv_page_indptr": max_requests + 1, "kv_lens": max_requests,
            "item_req": self.max_items, "item_start": self.max_items, "item_end": self.max_items,
            "req_item_indptr": max_requests + 1, "num_items": 4,
            "item_slot": self.max_items, "item_tile": self.max_items, "tile_members": 16 * max_requests,
            "logit_rows": rows, "temperature": rows, "top_k": rows, "top_p": rows, "min_p": rows,
            "mask_row": rows, "seeds": 2 * rows, "src_row": rows, "rs_slots": max_requests, "rs_reset": max_requests,
            "tile_req": max_tokens + max_requests, "tile_qstart": max_tokens + max_requests,
            "page_indices": self.max_page_refs,
        }, self.device)
        self.scratch = None
        if self.cuda:
            self.scratch = torch.empty(ops.decode_scratch_floats(self.max_items, self.model.hq, cfg.head_dim),
                                       dtype=torch.float32, device=self.device)
            self.sampled = torch.zeros(rows, dtype=torch.int32, device=self.device)
            self.sampled_host = torch.zeros(rows, dtype=torch.int32, pin_memory=True)
            self.cohort_sampled = [torch.zeros(rows, dtype=torch.int32, device=self.device) for _ in range(2)]
            self.cohort_host = [torch.zeros(rows, dtype=torch.int32, pin_memory=True) for _ in range(2)]
            self.status_host = torch.zeros(8, dtype=torch.int32, pin_memory=True)
        self._failed: Optional[str] = None
        # Fires come from the scheduler thread, page copies (fork, swap) from the threads of the
        # inferlets: one lock keeps "publish to the tensor-parallel followers + launch here" atomic, so
        # that every rank sees the same order of fires and copies and the control ring has one writer
        # at a time.
        self._order = threading.RLock()
        self.bounds_check = os.environ.get("PIE_BOUNDS", "0") == "1"
        self.use_graphs = use_graphs and self.cuda
        self.buckets = graph_buckets(max_requests)
        self.graphs: Dict[int, _Graph] = {}
        self.rng = np.random.default_rng(seed + 12345)
        self.stats = {"fires": 0, "graph_replays": 0, "eager": 0, "kernel_launches": 0}

    # ------------------------------------------------------------------ planning
    def _plan_memory(self, util: float, profile: str, max_requests: int, max_tokens: int):
        """KV pages (and, with a named profile, the forward limits) from what the device has left once
        the weights are resident: `driver.memory_planner` splits `util` of the device between the
        activation arena of the largest pass and the page pool. Without a profile the caller's limits
        stand and only the page count is planned. Returns (pages, max_requests, max_tokens)."""
        from . import memory_planner as mp
        if not self.cuda:
            return 4096, max_requests, max_tokens
        free, total = torch.cuda.mem_get_info(self.device)
        usable = int(total * util) - (total - free)          # what `util` of the device leaves beside the weights
        tp = self.par.tp_size
        if profile:
            plan = mp.plan(self.cfg, usable, 1.0, profile, self.page_size, tp)
            max_requests, max_tokens = plan.max_requests, plan.max_tokens
        else:
            arena = mp.arena_bytes(self.cfg, max_tokens, max_requests, tp)
            per_page = mp.kv_bytes_per_page(self.cfg, self.page_size, tp)
            if self.kv_dtype == "fp8_e4m3":       # one byte per element + an fp32 scale per row
                per_page = int(per_page * (0.5 + 2.0 / self.cfg.head_dim))
            pages = max(0, (usable - arena - (4 << 30)) // per_page)     # 4 GiB for the graphs' private pools and workspaces
            plan = mp.MemoryPlan("explicit", self.page_size, int(pages), max_requests, max_tokens, 0, arena,
                                 int(pages) * per_page)
        self.memory_plan = plan
        return max(64, plan.kv_pages), max_requests, max_tokens

    # ------------------------------------------------------------------ adapters
    def create_adapter(self, adapter_id: int, rank: int, alpha: float, seed: int = 0) -> None:
        from .lora import LoraAdapter
        if self.par.tp_size > 1:
            raise NotImplementedError("LoRA adapters are served by single-GPU replicas")
        self.adapters[adapter_id] = LoraAdapter(self.cfg, rank, alpha, self.device, self.dtype, self.model.hq,
                                                self.model.hkv, seed)

    def destroy_adapter(self, adapter_id: int) -> None:
        self.adapters.pop(adapter_id, None)

    def fork_adapter(self, src: int, dst: int) -> None:
        a = self.adapters[src]
        self.create_adapter(dst, a.rank, a.alpha)
        self.adapters[dst].copy_from(a)

    def save_adapter(self, adapter_id: int, path: str) -> None:
        from safetensors.torch import save_file
        a = self.adapters[adapter_id]
        save_file({k: v.detach().float().cpu().contiguous() for k, v in a.tensors().items()}, path,
                  metadata={"rank": str(a.rank), "alpha": str(a.alpha)})

    def load_adapter(self, adapter_id: int, path: str) -> None:
        from safetensors import safe_open
        with safe_open(path, framework="pt", device="cpu") as f:
            meta = f.metadata() or {}
            self.create_adapter(adapter_id, int(meta.get("rank", 8)), float(meta.get("alpha", 16.0)))
            self.adapters[adapter_id].load_tensors({k: f.get_tensor(k) for k in f.keys()})

    def zo_apply(self, adapter_id: int, seed: int, coeff: float) -> None:
        self.adapters[adapter_id].zo_apply(seed, coeff)

    def _bind_adapters(self, req: ForwardRequest):
        ids = req.adapter_ids
        if ids is None or not self.adapters or not (np.asarray(ids) >= 0).any():
            return None
        qo = np.asarray(req.qo_indptr)
        out = []
        for aid in sorted(set(int(a) for a in ids if a >= 0)):
            if aid not in self.adapters:
                raise KeyError(f"unknown adapter {aid}")
            rows = np.concatenate([np.arange(qo[i], qo[i + 1]) for i in range(len(ids)) if ids[i] == aid])
            out.append((self.adapters[aid], torch.from_numpy(rows.astype(np.int64)).to(self.device)))
        return out

    def _bind_thread(self) -> None:
        """The current CUDA device is per thread; the scheduler thread that calls into the driver
        starts on device 0, so every entry point selects this driver's device first."""
        if self.device.type == "cuda" and getattr(self._bound, "idx", None) != self.device.index:
            torch.cuda.set_device(self.device)
            self._bound.idx = self.device.index

    def capabilities(self) -> Capabilities:
        return Capabilities(
            total_pages=self.kv.num_pages, kv_page_size=self.page_size, swap_pool_size=self.kv.swap_pages,
            max_forward_tokens=self.max_tokens, max_forward_requests=self.max_requests,
            max_page_refs=self.max_page_refs, max_logit_rows=self.max_rows, max_prob_rows=self.max_rows,
            max_sampler_rows=self.max_rows, arch_name=self.cfg.model_type, vocab_size=self.cfg.vocab_size,
            max_model_len=self.cfg.max_position_embeddings, activation_dtype=str(self.dtype).replace("torch.", ""),
            tp_size=self.par.tp_size, rs_cache_slots=self.rs.num_slots if self.rs is not None else 0,
            cohort_decode=self.rs is None, media_spec=self._media_spec(),
            media=(("image", "video") if self.vision is not None else ()) + (("audio",) if self.audio is not None else ()))

    # ------------------------------------------------------------------ request -> slab
    def _derive(self, req: ForwardRequest):
        page = self.page_size
        qo = np.asarray(req.qo_indptr, dtype=np.int64)
        qlens = np.diff(qo)
        pptr = np.asarray(req.kv_page_indptr, dtype=np.int64)
        npages = np.diff(pptr)
        kv_lens = np.where(npages > 0, (npages - 1) * page + np.asarray(req.kv_last_page_lens, dtype=np.int64), 0)
        n = int(qo[-1])
        req_of_tok = np.repeat(np.arange(len(qlens)), qlens)
        j = np.arange(n) - qo[req_of_tok]
        kvidx = kv_lens[req_of_tok] - qlens[req_of_tok] + j
        pages = np.asarray(req.kv_page_indices, dtype=np.int64)
        if n and (kvidx < 0).any():
            raise ValueError("KV_INVARIANT_VIOLATION: more input tokens than KV slots")
        slots = pages[pptr[req_of_tok] + kvidx // page] * page + kvidx % page if n else np.zeros(0, np.int64)
        return qlens, kv_lens, slots

    def _fill_common(self, req, slots, kv_lens, n_pad_tokens=0, r_pad=0):
        s = self.slab
        n, r = req.num_tokens, req.num_requests
        if n + n_pad_tokens > self.max_tokens or r + r_pad > self.max_requests:
            raise ValueError("batch exceeds the advertised forward limits")
        if len(req.kv_page_indices) > self.max_page_refs:
            raise ValueError("batch exceeds max_page_refs")
        s.h("tokens")[:n] = req.tokens
        s.h("positions")[:n] = req.positions
        s.h("slots")[:n] = slots
        s.h("qo_indptr")[:r + 1] = req.qo_indptr
        s.h("kv_page_indptr")[:r + 1] = req.kv_page_indptr
        s.h("kv_lens")[:r] = kv_lens
        s.h("page_indices")[:len(req.kv_page_indices)] = req.kv_page_indices

    def _validate_request(self, req: ForwardRequest, slots) -> None:
        """`PIE_BOUNDS=1`: check every index table of the fire against its range before any kernel that
        trusts it runs (token ids, page indices, last-page lengths, KV write slots, logit rows). A bad
        entry fails the fire with the table and position; no kernel reads through it."""
        dev = self.device
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
        pages = self.kv.num_pages
        ops.validate_indices(t(req.tokens), 0, self.cfg.vocab_size, "tokens")
        ops.validate_indices(t(req.positions), 0, 1 << 30, "positions")
        ops.validate_indices(t(req.kv_page_indices), 0, pages, "kv_page_indices")
        ops.validate_indices(t(req.kv_last_page_lens), 1, self.page_size + 1, "kv_last_page_lens")
        ops.validate_indices(t(slots), 0, pages * self.page_size, "kv_slots")
        if req.slot_row is not None and len(req.slot_row):
            ops.validate_indices(t(req.slot_row), 0, max(1, req.num_tokens), "logit_rows")
        if self.cuda:
            torch.cuda.current_stream().synchronize()
            ops.check_kernel_status(dev)

    def _sampler_params(self, req: ForwardRequest, rows_of_slot: np.ndarray):
        """Fill per-row sampler parameter segments for the token-sampler slots."""
        s = self.slab
        token_slots = [i for i, sp in enumerate(req.slot_samplers) if sp.is_token]
        k = len(token_slots)
        if k > self.max_rows:
            raise ValueError("too many sampler rows")
        t, tk = s.h("temperature", np.float32), s.h("top_k")
        tp, mp = s.h("top_p", np.float32), s.h("min_p", np.float32)
        seeds = s.h("seeds", np.int64)
        for j, i in enumerate(token_slots):
            sp = req.slot_samplers[i]
            t[j] = sp.temperature
            tk[j] = sp.top_k if sp.kind in (SamplerKind.TOP_K, SamplerKind.TOP_K_TOP_P) else 0
            tp[j] = sp.top_p if sp.kind in (SamplerKind.TOP_P, SamplerKind.TOP_K_TOP_P) else 1.0
            mp[j] = sp.min_p if sp.kind == SamplerKind.MIN_P else 0.0
            if sp.seed and sp.seed_final:
                seeds[j] = sp.seed
            elif sp.seed:
                # a user-fixed seed is mixed with the position of the sampled row, as the cohort does
                row = int(req.slot_row[i]) if req.slot_row is not None else -1
                pos = int(req.positions[row]) if 0 <= row < len(req.positions) else 0
                seeds[j] = int(position_seed(sp.seed, pos))
            else:
                seeds[j] = int(self.rng.integers(1, 2**62))
        return token_slots

    # ------------------------------------------------------------------ forward variants
    def _forward_inputs_decode(self, rb: int, cascade: bool = False) -> ForwardInputs:
        s = self.slab
        plan = ops.DecodePlan(
            page_indices=s.d("page_indices"), kv_page_indptr=s.d("kv_page_indptr"), item_req=s.d("item_req"),
            item_start=s.d("item_start"), item_end=s.d("item_end"), req_item_indptr=s.d("req_item_indptr"),
            num_items=s.d("num_items"), scratch=self.scratch, max_items=self.max_items, num_reqs=rb,
            num_ctas=self.num_ctas, page_size=self.page_size, window_left=self.window_left)
        if cascade:
            plan.item_slot, plan.item_tile, plan.tile_members = s.d("item_slot"), s.d("item_tile"), s.d("tile_members")
        return ForwardInputs(tokens=s.d("tokens", rb), positions=s.d("positions", rb), slots=s.d("slots", rb),
                             attn=plan, logit_rows=None, is_decode=True,
                             rs=self._rs_inputs_decode(rb) if self.rs is not None else None)

    def _rs_inputs_decode(self, rb: int):
        """Recurrent-state inputs of a decode step over `rb` rows at fixed addresses (a graph replays them): one token
        per request, slots and reset flags in the slab; a row whose slot is -1 is padding and the mixers skip it."""
        cache = self.__dict__.setdefault("_rs_decode", {})
        if rb not in cache:
            from .recurrent import RecurrentInputs
            s, dev = self.slab, self.device
            scratch = torch.empty(rb, self.rs.conv_channels, dtype=torch.float32, device=dev) if self.cuda else None
            cache[rb] = RecurrentInputs(
                torch.arange(rb + 1, dtype=torch.int32, device=dev), torch.arange(rb, dtype=torch.int32, device=dev),
                s.d("rs_slots", rb), s.d("rs_reset", rb), list(range(rb + 1)), [-1] * rb, [0] * rb,
                self.rs.conv_state, self.rs.rec_state, self.rs.layer_index, scratch)
        return cache[rb]

    def _fill_rs_decode(self, req: ForwardRequest, r: int, rb: int) -> None:
        s = self.slab
        if req.rs_slots is None or len(req.rs_slots) != r:
            raise ValueError("this model has recurrent layers: every request needs a recurrent-state slot")
        slots = np.asarray(req.rs_slots, dtype=np.int32)
        if len(slots) and (slots.min() < 0 or slots.max() >= self.rs.num_slots):
            raise ValueError(f"recurrent-state slot outside 0..{self.rs.num_slots - 1}")
        if len(np.unique(slots)) != len(slots):
            raise ValueError("two requests of one fire share a recurrent-state slot")
        s.h("rs_slots")[:r] = slots
        s.h("rs_slots")[r:rb] = -1
        s.h("rs_reset")[:r] = req.rs_reset if req.rs_reset is not None else 0
        s.h("rs_reset")[r:rb] = 0

    def _plan_decode(self, kv_lens, page_indptr, page_indices, r: int, rb: int) -> bool:
        """Fill the slab's decode work list for `r` requests padded to `rb`. Returns True when the plan
        has shared-prefix items (forks of one context: their common pages are then read once per
        tile of members instead of once per request), which selects the cascade graph variant."""
        s = self.slab
        plan = None
        if self.cascade and r >= 2:
            groups = ops.find_shared_prefixes(kv_lens, page_indptr, page_indices, self.page_size,
                                              cache=self._prefix_cache)
            if groups:
                plan = ops.plan_decode_cascade(kv_lens, groups, self.model.hkv, self.model.hq // self.model.hkv,
                                               self.num_ctas, self.max_items)
        if plan is not None and len(plan.tile_members) <= self.max_requests:
            ni = len(plan.item_req)
            s.h("item_req")[:ni], s.h("item_start")[:ni], s.h("item_end")[:ni] = plan.item_req, plan.item_start, plan.item_end
            s.h("item_slot")[:ni], s.h("item_tile")[:ni] = plan.item_slot, plan.item_tile
            nt = plan.tile_members.size
            s.h("tile_members")[:nt] = plan.tile_members.reshape(-1)
            indptr = plan.req_slot_indptr
            self.stats["cascade_steps"] = self.stats.get("cascade_steps", 0) + 1
            self.stats["cascade_tokens_saved"] = self.stats.get("cascade_tokens_saved", 0) + plan.shared_tokens
        else:
            plan = None
            item_req, st, en, indptr = ops.plan_decode_items(kv_lens, self.model.hkv, self.num_ctas, self.max_items,
                                                             window_left=self.window_left)
            ni = len(item_req)
            s.h("item_req")[:ni], s.h("item_start")[:ni], s.h("item_end")[:ni] = item_req, st, en
        s.h("req_item_indptr")[:r + 1] = indptr
        s.h("req_item_indptr")[r + 1:rb + 1] = indptr[-1]
        s.h("num_items")[0] = ni
        return plan is not None

    @staticmethod
    def _gkey(rb: int, cascade: bool):
        return (rb, "cascade") if cascade else rb

    def _capture(self, rb: int, cascade: bool = False) -> _Graph:
        fi = self._forward_inputs_decode(rb, cascade)
        # warm-up on a side stream (sets kernel attributes, fills allocator pools), then capture
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self.model.forward(fi, self.kv.data)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(self.device)
        from ..ops import _lib
        g = torch.cuda.CUDAGraph()
        before = _lib.LAUNCHES
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            logits = self.model.forward(fi, self.kv.data)
        # the decode-attention launcher issues two kernels (split-KV pass + merge) per layer
        return _Graph(g, logits, rb, _lib.LAUNCHES - before + self.cfg.num_hidden_layers)

    def precapture_graphs(self, buckets: Optional[List[int]] = None, cascade: bool = False) -> int:
        """Capture the decode graphs of the bucket lattice ahead of the first request, so that no fire
        pays for a capture (`cascade`: the variant for plans with shared-prefix items; it is captured on
        first use otherwise). The reference pre-captures its lattice at start-up too (
        driver/cuda/src/entry.cpp, executor/forward_graph.hpp:63-91). The capture runs on a plan
        without attention work or KV writes. Returns the number of graphs captured.
        Under tensor parallelism EVERY rank must call this at the same point of its start-up (before
        the followers enter their loop): the warm-up forwards of a capture run the fused kernels,
        which wait for their peers."""
        if not self.use_graphs:
            return 0
        self._bind_thread()
        s, n = self.slab, 0
        for rb in (buckets or self.buckets):
            key = self._gkey(rb, cascade)
            if key in self.graphs or rb > self.max_requests:
                continue
            s.h("tokens")[:rb] = 0
            s.h("positions")[:rb] = 0
            s.h("slots")[:rb] = -1
            s.h("rs_slots")[:rb] = -1          # every row is padding: the capture's forwards touch no recurrent state
            s.h("kv_page_indptr")[:rb + 1] = 0
            s.h("req_item_indptr")[:rb + 1] = 0
            s.h("num_items")[0] = 0
            s.upload("tile_qstart")
            self.graphs[key] = self._capture(rb, cascade)
            n += 1
        torch.cuda.synchronize(self.device)
        ops.kernel_status(self.device).zero_()
        return n

    def _bucket(self, r: int) -> int:
        for b in self.buckets:
            if b >= r:
                return b
        return self.buckets[-1]

    def _run_decode(self, req: ForwardRequest, slots, kv_lens) -> torch.Tensor:
        s = self.slab
        r = req.num_requests
        rb = self._bucket(r) if self.use_graphs else r
        self._fill_common(req, slots, kv_lens, n_pad_tokens=rb - r, r_pad=rb - r)
        if rb > r:  # padding requests: token 0 at position 0, no KV write, no attention work
            s.h("tokens")[r:rb] = 0
            s.h("positions")[r:rb] = 0
            s.h("slots")[r:rb] = -1
            s.h("kv_page_indptr")[r + 1:rb + 1] = req.kv_page_indptr[-1]
        cascade = self._plan_decode(kv_lens, np.asarray(req.kv_page_indptr), np.asarray(req.kv_page_indices), r, rb)
        if self.rs is not None:
            self._fill_rs_decode(req, r, rb)
        s.upload("tile_qstart", ("page_indices", len(req.kv_page_indices)))
        if self.use_graphs:
            key = self._gkey(rb, cascade)
            if key not in self.graphs:
                if self.rs is not None:
                    # the capture runs the forward for real (twice to warm up): attention KV writes repeat harmlessly,
                    # a recurrent state would advance, so the rows are padding while it runs
                    s.h("rs_slots")[:rb] = -1
                    s.upload("tile_qstart", ("page_indices", len(req.kv_page_indices)))
                self.graphs[key] = self._capture(rb, cascade)
                if self.rs is not None:
                    self._fill_rs_decode(req, r, rb)
                s.upload("tile_qstart", ("page_indices", len(req.kv_page_indices)))
            g = self.graphs[key]
            g.graph.replay()
            self.stats["graph_replays"] += 1
            return g.logits
        self.stats["eager"] += 1
        return self.model.forward(self._forward_inputs_decode(rb, cascade), self.kv.data)

    def _mask_rows_for_request(self, req: ForwardRequest, r: int, ql: int, kl: int):
        if req.has_user_mask is not None and req.has_user_mask[r]:
            a, b = int(req.mask_row_indptr[r]), int(req.mask_row_indptr[r + 1])
            return req.mask_runs[a:b]
        return [[0, kl - ql + i + 1] for i in range(ql)]

    def _host_batch(self, req: ForwardRequest, qlens, kv_lens, custom: bool):
        """The fire's attention work as host arrays (and boolean masks): the form the torch statement of the op takes."""
        masks = None
        if custom:
            from ..ops.reference import brle_to_bool
            masks = []
            for i in range(req.num_requests):
                ql, kl = int(qlens[i]), int(kv_lens[i])
                if req.has_user_mask[i]:
                    runs = self._mask_rows_for_request(req, i, ql, kl)
                    masks.append(np.stack([brle_to_bool(rr, kl).numpy() for rr in runs]) if ql else None)
                else:
                    masks.append(None)
        return ops.AttnBatch(np.asarray(req.qo_indptr), np.asarray(req.kv_page_indptr),
                             np.asarray(req.kv_page_indices), kv_lens, masks, self.window_left)

    def _run_general(self, req: ForwardRequest, qlens, slots, kv_lens) -> torch.Tensor:
        s = self.slab
        n, r = req.num_tokens, req.num_requests
        self._fill_common(req, slots, kv_lens)
        custom = req.has_user_mask is not None and bool(np.any(req.has_user_mask))
        rows = np.asarray(req.slot_row, dtype=np.int32) if req.slot_row is not None else np.zeros(0, np.int32)
        # compact logit rows: slots that read the same token row share one row of the vocabulary projection
        rows, self._slot_logit_row = np.unique(rows, return_inverse=True)
        rows = rows.astype(np.int32)
        self.stats["logit_rows"] = self.stats.get("logit_rows", 0) + len(rows)
        if self.cuda:
            group = self.model.hq // self.model.hkv
            tile_rows = ops.prefill_tile_rows(self.model.hq, self.model.hkv, self.model.cfg.head_dim, self.page_size,
                                              softcap=self.softcap)
            tile_req, tile_q = ops.plan_prefill_tiles(np.asarray(req.qo_indptr), group, tile_rows, kv_lens)
            nt = len(tile_req)
            s.h("tile_req")[:nt], s.h("tile_qstart")[:nt] = tile_req, tile_q
            s.h("logit_rows")[:len(rows)] = rows
            s.upload("tile_qstart", ("page_indices", len(req.kv_page_indices)))
            mask_bits = mask_indptr = None
            if custom:
                # every mask row of the fire in one expansion: rows of a request back to back, each ceil(kv_len / 32) words
                all_rows, row_bits, indptr = [], [], [0]
                for i in range(r):
                    ql, kl = int(qlens[i]), int(kv_lens[i])
                    if ql:
                        all_rows.extend(self._mask_rows_for_request(req, i, ql, kl))
                        row_bits.extend([kl] * ql)
                    indptr.append(indptr[-1] + ql * ((kl + 31) // 32))
                mask_bits, _ = ops.brle_expand_ragged(all_rows, row_bits, self.device)
                mask_indptr = torch.tensor(indptr, dtype=torch.int64, device=self.device)
            plan = ops.PrefillPlan(s.d("page_indices"), s.d("kv_page_indptr"), s.d("qo_indptr"), s.d("kv_lens"),
                                   s.d("tile_req"), s.d("tile_qstart"), nt, self.page_size, mask_bits, mask_indptr,
                                   window_left=self.window_left, tile_rows=tile_rows)
            fi = ForwardInputs(s.d("tokens", n), s.d("positions", n), s.d("slots", n), plan,
                               logit_rows=s.d("logit_rows", len(rows)), is_decode=False,
                               attn_num_pages=len(req.kv_page_indices))
        else:
            batch = self._host_batch(req, qlens, kv_lens, custom)
            fi = ForwardInputs(torch.from_numpy(np.ascontiguousarray(req.tokens, dtype=np.int32)),
                               torch.from_numpy(np.ascontiguousarray(req.positions, dtype=np.int32)),
                               torch.from_numpy(slots.astype(np.int32)), batch,
                               logit_rows=torch.from_numpy(rows), is_decode=False)
        self.stats["eager"] += 1
        fi.lora = self._lora_bindings
        if req.media_slot is not None and len(req.media_slot):
            fi.media = self._media_inputs(req)
        if self.rs is not None:
            if req.spec_counts is not None and np.any(req.spec_counts):
                raise ValueError("draft tokens on a model with recurrent layers: a rejected draft cannot be rolled "
                                 "out of the recurrent state")
            fi.rs = self.rs.inputs(req.qo_indptr, req.rs_slots, req.rs_reset)
        hidden = self.model.forward_hidden(fi, self.kv.data)
        if len(rows) == 0:
            return None
        return self.model.logits(hidden, fi)

    def _media_spec(self) -> dict:
        spec: dict = {}
        v = self.vision
        if v is not None:
            c = v.cfg
            if hasattr(c, "mm_tokens_per_image"):          # fixed-resolution SigLIP tower (Gemma-3)
                # the rows of one image attend to each other in both directions (Gemma-3)
                spec = {"style": "siglip", "image_size": c.image_size, "patch": c.patch_size, "pool": c.pool, "bidirectional": True}
            else:
                spec = {"style": "qwen", "patch": c.patch_size, "merge": c.spatial_merge_size, "temporal": c.temporal_patch_size}
        # the text a clip is wrapped in (the model's own span markers), per kind: {"image": [before, after], ...}
        marks = {}
        for kinds, enc in ((("image", "video"), v), (("audio",), self.audio)):
            d = getattr(enc, "delimiters", None)
            if d and (d[0] or d[1]):
                marks.update({k: [d[0], d[1]] for k in kinds})
        if marks:
            spec["delimiters"] = marks
        return spec

    def put_media(self, slot: int, kind: str, patches, grids) -> int:
        """Encode a clip and keep the encoder's output on the device under `slot`; forward requests then name it in
        their media spans. Images and video: patch rows + their (t, h, w) grids (`runtime.multimodal.patchify`);
        audio: the log-mel spectrogram [n_mels, frames] (`grids` unused). Returns the number of rows (placeholder
        tokens). Counterpart of the image / audio side channels of the reference's forward request
        (driver/bridge/src/schema.rs, driver/cuda/src/model/qwen3_vl_vision.cpp)."""
        enc = self.audio if kind == "audio" else self.vision if kind in ("image", "video") else None
        if enc is None:
            raise ValueError(f"this driver has no encoder for {kind}")
        grids = [tuple(int(x) for x in g) for g in grids]
        if enc is self.vision and hasattr(enc.cfg, "mm_tokens_per_image"):
            grids = [(1, h, w) for t, h, w in grids for _ in range(t)]      # every frame is an image of its own
        self._bind_thread()
        if self.cuda:
            # the encoder runs on a stream of its own, outside the lock that orders fires: decode steps of other requests
            # go on while a clip is encoded; the rows are published once they are complete
            stream = self.__dict__.get("_media_stream")
            if stream is None:
                stream = self._media_stream = torch.cuda.Stream(self.device)
            with torch.cuda.stream(stream):
                feats = enc(np.asarray(patches, dtype=np.float32), grids).to(self.dtype).contiguous()
            stream.synchronize()
        else:
            feats = enc(np.asarray(patches, dtype=np.float32), grids).to(self.dtype).contiguous()
        with self._order:
            self.media[int(slot)] = feats
        return int(feats.shape[0])

    def release_media(self, slot: int) -> None:
        with self._order:
            self.media.pop(int(slot), None)

    def _media_inputs(self, req: ForwardRequest):
        out = []
        for sl, src, dst, cnt in zip(req.media_slot, req.media_src, req.media_dst, req.media_count):
            feats = self.media.get(int(sl))
            if feats is None or int(src) + int(cnt) > feats.shape[0]:
                raise ValueError(f"media slot {int(sl)} rows {int(src)}+{int(cnt)}: no such encoded clip on this driver")
            out.append((feats, int(src), int(dst), int(cnt)))
        return out

    def copy_rs(self, src_slot: int, dst_slot: int) -> None:
        """Recurrent-state slot copy (a forked context starts from its parent's state)."""
        if self.rs is None:
            return
        with self._order:
            self._bind_thread()
            self.rs.copy_slot(int(src_slot), int(dst_slot))

    # ------------------------------------------------------------------ sampling + response
    def _respond(self, req: ForwardRequest, logits: Optional[torch.Tensor], slot_logit_row: np.ndarray):
        nslots = len(req.slot_samplers)
        if nslots == 0:
            return ForwardResponse(slots=[], tokens=np.zeros(0, np.int32))
        token_slots = self._token_slots
        out_slots: List[Optional[SlotOutput]] = [None] * nslots
        tokens = None
        if token_slots:
            rows = slot_logit_row[token_slots]
            k = len(token_slots)
            contiguous = bool((rows == np.arange(k)).all()) and k <= logits.shape[0]
            lg = logits[:k] if contiguous else logits[torch.from_numpy(rows.astype(np.int64)).to(logits.device)]
            mask_bits, mask_row = self._logit_mask_rows(req, token_slots)
            if self.cuda:
                self._sample(lg, k, mask_bits, mask_row, self.sampled)
                self.sampled_host[:k].copy_(self.sampled[:k], non_blocking=True)
                self.status_host.copy_(ops.kernel_status(self.device), non_blocking=True)
                torch.cuda.current_stream().synchronize()
                tokens = self.sampled_host[:k].numpy().copy()
                self.check_status_host()
            else:
                tokens = self._sample_cpu(lg, k, mask_bits, mask_row)
            for j, i in enumerate(token_slots):
                out_slots[i] = SlotOutput("token", token=int(tokens[j]))
        probe_slots = [i for i in range(nslots) if out_slots[i] is None]
        if probe_slots:
            self._probes(req, logits, slot_logit_row, probe_slots, out_slots)
        all_tokens = tokens if len(token_slots) == nslots else None
        resp = ForwardResponse(slots=out_slots, tokens=all_tokens)
        if req.spec_counts is not None and token_slots and np.any(req.spec_counts):
            resp.spec_accepted = verify_drafts(req, {int(req.slot_row[i]): int(tokens[j])
                                                     for j, i in enumerate(token_slots)})
        return resp

    def _sample(self, lg, k: int, mask_bits, mask_row, out):
        """Token sampler over `k` logit rows: the single-GPU kernel, or under fused tensor
        parallelism the vocabulary-sharded one (every rank holds a slice of each row)."""
        s = self.slab
        args = (s.d("temperature", k).view(torch.float32), s.d("top_k", k), s.d("top_p", k).view(torch.float32),
                s.d("min_p", k).view(torch.float32), s.d("seeds", k, torch.int64), mask_bits, mask_row)
        if self.model.sharded_logits:
            return self.par.comm.sample_sharded(lg, *args, out=out)
        return ops.sample(lg, *args, out=out)

    def _logit_mask_rows(self, req, token_slots):
        if not req.logit_masks or not any(m is not None for m in req.logit_masks):
            return None, None
        reqs = sorted({int(req.slot_req[i]) for i in token_slots if req.logit_masks[int(req.slot_req[i])] is not None})
        index = {r: j for j, r in enumerate(reqs)}
        vocab = self.model.vocab_local
        bits = ops.brle_expand([req.logit_masks[r] for r in reqs], vocab, self.device)
        mrow = np.array([index.get(int(req.slot_req[i]), -1) for i in token_slots], dtype=np.int32)
        if self.cuda:
            self.slab.h("mask_row")[:len(mrow)] = mrow
            o, _ = self.slab.offsets["mask_row"]
            self.slab.dev[o:o + len(mrow)].copy_(self.slab.host[o:o + len(mrow)], non_blocking=True)
            return bits, self.slab.d("mask_row", len(mrow))
        return bits, torch.from_numpy(mrow)

    def _sample_cpu(self, lg, k, mask_bits, mask_row):
        from ..ops import reference
        s = self.slab
        masks = None
        if mask_bits is not None:
            vocab = lg.shape[1]
            words = mask_bits.numpy().view(np.uint32)
            unpacked = np.unpackbits(words.view(np.uint8), bitorder="little").reshape(words.shape[0], -1)[:, :vocab].astype(bool)
            masks = [None if int(mask_row[j]) < 0 else torch.from_numpy(unpacked[int(mask_row[j])]) for j in range(k)]
        return reference.sample(lg, s.h("temperature", np.float32)[:k], s.h("top_k")[:k], s.h("top_p", np.float32)[:k],
                                s.h("min_p", np.float32)[:k], s.h("seeds", np.int64)[:k], masks).numpy()

    def _probes(self, req, logits, slot_logit_row, probe_slots, out_slots):
        """Probe slots (distribution, raw logits, log-probabilities of labels, entropy) of one fire, batched per kind:
        one pass of device work and one device-to-host copy per kind, whatever the number of slots."""
        rows = torch.from_numpy(slot_logit_row[probe_slots].astype(np.int64)).to(logits.device)
        lg = logits[rows]
        if self.model.sharded_logits:       # probes read whole rows: gather the few rows they name
            lg = self.par.comm.all_gather_logits(lg)
        lg = lg.contiguous()
        stats = ops.row_stats(lg).float().cpu().numpy()            # max, log-sum-exp, entropy per row
        by_kind: Dict[int, list] = {}
        for j, i in enumerate(probe_slots):
            by_kind.setdefault(int(req.slot_samplers[i].kind), []).append((j, i))
        dev = lg.device
        for kind, members in by_kind.items():
            js = torch.tensor([j for j, _ in members], dtype=torch.long, device=dev)
            sps = [req.slot_samplers[i] for _, i in members]
            if kind == SamplerKind.DIST:
                temp = torch.tensor([sp.temperature if sp.temperature > 0 else 1.0 for sp in sps], dtype=torch.float32, device=dev)
                ks = [min(sp.top_k if sp.top_k > 0 else 32, lg.shape[1]) for sp in sps]
                pv, pi = torch.topk(torch.softmax(lg[js].float() / temp[:, None], -1), max(ks))
                pv, pi = pv.cpu().numpy(), pi.cpu().numpy()
                for n, (_, i) in enumerate(members):
                    out_slots[i] = SlotOutput("distribution", ids=pi[n, :ks[n]].tolist(), probs=pv[n, :ks[n]].tolist())
            elif kind == SamplerKind.RAW_LOGITS:
                raw = lg[js].float().cpu().numpy()
                for n, (_, i) in enumerate(members):
                    out_slots[i] = SlotOutput("logits", logits=raw[n].tobytes())
            elif kind in (SamplerKind.LOGPROB, SamplerKind.LOGPROBS):
                counts = [len(sp.labels) for sp in sps]
                row_of = torch.tensor([j for (j, _), c in zip(members, counts) for _ in range(c)], dtype=torch.long, device=dev)
                labs = torch.tensor([int(x) for sp in sps for x in sp.labels], dtype=torch.long, device=dev)
                vals = lg[row_of, labs].float().cpu().numpy() if labs.numel() else np.zeros(0, np.float32)
                a = 0
                for (j, i), c in zip(members, counts):
                    out_slots[i] = SlotOutput("logprobs", logprobs=(vals[a:a + c] - float(stats[j, 1])).tolist())
                    a += c
            elif kind == SamplerKind.ENTROPY:
                for j, i in members:
                    out_slots[i] = SlotOutput("entropy", entropy=float(stats[j, 2]))
            elif kind == SamplerKind.EMBEDDING:
                for _, i in members:
                    out_slots[i] = SlotOutput("embedding", logits=b"")
            else:
                raise ValueError(f"unsupported sampler kind {kind}")

    # ------------------------------------------------------------------ public entry points
    def fire_batch(self, req: ForwardRequest) -> ForwardResponse:
        with self._order, nvtx.range("pie.fire"):
            return self._fire_batch(req)

    def _fire_batch(self, req: ForwardRequest) -> ForwardResponse:
        self._bind_thread()
        t0 = time.perf_counter()
        self.stats["fires"] += 1
        qlens, kv_lens, slots = self._derive(req)
        if self.bounds_check:
            self._validate_request(req, slots)
        nslots = len(req.slot_samplers)
        self._lora_bindings = self._bind_adapters(req)
        decode = (req.num_requests > 0 and bool((qlens == 1).all()) and self._lora_bindings is None
                  and not (req.has_user_mask is not None and np.any(req.has_user_mask)) and req.media_slot is None)
        if self.par.tp_size > 1 and self.par.comm is not None and self.par.tp_rank == 0:
            # followers must draw the same tokens: fix the per-fire seeds before publishing
            from dataclasses import replace as _replace
            req.slot_samplers = [_replace(sp, seed=int(self.rng.integers(1, 2**62))) if sp.is_token and not sp.seed
                                 else sp for sp in req.slot_samplers]
            self.par.comm.publish_step(req, decode)
        self._token_slots = self._sampler_params(req, None) if nslots else []
        t1 = time.perf_counter()
        if decode and self.cuda:
            with nvtx.range("forward.decode"):
                logits = self._run_decode(req, slots, kv_lens)
            slot_logit_row = np.asarray(req.slot_req, dtype=np.int64) if nslots else np.zeros(0, np.int64)
        else:
            with nvtx.range("forward.general"):
                logits = self._run_general(req, qlens, slots, kv_lens)
            slot_logit_row = np.asarray(self._slot_logit_row, dtype=np.int64)
        t2 = time.perf_counter()
        with nvtx.range("respond"):
            resp = self._respond(req, logits, slot_logit_row)
        if self.cuda and nslots == 0:
            torch.cuda.current_stream().synchronize()
        t3 = time.perf_counter()
        resp.t_build_us = (t1 - t0) * 1e6
        resp.t_forward_us = (t2 - t1) * 1e6
        resp.t_sample_us = (t3 - t2) * 1e6
        resp.t_total_us = (t3 - t0) * 1e6
        return resp

    # ------------------------------------------------------------------ pipelined decode
    def decode_async(self, step: "CohortStep", parity: int) -> "AsyncTokens":
        """Launch one pure-decode step for the rows of `step` and return at once.

        Rows whose `src_row` is >= 0 take their input token from the tokens sampled by the
        previous pipelined step (device to device), so the host never has to wait for one step's
        result before launching the next; it reads each step's tokens one step late.
        """
        with self._order:
            return self._decode_async(step, parity)

    def _decode_async(self, step: "CohortStep", parity: int) -> "AsyncTokens":
        self._bind_thread()
        r = step.r
        ps = self.page_size
        if not self.cuda:
            return self._decode_sync_cpu(step)
        s = self.slab
        s.select(parity)
        rb = self._bucket(r) if self.use_graphs else r
        if r > self.max_requests or len(step.page_indices) > self.max_page_refs:
            raise ValueError("decode step exceeds the advertised forward limits")
        idx = step.kv_lens.astype(np.int64) - 1
        pg = step.page_indices[step.page_indptr[:-1].astype(np.int64) + idx // ps].astype(np.int64)
        s.h("tokens")[:r] = step.host_tokens
        s.h("positions")[:r] = step.positions
        s.h("slots")[:r] = pg * ps + idx % ps
        s.h("src_row")[:r] = step.src_row
        s.h("qo_indptr")[:rb + 1] = np.arange(rb + 1, dtype=np.int32)
        s.h("kv_page_indptr")[:r + 1] = step.page_indptr
        s.h("kv_lens")[:r] = step.kv_lens
        npg = len(step.page_indices)
        s.h("page_indices")[:npg] = step.page_indices
        if rb > r:
            s.h("tokens")[r:rb] = 0
            s.h("positions")[r:rb] = 0
            s.h("slots")[r:rb] = -1
            s.h("src_row")[r:rb] = -1
            s.h("kv_page_indptr")[r + 1:rb + 1] = step.page_indptr[-1]
        cascade = self._plan_decode(step.kv_lens, step.page_indptr, step.page_indices, r, rb)
        s.h("temperature", np.float32)[:r] = step.temperature
        s.h("top_k")[:r] = step.top_k
        s.h("top_p", np.float32)[:r] = step.top_p
        s.h("min_p", np.float32)[:r] = step.min_p
        s.h("seeds", np.int64)[:r] = step.seeds
        if self.par.tp_size > 1 and self.par.comm is not None:
            self.par.comm.publish_decode(s, r, rb, npg, parity, cascade)
        if self.use_graphs and self._gkey(rb, cascade) not in self.graphs:
            s.upload("tile_qstart", ("page_indices", npg))
            self.graphs[self._gkey(rb, cascade)] = self._capture(rb, cascade)
        self._launch_decode(r, rb, npg, parity, cascade)
        ev = torch.cuda.Event()
        ev.record()
        self.stats["fires"] += 1
        return AsyncTokens(ev, self.cohort_host[parity & 1], r, driver=self)

    def _launch_decode(self, r: int, rb: int, npg: int, parity: int, cascade: bool = False) -> None:
        """Device side of a pipelined decode step (also what tensor-parallel followers run)."""
        with nvtx.range("pie.decode.launch"):
            self._launch_decode_impl(r, rb, npg, parity, cascade)

    def _launch_decode_impl(self, r: int, rb: int, npg: int, parity: int, cascade: bool) -> None:
        s = self.slab
        s.upload("tile_qstart", ("page_indices", npg))
        cur, prev = self.cohort_sampled[parity & 1], self.cohort_sampled[(parity & 1) ^ 1]
        ops.feed_tokens(s.d("tokens"), s.d("src_row"), prev, r)
        if self.use_graphs:
            g = self.graphs[self._gkey(rb, cascade)]
            g.graph.replay()
            logits = g.logits
            self.stats["graph_replays"] += 1
        else:
            logits = self.model.forward(self._forward_inputs_decode(rb, cascade), self.kv.data)
            self.stats["eager"] += 1
        self._sample(logits[:r], r, None, None, cur)
        self.cohort_host[parity & 1][:r].copy_(cur[:r], non_blocking=True)
        self.status_host.copy_(ops.kernel_status(self.device), non_blocking=True)

    def _decode_sync_cpu(self, step: "CohortStep") -> "AsyncTokens":
        """CPU drivers have no stream to pipeline on: resolve the token feed on the host and run
        the step through the ordinary batch path."""
        r = step.r
        toks = np.array(step.host_tokens, dtype=np.int32)
        prev = getattr(self, "_cpu_prev_tokens", None)
        sel = step.src_row >= 0
        if sel.any():
            toks[sel] = prev[step.src_row[sel]]
        last = (step.kv_lens - 1) % self.page_size + 1
        samplers = [SamplerSpec(SamplerKind.TOP_K_TOP_P, float(step.temperature[i]), int(step.top_k[i]),
                                float(step.top_p[i]), 0.0, int(step.seeds[i]), seed_final=True) if step.min_p[i] == 0 else
                    SamplerSpec(SamplerKind.MIN_P, float(step.temperature[i]), 0, 1.0, float(step.min_p[i]),
                                int(step.seeds[i]), seed_final=True) for i in range(r)]
        req = ForwardRequest(tokens=toks, positions=step.positions, qo_indptr=np.arange(r + 1, dtype=np.int32),
                             kv_page_indices=step.page_indices, kv_page_indptr=step.page_indptr,
                             kv_last_page_lens=last.astype(np.int32), slot_req=np.arange(r, dtype=np.int32),
                             slot_row=np.arange(r, dtype=np.int32), slot_samplers=samplers, single_token_mode=True)
        resp = self.fire_batch(req)
        self._cpu_prev_tokens = np.asarray(resp.tokens, dtype=np.int32)
        return AsyncTokens(None, None, r, ready=self._cpu_prev_tokens)

    # ------------------------------------------------------------------ device-resident decode loop
    def stage_decode(self, req: ForwardRequest) -> dict:
        """Prepare one pure-decode step without running it: returns device copies of the slab
        contents so that `replay_staged` can run the step with no host work in between.
        Used to time the device path alone (tokens are fed from the previous step's samples)."""
        self._bind_thread()
        qlens, kv_lens, slots = self._derive(req)
        assert self.cuda and bool((qlens == 1).all())
        s = self.slab
        r = req.num_requests
        rb = self._bucket(r)
        self._token_slots = self._sampler_params(req, None)
        self._fill_common(req, slots, kv_lens, n_pad_tokens=rb - r, r_pad=rb - r)
        if rb > r:
            s.h("tokens")[r:rb] = 0
            s.h("positions")[r:rb] = 0
            s.h("slots")[r:rb] = -1
            s.h("kv_page_indptr")[r + 1:rb + 1] = req.kv_page_indptr[-1]
        cascade = self._plan_decode(kv_lens, np.asarray(req.kv_page_indptr), np.asarray(req.kv_page_indices), r, rb)
        o, n = s.offsets["tile_qstart"]
        end = o + n
        po, _ = s.offsets["page_indices"]
        npg = len(req.kv_page_indices)
        key = self._gkey(rb, cascade)
        if key not in self.graphs:
            s.upload("tile_qstart", ("page_indices", npg))
            self.graphs[key] = self._capture(rb, cascade)
        return {"fixed": s.host[:end].to(self.device), "pages": s.host[po:po + npg].to(self.device),
                "rb": rb, "r": r, "end": end, "po": po, "npg": npg, "key": key}

    def replay_staged(self, st: dict, feed_sampled: bool) -> None:
        self._bind_thread()
        s = self.slab
        s.dev[:st["end"]].copy_(st["fixed"], non_blocking=True)
        s.dev[st["po"]:st["po"] + st["npg"]].copy_(st["pages"], non_blocking=True)
        r = st["r"]
        if feed_sampled:
            s.d("tokens", r).copy_(self.sampled[:r], non_blocking=True)
        g = self.graphs[st.get("key", st["rb"])]
        g.graph.replay()
        self._sample(g.logits[:r], r, None, None, self.sampled)

    def launches_per_decode_step(self, rb: int) -> int:
        """Kernels of this library launched by one decode step of bucket `rb`: the captured
        forward (counted at capture time) plus the sampler."""
        return self.graphs[rb].launches + 1

    def copy(self, req: CopyRequest) -> None:
        with self._order, nvtx.range("pie.copy"):
            self._bind_thread()
            if self.par.tp_size > 1 and self.par.comm is not None:
                self.par.comm.publish_copy(req)     # every rank holds a shard of each page
            self.kv.copy(req)

    def check_status_host(self) -> None:
        """Raise if a kernel gave up on a bounded wait (reads the pinned copy of the status word
        that the last fire brought back; call only after that fire's stream work is complete)."""
        if self.cuda and int(self.status_host[0]) != 0:
            code = int(self.status_host[0])
            self._failed = f"a kernel gave up on a bounded wait (status {code})"
            self.status_host[0] = 0
            ops.kernel_status(self.device).zero_()
            from ..ops._lib import KernelLibraryError
            raise KernelLibraryError(self._failed)

    def health(self) -> bool:
        """Called from the watchdog thread: host state only (a CUDA call here could invalidate a
        graph capture running on the scheduler thread)."""
        return self._failed is None

    def shutdown(self) -> None:
        self.graphs.clear()
