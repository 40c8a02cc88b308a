"""Tensor-parallel communication for one model replica: one process per GPU.

Data plane (device): peer-mapped symmetric buffers (torch symmetric memory over NVLink /
NVSwitch) that the fused kernels read and write directly:
  * `gemm_rs`            o_proj / down GEMM whose epilogue stores each output row into the
                         receive buffer of the rank that owns the row (reduce-scatter by peer stores)
  * `reduce_norm_push`   owner sums the partial rows + residual, RMSNorm, pushes the normalised
                         rows into every rank's gathered-activation buffer (all-gather by peer stores)
  * `gemm_gated`         QKV / gate-up / lm_head GEMM whose TMA producer waits for the push flags
The residual stream is row-sharded between blocks, so a transformer block costs one
reduce-scatter + one all-gather per GEMM pair instead of the reference's two all-reduces
(driver/cuda/src/model/llama_like.cpp:633-647, 706-742). NCCL remains for bootstrap, the
logits all-gather and as the baseline path (`all_reduce`, `gemm_allreduce`).

Control plane (host): rank 0 runs the engine; it publishes every fire (a batch request as a flat wire frame, `driver/abi.py`,
or the raw input slab of a pipelined decode step) into a POSIX shared-memory ring that the
follower ranks poll - one host memcpy per fire instead of the reference's eight NCCL broadcasts
(driver/cuda/src/executor/executor.cpp:1305-1360), and page copies reach every rank (the
reference only executes them on rank 0).
"""
from __future__ import annotations

import ctypes as C
import os
import time
from dataclasses import replace
from multiprocessing import shared_memory
from typing import Optional

import numpy as np
import torch

from .. import ops
from ..ops import _lib
from ..ops._lib import check, ptr, stream_ptr
from ..driver import abi

KIND_BATCH, KIND_DECODE, KIND_COPY, KIND_STOP, KIND_MARK = 1, 2, 3, 4, 5
_HDR_WORDS = 64


def _round32(x: int) -> int:
    return -(-x // 32) * 32


def _pid_alive(pid: int) -> bool:
    if pid <= 0:
        return True          # not registered yet
    try:
        os.kill(pid, 0)
    except ProcessLookupError:
        return False
    except PermissionError:
        return True
    try:        # a process that exited but was not reaped yet still answers signals
        with open(f"/proc/{pid}/stat") as f:
            return f.read().rsplit(")", 1)[1].split()[0] != "Z"
    except (OSError, IndexError):
        return True


class StepRing:
    """Single-writer (rank 0), multi-reader shared-memory mailbox with two payload slots.

    Memory ordering: the writer stores the payload, then the header words, then the sequence word,
    all as plain stores through numpy; readers poll the sequence word and then read the rest. That
    is only ordered on hosts with total store order (x86-64, which is what B200 HGX boxes are); an
    Arm host (Grace) would need a release store / acquire load of the sequence word.

    Liveness: every rank registers its pid in the header. A writer that waits for a follower's
    acknowledgement, and a reader that waits for the next step, back off to short sleeps, check that
    the other side's process still exists, and give up after `ack_timeout_s` / the receive timeout.
    """

    def __init__(self, name: str, world: int, rank: int, cap: int = 48 << 20, create: bool = False,
                 ack_timeout_s: Optional[float] = None):
        self.world, self.rank, self.cap = world, rank, cap
        if ack_timeout_s is None:
            ack_timeout_s = float(os.environ.get("PIE_TP_ACK_TIMEOUT_S", "120"))
        self.ack_timeout_s = ack_timeout_s
        size = _HDR_WORDS * 8 * 2 + 2 * cap
        self.shm = shared_memory.SharedMemory(name=name, create=create, size=size)
        self.hdr = np.ndarray((2, _HDR_WORDS), dtype=np.int64, buffer=self.shm.buf)
        if create:
            self.hdr[:] = 0
        self.payload = [np.ndarray((cap,), dtype=np.uint8, buffer=self.shm.buf, offset=_HDR_WORDS * 16 + i * cap)
                        for i in range(2)]
        self.seq = 0
        self.hdr[0, 48 + rank] = os.getpid()

    # header words: 0 seq, 1 kind, 2 nbytes, 3..10 meta; slot-0 header also holds 32+r acks and 48+r pids
    def publish(self, kind: int, data: Optional[np.ndarray], meta=()) -> None:
        self.seq += 1
        slot = self.seq & 1
        h = self.hdr[slot]
        # the slot was last used by seq-2: every follower must have consumed it
        deadline = time.time() + self.ack_timeout_s
        for r in range(1, self.world):
            spins = 0
            while self.hdr[0, 32 + r] < self.seq - 2:
                spins += 1
                if spins > 2000:
                    time.sleep(0.0001)
                    if spins % 256 == 0:
                        if not _pid_alive(int(self.hdr[0, 48 + r])):
                            raise RuntimeError(f"tensor-parallel follower {r} exited")
                        if time.time() > deadline:
                            raise RuntimeError(f"tensor-parallel follower {r} stopped consuming steps")
        n = 0 if data is None else data.nbytes
        if n > self.cap:
            raise ValueError("step payload exceeds the control ring capacity")
        if n:
            self.payload[slot][:n] = data.view(np.uint8).reshape(-1)
        h[1], h[2] = kind, n
        for i, m in enumerate(meta):
            h[3 + i] = m
        h[0] = self.seq   # written last: readers poll this word

    def receive(self, timeout: float = 3600.0):
        want = self.seq + 1
        slot = want & 1
        h = self.hdr[slot]
        deadline = time.time() + timeout
        spins = 0
        while h[0] != want:
            spins += 1
            if spins > 2000:
                time.sleep(0.00005)
                if spins % 512 == 0:
                    if not _pid_alive(int(self.hdr[0, 48])):
                        raise TimeoutError("rank 0 exited")
                    if time.time() > deadline:
                        raise TimeoutError("no step from rank 0")
        self.seq = want
        n = int(h[2])
        return int(h[1]), self.payload[slot][:n], [int(x) for x in h[3:11]]

    def ack(self) -> None:
        self.hdr[0, 32 + self.rank] = self.seq

    def close(self, unlink: bool = False) -> None:
        try:
            self.hdr = None
            self.payload = None
            self.shm.close()
            if unlink:
                self.shm.unlink()
        except Exception:  # noqa: BLE001
            pass


class TPComm:
    def __init__(self, rank: int, world: int, device, fused: bool = True):
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.fused = fused
        self.driver = None
        self.ring: Optional[StepRing] = None
        self._stopped = False

    # ------------------------------------------------------------------ setup
    def attach(self, driver) -> None:
        """Allocate the symmetric buffers for `driver`'s model and open the control ring."""
        import torch.distributed as dist
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer loads/stores only
        import torch.distributed._symmetric_memory as symm_mem

        self.driver = driver
        cfg = driver.cfg
        self.hidden = cfg.hidden_size
        self.rpr_max = _round32(-(-driver.max_tokens // self.world))
        rows = self.rpr_max * self.world
        nb_act = rows * self.hidden * 2
        self.off_recv, self.off_xfull, self.off_flags = 0, nb_act, 2 * nb_act
        self.ar_cap = 512 * 1024                       # bf16 elements per one-shot all-reduce slot (1 MiB)
        self.off_ar = 2 * nb_act + 4096
        # mailboxes + flags of the vocabulary-sharded sampler (one mailbox per resident CTA)
        self.ts_grid = max(1, min(1024, _lib.declare("pie_tp_sample_max_grid", [C.c_int], C.c_int)(
            ops.num_sms(self.device))))
        self.off_ts_box = self.off_ar + 2 * self.world * self.ar_cap * 2
        ts_box = _lib.declare("pie_tp_sample_mailbox_bytes", [C.c_int, C.c_int], C.c_long)(self.ts_grid, self.world)
        total = self.off_ts_box + ts_box
        self.sym = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        self.sym.zero_()
        torch.cuda.synchronize(self.device)
        self.hdl = symm_mem.rendezvous(self.sym, dist.group.WORLD)
        base = [int(p) for p in self.hdl.buffer_ptrs]
        self.local_base = base[self.rank]
        assert self.local_base == self.sym.data_ptr()
        self.xfull = self.sym[self.off_xfull:self.off_xfull + nb_act].view(torch.bfloat16).view(rows, self.hidden)
        self.recv = self.sym[self.off_recv:self.off_recv + nb_act].view(torch.bfloat16)
        # counters private to this rank: rs_done, rs_epoch, ag_done, ag_epoch
        self.local_ctr = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.residual = torch.zeros(self.rpr_max, self.hidden, dtype=torch.bfloat16, device=self.device)
        status = ops.kernel_status(self.device)
        W = self.world
        arr_p = (C.c_void_p * W)
        rs_flags = [b + self.off_flags for b in base]           # int32[8] per rank
        ag_flags = [b + self.off_flags + 256 for b in base]     # int32[8] per rank
        lc = self.local_ctr.data_ptr()
        self.tp_blob = C.create_string_buffer(_lib.declare("pie_tp_args_size", [], C.c_int)())
        fill = _lib.declare("pie_tp_fill_args", [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                 C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int])
        check(fill(self.tp_blob, ag_flags[self.rank], lc + 12, arr_p(*[b + self.off_recv for b in base]),
                   arr_p(*rs_flags), lc + 0, lc + 4, W, self.rank, 32, 0), "tp_fill_args")
        self.norm_blob = C.create_string_buffer(_lib.declare("pie_tp_norm_args_size", [], C.c_int)())
        filln = _lib.declare("pie_tp_fill_norm_args", [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                       C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int])
        check(filln(self.norm_blob, self.local_base + self.off_recv, rs_flags[self.rank], lc + 4,
                    arr_p(*[b + self.off_xfull for b in base]), arr_p(*ag_flags), lc + 8, lc + 12,
                    status.data_ptr(), W, self.rank), "tp_fill_norm_args")
        # one-shot small all-reduce: slots [2][world][cap] on every rank, flags at +512, counters private
        self.ar_ctr = torch.zeros(2, dtype=torch.int32, device=self.device)
        ar_flags = [b + self.off_flags + 512 for b in base]
        self.ar_blob = C.create_string_buffer(_lib.declare("pie_tp_ar_args_size", [], C.c_int)())
        fill_ar = _lib.declare("pie_tp_fill_ar_args", [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                       C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_long])
        check(fill_ar(self.ar_blob, arr_p(*[b + self.off_ar for b in base]), arr_p(*ar_flags), ar_flags[self.rank],
                      self.ar_ctr.data_ptr(), self.ar_ctr.data_ptr() + 4, status.data_ptr(), W, self.rank,
                      self.ar_cap), "tp_fill_ar_args")
        self._ar_small = _lib.declare("pie_tp_allreduce_small", [C.c_void_p, C.c_void_p, C.c_void_p, C.c_long, C.c_int,
                                                                 C.c_void_p])
        # vocabulary-sharded sampler
        self.vocab_local = driver.model.w["lm_head"].shape[0]
        self.ts_seq = torch.zeros(self.ts_grid, dtype=torch.int32, device=self.device)
        self.ts_blob = C.create_string_buffer(_lib.declare("pie_tp_sample_args_size", [], C.c_int)())
        fill_ts = _lib.declare("pie_tp_sample_fill_args", [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                           C.c_int, C.c_int, C.c_int, C.c_int, C.c_longlong])
        check(fill_ts(self.ts_blob, arr_p(*[b + self.off_ts_box for b in base]),
                      self.ts_seq.data_ptr(), status.data_ptr(), W,
                      self.rank, self.vocab_local, self.ts_grid, 0), "tp_sample_fill_args")
        self._ag_flags_local = ag_flags[self.rank]
        self._ag_epoch_ptr = lc + 12
        self._gemm_tp = _lib.declare("pie_gemm_bf16_tp", [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                                          C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                                          C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p])
        self._gemm_fp8_tp = _lib.declare("pie_gemm_fp8_blockscaled_tp",
                                         [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                          C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p])
        self._norm_push = _lib.declare("pie_tp_reduce_norm_push", [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                                                  C.c_int, C.c_int, C.c_float, C.c_void_p])
        self._wait_ag = _lib.declare("pie_tp_wait_ag", [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p])
        self._status = status
        self._sms = ops.num_sms(self.device)
        ops.ensure_gemm_workspace(self.device)
        # control ring
        name = [f"pie_b200_ring_{os.getpid()}_{int(time.time() * 1e3) & 0xFFFFFF}"] if self.rank == 0 else [None]
        if self.rank == 0:
            self.ring = StepRing(name[0], self.world, 0, create=True)
        dist.broadcast_object_list(name, src=0)
        if self.rank != 0:
            self.ring = StepRing(name[0], self.world, self.rank, create=False)
        dist.barrier()

    # ------------------------------------------------------------------ fused data plane
    def rows_per_rank(self, n: int) -> int:
        return _round32(-(-n // self.world))

    def _valid_rows(self, n: int, rpr: int) -> int:
        return max(0, min(rpr, n - self.rank * rpr))

    def embed_norm_push(self, tokens: torch.Tensor, embed: torch.Tensor, weight, eps: float, n: int) -> None:
        """Residual rows of this rank = embeddings of its tokens; push norm(residual) to all ranks."""
        rpr = self.rows_per_rank(n)
        valid = self._valid_rows(n, rpr)
        if valid:
            ops.embed(tokens[self.rank * rpr:self.rank * rpr + valid], embed, out=self.residual[:valid])
        check(self._norm_push(self.norm_blob, ptr(self.residual), ptr(weight), rpr, self.hidden, valid, 0, eps,
                              stream_ptr()), "tp_norm_push")

    def reduce_norm_push(self, weight, eps: float, n: int) -> None:
        rpr = self.rows_per_rank(n)
        check(self._norm_push(self.norm_blob, ptr(self.residual), ptr(weight), rpr, self.hidden,
                              self._valid_rows(n, rpr), 1, eps, stream_ptr()), "tp_reduce_norm_push")

    def _fp8(self, a: torch.Tensor, q, n: int, epilogue: int, out, rpr: int = 32):
        """Block-scaled fp8 weight: quantise the (already gathered) activation rows 1x128 and run the
        fp8 tcgen05 GEMM, with the reduce-scatter epilogue when `epilogue` is EPI_RS."""
        x8, sx = ops.quant_act_fp8(a)
        nn, k = q.shape
        check(self._gemm_fp8_tp(ptr(x8), ptr(sx), ptr(q.w8), ptr(q.scale), ptr(out), n, nn, k,
                                out.stride(0) if out is not None else 0, epilogue, self.tp_blob, rpr,
                                ptr(self._status), self._sms, stream_ptr()), "gemm_fp8_tp")
        return out

    def gemm_gated(self, w, n: int, swiglu: bool = False, x: Optional[torch.Tensor] = None):
        """y = gathered_activation[:n] @ w.T. The kernel's loads of a row tile wait for the push of the
        ranks that own those rows (for an explicit `x`, which is not laid out by owner, for every rank)."""
        if isinstance(w, ops.Fp8Linear):
            a = self.wait_gathered(n) if x is None else x
            nn = w.shape[0]
            out = torch.empty(n, nn // 2 if swiglu else nn, dtype=torch.bfloat16, device=self.device)
            return self._fp8(a, w, n, ops.EPI_SWIGLU if swiglu else ops.EPI_STORE, out)
        a = self.xfull[:n] if x is None else x
        nn = w.shape[0]
        out = torch.empty(n, nn // 2 if swiglu else nn, dtype=torch.bfloat16, device=self.device)
        check(self._gemm_tp(ptr(a), ptr(w), ptr(out), n, nn, a.shape[1], a.stride(0), w.stride(0), out.stride(0),
                            ops.EPI_SWIGLU if swiglu else ops.EPI_STORE, self.tp_blob,
                            self.rows_per_rank(n) if x is None else 0, 1, 0,
                            ptr(self._status), self._sms, stream_ptr()), "gemm_gated")
        return out

    def gemm_rs(self, a: torch.Tensor, w, n: int) -> None:
        """Partial y = a @ w.T scattered row-wise into the owners' receive buffers."""
        rpr = self.rows_per_rank(n)
        if isinstance(w, ops.Fp8Linear):
            self._fp8(a, w, n, 3, None, rpr)
            return
        check(self._gemm_tp(ptr(a), ptr(w), None, n, w.shape[0], a.shape[1], a.stride(0), w.stride(0), 0, 3,
                            self.tp_blob, rpr, 0, 0, ptr(self._status), self._sms, stream_ptr()), "gemm_rs")

    def wait_gathered(self, n: int) -> torch.Tensor:
        check(self._wait_ag(self._ag_flags_local, self._ag_epoch_ptr, self.world, ptr(self._status), stream_ptr()),
              "tp_wait_ag")
        return self.xfull[:n]

    def sample_sharded(self, local_logits: torch.Tensor, temperature, top_k, top_p, min_p, seeds, mask_bits,
                       mask_row, out: torch.Tensor) -> torch.Tensor:
        """One token per row from logits that are sharded over the ranks' vocabulary slices
        (`local_logits` is this rank's [rows, V / world] slice). Every rank calls it in step with
        the same parameters and receives the same tokens; a few words per row cross NVLink."""
        rows, v = local_logits.shape
        assert v == self.vocab_local and local_logits.stride(1) == 1
        mask_words = mask_bits.shape[1] if mask_bits is not None else 0
        check(_lib.fn("pie_tp_sample")(self.ts_blob, ptr(local_logits), local_logits.stride(0), rows, ptr(temperature),
                                       ptr(top_k), ptr(top_p), ptr(min_p), ptr(seeds), ptr(mask_bits), ptr(mask_row),
                                       mask_words, ptr(out), self._sms, stream_ptr()), "tp_sample")
        return out

    # ------------------------------------------------------------------ NCCL paths
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Sum over ranks, in place. Small bf16 tensors go through the one-shot peer-memory kernel
        (when the fused data plane is attached), everything else through NCCL."""
        n = x.numel()
        if (self.fused and getattr(self, "_ar_small", None) is not None and x.dtype == torch.bfloat16
                and x.is_contiguous() and n % 8 == 0 and n <= self.ar_cap):
            check(self._ar_small(self.ar_blob, ptr(x), ptr(x), n, self._sms, stream_ptr()), "tp_allreduce_small")
            return x
        import torch.distributed as dist
        dist.all_reduce(x)
        return x

    def gemm_allreduce(self, a, w, model):
        """Baseline row-parallel linear: library-style GEMM then NCCL all-reduce."""
        y = model._gemm(a, w)
        return self.all_reduce(y)

    def all_gather_logits(self, local: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        rows, v = local.shape
        out = torch.empty(self.world, rows, v, dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous())
        return out.permute(1, 0, 2).reshape(rows, self.world * v)

    # ------------------------------------------------------------------ control plane
    def publish_step(self, req, decode: bool) -> None:
        if self.rank != 0 or self.ring is None:
            return
        data = np.frombuffer(abi.pack_forward_request(req), dtype=np.uint8)
        self.ring.publish(KIND_BATCH, data)

    def publish_decode(self, slab, r: int, rb: int, npg: int, parity: int, cascade: bool = False) -> None:
        if self.rank != 0 or self.ring is None:
            return
        o, n = slab.offsets["tile_qstart"]
        end = o + n
        po, _ = slab.offsets["page_indices"]
        buf = np.concatenate([slab.np[:end], slab.np[po:po + npg]])
        self.ring.publish(KIND_DECODE, buf, (r, rb, npg, parity, end, int(cascade)))

    def publish_copy(self, req) -> None:
        if self.rank != 0 or self.ring is None:
            return
        self.ring.publish(KIND_COPY, np.frombuffer(abi.pack_copy_request(req), dtype=np.uint8))

    def mark(self, end: bool) -> float:
        """Timed-region bracket on every rank: device synchronise + barrier, a CUDA event on each
        rank's stream, and at the end mark the MAX over ranks of the event-to-event time (ms)."""
        import torch.distributed as dist
        if self.rank == 0 and self.ring is not None:
            self.ring.publish(KIND_MARK, None, (1 if end else 0,))
        return self._mark_local(end)

    def _mark_local(self, end: bool) -> float:
        import torch.distributed as dist
        if not end:
            torch.cuda.synchronize(self.device)
            dist.barrier()
            self._ev0 = torch.cuda.Event(enable_timing=True)
            self._ev0.record()
            return 0.0
        ev1 = torch.cuda.Event(enable_timing=True)
        ev1.record()
        torch.cuda.synchronize(self.device)
        ms = torch.tensor([self._ev0.elapsed_time(ev1)], dtype=torch.float32, device=self.device)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.barrier()
        return float(ms.item())

    def stop_followers(self) -> None:
        if self.rank == 0 and self.ring is not None and not self._stopped:
            self._stopped = True
            self.ring.publish(KIND_STOP, None)

    def follower_loop(self, driver) -> None:
        """Ranks > 0: execute every fire rank 0 publishes, in lock step, until STOP."""
        ring = self.ring
        while True:
            kind, payload, meta = ring.receive()
            if kind == KIND_STOP:
                ring.ack()
                break
            if kind == KIND_BATCH:
                req = abi.unpack_forward_request(payload.tobytes())
                ring.ack()
                driver.fire_batch(req)
            elif kind == KIND_DECODE:
                r, rb, npg, parity, end = meta[:5]
                cascade = bool(meta[5])
                s = driver.slab
                s.select(parity)
                words = payload.view(np.int32)
                s.np[:end] = words[:end]
                po, _ = s.offsets["page_indices"]
                s.np[po:po + npg] = words[end:end + npg]
                ring.ack()
                key = driver._gkey(rb, cascade)
                if driver.use_graphs and key not in driver.graphs:
                    s.upload("tile_qstart", ("page_indices", npg))
                    driver.graphs[key] = driver._capture(rb, cascade)
                driver._launch_decode(r, rb, npg, parity, cascade)
            elif kind == KIND_COPY:
                req = abi.unpack_copy_request(payload.tobytes())
                ring.ack()
                driver.kv.copy(req)
            elif kind == KIND_MARK:
                ring.ack()
                self._mark_local(bool(meta[0]))
        torch.cuda.synchronize(self.device)

    def close(self) -> None:
        if self.ring is not None:
            self.ring.close(unlink=self.rank == 0)
            self.ring = None
