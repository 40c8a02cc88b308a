"""Vocabulary-sharded sampler (`pie_tp_sample`): all ranks of a tensor-parallel group run as ONE
cooperative launch on one GPU (blockIdx.y = rank, every rank's mailbox in local memory), and every
rank's tokens must equal the single-GPU sampler's on the concatenated logits."""
import ctypes as C

import numpy as np
import pytest
import torch

from pie_b200 import ops
from pie_b200.ops import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class Emu:
    """Buffers of an emulated group: per-rank mailbox, flags, counters and outputs."""

    def __init__(self, world: int, vocab_local: int, grid_max: int, rows_max: int):
        self.world, self.vocab_local, self.grid_max = world, vocab_local, grid_max
        lib = _lib.load(required=True)
        box = _lib.declare("pie_tp_sample_mailbox_bytes", [C.c_int, C.c_int], C.c_long)(grid_max, world)
        self.xbuf = [torch.zeros(box, dtype=torch.uint8, device=DEV) for _ in range(world)]
        self.seq = [torch.zeros(grid_max, dtype=torch.int32, device=DEV) for _ in range(world)]
        self.out = [torch.full((rows_max,), -1, dtype=torch.int32, device=DEV) for _ in range(world)]
        self.status = ops.kernel_status(DEV)
        self.fn = lib.pie_tp_sample_emulated
        self.fn.restype = C.c_int
        self.fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_longlong,
                            C.c_void_p, C.c_long, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                            C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]

    def sample(self, logits, temperature, top_k, top_p, min_p, seeds, mask_bits=None, mask_row=None,
               wait_cycles: int = 0):
        rows = logits.shape[0]
        w, vl = self.world, self.vocab_local
        shards = [logits[:, r * vl:(r + 1) * vl].contiguous() for r in range(w)]
        arr = lambda ts: (C.c_void_p * w)(*[t.data_ptr() for t in ts])
        rc = self.fn(arr(self.xbuf), arr(self.seq), self.status.data_ptr(), w, vl, self.grid_max,
                     wait_cycles, arr(shards), vl, rows, temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(),
                     min_p.data_ptr(), seeds.data_ptr(), 0 if mask_bits is None else mask_bits.data_ptr(),
                     0 if mask_row is None else mask_row.data_ptr(), 0 if mask_bits is None else mask_bits.shape[1],
                     arr(self.out), ops.num_sms(DEV), torch.cuda.current_stream().cuda_stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        return [o[:rows].clone() for o in self.out]


def params(rows, kind, seed):
    g = torch.Generator().manual_seed(seed)
    t = torch.ones(rows)
    k = torch.zeros(rows, dtype=torch.int32)
    p = torch.ones(rows)
    mp = torch.zeros(rows)
    if kind == "greedy":
        t[:] = 0
    elif kind == "temperature":
        t = 0.5 + torch.rand(rows, generator=g)
    elif kind == "top_p":
        p[:] = 0.9
    elif kind == "top_p_small":
        p[:] = 0.3
    elif kind == "top_k":
        k[:] = 50
    elif kind == "top_k_top_p":
        k[:] = 40
        p[:] = 0.8
    elif kind == "min_p":
        mp[:] = 0.05
    elif kind == "mixed":
        t = torch.where(torch.arange(rows) % 5 == 0, torch.zeros(rows), 0.7 + torch.rand(rows, generator=g))
        k = torch.where(torch.arange(rows) % 3 == 0, torch.full((rows,), 20), torch.zeros(rows, dtype=torch.long)).int()
        p = torch.where(torch.arange(rows) % 2 == 0, torch.full((rows,), 0.9), torch.ones(rows))
    seeds = torch.randint(1, 2**62, (rows,), generator=g, dtype=torch.int64)
    return [x.to(DEV) for x in (t.float(), k, p.float(), mp.float(), seeds)]


def make_logits(rows, vocab, seed, peaked):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, vocab, generator=g) * (4.0 if peaked else 0.3)
    return x.to(torch.bfloat16).to(DEV)


@pytest.mark.parametrize("world,vocab_local", [(2, 4096), (4, 2008), (8, 16032)])
@pytest.mark.parametrize("kind", ["greedy", "temperature", "top_p", "top_p_small", "top_k", "top_k_top_p", "min_p",
                                  "mixed"])
def test_sharded_sampler_equals_single_gpu_sampler(world, vocab_local, kind):
    rows = 37
    emu = Emu(world, vocab_local, grid_max=16, rows_max=64)      # 16 CTAs per rank: several rows per CTA
    vocab = world * vocab_local
    for call, peaked in enumerate((False, True)):               # two calls: counters and parity carry over
        lg = make_logits(rows, vocab, 7 + call, peaked)
        pr = params(rows, kind, 100 + call)
        want = ops.sample(lg, *pr)
        got = emu.sample(lg, *pr)
        torch.cuda.synchronize()
        assert int(emu.status[0].item()) == 0
        for r in range(world):
            assert torch.equal(got[r], got[0])
        same = (got[0] == want).float().mean().item()
        assert same == 1.0, (kind, call, same, got[0][:8].tolist(), want[:8].tolist())
        assert int(want.min()) >= 0 and int(want.max()) < vocab


def test_sharded_sampler_honours_vocabulary_masks():
    world, vl, rows = 4, 2048, 19
    vocab = world * vl
    emu = Emu(world, vl, grid_max=8, rows_max=32)
    lg = make_logits(rows, vocab, 3, True)
    g = torch.Generator().manual_seed(5)
    allowed = torch.rand(3, vocab, generator=g) < 0.02
    allowed[2] = False
    allowed[2, vocab - 7] = True                        # a single allowed token in the last shard
    bits = np.packbits(allowed.numpy().astype(np.uint8), axis=1, bitorder="little").view(np.uint32)
    mask_bits = torch.from_numpy(bits.view(np.int32).copy()).to(DEV)
    mask_row = torch.tensor([i % 4 - 1 for i in range(rows)], dtype=torch.int32, device=DEV)   # -1: no mask
    for kind in ("greedy", "top_p", "top_k"):
        pr = params(rows, kind, 11)
        want = ops.sample(lg, *pr, mask_bits=mask_bits, mask_row=mask_row)
        got = emu.sample(lg, *pr, mask_bits=mask_bits, mask_row=mask_row)
        assert torch.equal(got[0], want) and torch.equal(got[-1], want)
        mr = mask_row.cpu().numpy()
        tok = want.cpu().numpy()
        for i in range(rows):
            if mr[i] >= 0:
                assert allowed[mr[i], tok[i]]
        assert all(tok[i] == vocab - 7 for i in range(rows) if mr[i] == 2)


def test_sharded_sampler_distribution():
    """Temperature sampling draws from softmax(logits): chi-square-free sanity check on a tiny vocabulary."""
    world, vl = 2, 8
    vocab = world * vl
    rows = 4096
    emu = Emu(world, vl, grid_max=64, rows_max=rows)
    row = torch.linspace(-2, 2, vocab)
    lg = row.to(torch.bfloat16).repeat(rows, 1).to(DEV)
    pr = params(rows, "temperature", 3)
    pr[0][:] = 1.0
    got = emu.sample(lg, *pr)[0].cpu().numpy()
    freq = np.bincount(got, minlength=vocab) / rows
    want = torch.softmax(lg[0].float().cpu(), -1).numpy()
    assert np.abs(freq - want).max() < 0.03


def test_missing_peer_runs_out_of_time_and_reports():
    """Rank 0 of a two-rank group whose peer never launches: the flag wait gives up after its cycle
    limit, the kernel returns by itself with PIE_ERR_WAIT_PEER in the status word, and the host check
    raises. Nothing hangs and the context stays usable."""
    world, vl, rows = 2, 1024, 5
    lib = _lib.load(required=True)
    box = _lib.declare("pie_tp_sample_mailbox_bytes", [C.c_int, C.c_int], C.c_long)(8, world)
    xbuf = [torch.zeros(box, dtype=torch.uint8, device=DEV) for _ in range(world)]
    seq = torch.zeros(8, dtype=torch.int32, device=DEV)
    status = ops.kernel_status(DEV)
    status.zero_()
    blob = C.create_string_buffer(_lib.declare("pie_tp_sample_args_size", [], C.c_int)())
    fill = _lib.declare("pie_tp_sample_fill_args", [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                    C.c_int, C.c_int, C.c_int, C.c_int, C.c_longlong])
    arr = lambda ts: (C.c_void_p * world)(*[t.data_ptr() for t in ts])
    assert fill(blob, arr(xbuf), seq.data_ptr(), status.data_ptr(), world, 0, vl, 8, 2_000_000) == 0
    lg = make_logits(rows, vl, 1, True)
    pr = params(rows, "top_p", 1)
    out = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
    rc = _lib.fn("pie_tp_sample")(blob, lg.data_ptr(), lg.stride(0), rows, pr[0].data_ptr(), pr[1].data_ptr(),
                                  pr[2].data_ptr(), pr[3].data_ptr(), pr[4].data_ptr(), 0, 0, 0, out.data_ptr(),
                                  ops.num_sms(DEV), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()                     # returns: the wait is bounded
    assert int(status[0].item()) == 4               # PIE_ERR_WAIT_PEER
    with pytest.raises(_lib.KernelLibraryError):
        ops.check_kernel_status(DEV)
    assert int(status[0].item()) == 0
    assert float(torch.ones(4, device=DEV).sum().item()) == 4.0    # the context still works
