"""Numerics of every sm_100a kernel against the plain PyTorch fp32 reference of the same op."""
import math

import numpy as np
import pytest
import torch

from pie_b200 import ops
from pie_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def bf(*shape, scale=1.0, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=DEV) * scale).to(torch.bfloat16)


def close(a, b, atol, rtol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4g} (allowed {tol.max().item():.4g})"


def test_embed_and_shard():
    table = bf(1000, 256)
    tok = torch.randint(0, 1000, (77,), device=DEV, dtype=torch.int32)
    assert torch.equal(ops.embed(tok, table), ref.embed(tok, table))
    shard = table[250:500].contiguous()
    assert torch.equal(ops.embed(tok, shard, vocab_start=250), ref.embed(tok, shard, 250))


@pytest.mark.parametrize("hidden", [256, 2048, 4096, 5120, 8192])
def test_rmsnorm(hidden):
    x, w = bf(33, hidden, seed=1), bf(hidden, seed=2) + 1
    close(ops.rmsnorm(x, w, 1e-5), ref.rmsnorm(x, w, 1e-5), 2e-2)
    res, res2 = bf(33, hidden, seed=3), None
    res2 = res.clone()
    y = ops.add_rmsnorm(x, res, w, 1e-5)
    y2 = ref.add_rmsnorm(x, res2, w, 1e-5)
    close(res, res2, 1e-2)
    close(y, y2, 3e-2)


def test_swiglu():
    gu = bf(50, 2 * 1408, seed=4)
    close(ops.swiglu(gu), ref.swiglu(gu), 2e-2)


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
def test_glu_interleaved(act):
    gu = bf(50, 2 * 1408, seed=4) * 3
    close(ops.glu_interleaved(gu, act), ref.glu_interleaved(gu.float(), act).to(gu.dtype), 2e-2)
    assert ops.glu_interleaved(gu[:0], act).shape == (0, 1408)


@pytest.mark.parametrize("d,hq,hkv,norm", [(128, 8, 2, False), (64, 4, 2, True), (256, 4, 1, False)])
def test_qk_norm_rope_kvwrite_with_projection_bias(d, hq, hkv, norm):
    """The projection bias added inside the kernel equals adding it to the packed rows first."""
    n, page, pages = 33, 16, 8
    qkv = bf(n, (hq + 2 * hkv) * d, seed=5)
    bias = bf((hq + 2 * hkv) * d, seed=9)
    pos = torch.randint(0, 5000, (n,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(pages * page, device=DEV)[:n].to(torch.int32)
    inv = ref.rope_inv_freq(d, 500000.0, None, DEV)
    qn = (bf(d, seed=6) + 1) if norm else None
    kn = (bf(d, seed=7) + 1) if norm else None
    kv_a = torch.zeros(pages, 2, hkv, page, d, dtype=torch.bfloat16, device=DEV)
    kv_b = torch.zeros_like(kv_a)
    qa = ops.qk_norm_rope_kvwrite(qkv, pos, slots, inv, qn, kn, kv_a, hq, hkv, d, page, 1e-6, bias=bias)
    qb = ops.qk_norm_rope_kvwrite(qkv + bias, pos, slots, inv, qn, kn, kv_b, hq, hkv, d, page, 1e-6)
    assert torch.equal(qa, qb) and torch.equal(kv_a, kv_b)


@pytest.mark.parametrize("d,hq,hkv,norm", [(128, 8, 2, False), (128, 8, 2, True), (64, 4, 2, True)])
def test_qk_norm_rope_kvwrite(d, hq, hkv, norm):
    n, page, pages = 41, 16, 12
    qkv = bf(n, (hq + 2 * hkv) * d, seed=5)
    pos = torch.randint(0, 5000, (n,), device=DEV, dtype=torch.int32)
    perm = torch.randperm(pages * page, device=DEV)[:n].to(torch.int32)
    perm[3] = -1
    inv = ref.rope_inv_freq(d, 500000.0, None, DEV)
    qn = (bf(d, seed=6) + 1) if norm else None
    kn = (bf(d, seed=7) + 1) if norm else None
    kv1 = torch.zeros(pages, 2, hkv, page, d, dtype=torch.bfloat16, device=DEV)
    kv2 = kv1.clone()
    q1 = ops.qk_norm_rope_kvwrite(qkv, pos, perm, inv, qn, kn, kv1, hq, hkv, d, page, 1e-6)
    q2 = ref.qk_norm_rope_kvwrite(qkv, pos, perm, inv, qn, kn, kv2, hq, hkv, d, page, 1e-6)
    close(q1, q2, 3e-2)
    close(kv1, kv2, 3e-2)


def test_gather_copy_pages():
    x = bf(100, 512, seed=8)
    idx = torch.randint(0, 100, (37,), device=DEV, dtype=torch.int32)
    assert torch.equal(ops.gather_rows(x, idx), x[idx.long()])
    kv = bf(3, 10, 2, 2, 16, 64, seed=9)
    want = kv.clone()
    src = torch.tensor([1, 4], device=DEV, dtype=torch.int32)
    dst = torch.tensor([7, 2], device=DEV, dtype=torch.int32)
    want[:, dst.long()] = want[:, src.long()]
    ops.copy_pages(kv, src, dst)
    assert torch.equal(kv, want)


def test_brle_expand():
    rng = np.random.default_rng(0)
    rows, nbits = [], 1000
    for _ in range(9):
        runs, tot = [], 0
        while tot < nbits:
            r = int(rng.integers(0, 90))
            runs.append(r)
            tot += r
        rows.append(runs)
    rows.append([0, nbits])
    rows.append([nbits])
    rows.append([5, 3])      # short vector: tail is zeros
    got = ops.brle_expand(rows, nbits, DEV).cpu()
    want = ops.brle_expand(rows, nbits, "cpu")
    assert torch.equal(got, want)


def test_brle_expand_ragged_equals_row_by_row():
    rng = np.random.default_rng(1)
    rows, bits = [], []
    for nbits in (1, 31, 32, 33, 700, 64, 5000, 17):
        for _ in range(3):
            runs, tot = [], 0
            while tot < nbits:
                r = int(rng.integers(0, 90))
                runs.append(r)
                tot += r
            rows.append(runs)
            bits.append(nbits)
    rows.append([4, 2])          # short row: the tail is zeros
    bits.append(100)
    got, offs = ops.brle_expand_ragged(rows, bits, DEV)
    assert offs[-1] == got.numel() == sum((b + 31) // 32 for b in bits)
    for i, (r, b) in enumerate(zip(rows, bits)):
        want = ops.brle_expand([r], b, "cpu").reshape(-1)
        assert torch.equal(got[offs[i]:offs[i + 1]].cpu(), want), (i, b)
    cpu, offs2 = ops.brle_expand_ragged(rows, bits, "cpu")
    assert torch.equal(cpu, got.cpu()) and np.array_equal(offs, offs2)


def make_paged(nreq, kv_lens, hkv, d, page, seed=0, extra_pages=5):
    npages = [-(-int(k) // page) for k in kv_lens]
    total = sum(npages) + extra_pages
    kv = bf(total, 2, hkv, page, d, seed=seed)
    perm = torch.randperm(total)[: sum(npages)].numpy().astype(np.int32)
    indptr = np.zeros(nreq + 1, dtype=np.int32)
    indptr[1:] = np.cumsum(npages)
    return kv, perm, indptr


@pytest.mark.parametrize("d,hq,hkv", [(128, 32, 8), (128, 8, 1), (64, 4, 2), (128, 16, 16), (128, 16, 1)])
def test_paged_decode_attention(d, hq, hkv):
    page = 16
    kv_lens = np.array([1, 15, 16, 17, 300, 1000, 2305, 64], dtype=np.int32)
    r = len(kv_lens)
    kv, pages, indptr = make_paged(r, kv_lens, hkv, d, page, seed=11)
    q = bf(r, hq, d, seed=12)
    item_req, st, en, iptr = ops.plan_decode_items(kv_lens, hkv, target_ctas=64, min_chunk=256)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)
    max_items = len(item_req) + 3
    plan = ops.DecodePlan(t(pages), t(indptr), t(item_req), t(st), t(en), t(iptr),
                          torch.tensor([len(item_req)], dtype=torch.int32, device=DEV),
                          torch.empty(ops.decode_scratch_floats(max_items, hq, d), device=DEV),
                          max_items, r, 64, page)
    scale = 1 / math.sqrt(d)
    out = ops.paged_decode_attention(q, kv, plan, scale)
    qo = np.arange(r + 1, dtype=np.int32)
    want = ref.paged_attention(q, kv, qo, indptr, torch.from_numpy(pages).to(DEV), kv_lens, scale)
    close(out, want, 2e-2)


@pytest.mark.parametrize("d,hq,hkv,softcap,window", [(256, 8, 4, 0.0, -1), (256, 8, 1, 0.0, 100), (256, 16, 16, 0.0, -1), (256, 8, 2, 1.5, -1),
                                                     (128, 32, 8, 1.5, -1), (128, 16, 8, 2.0, 100), (64, 4, 2, 1.5, -1)])
def test_paged_decode_attention_head_dim_256_and_softcap(d, hq, hkv, softcap, window):
    """head_dim 256 (Gemma sizes) and soft-capped scores (softmax over cap * tanh(s / cap), Gemma-2), alone and together."""
    page = 16
    kv_lens = np.array([1, 15, 16, 17, 300, 1000, 2305, 64], dtype=np.int32)
    r = len(kv_lens)
    kv, pages, indptr = make_paged(r, kv_lens, hkv, d, page, seed=11)
    q = bf(r, hq, d, seed=12)
    item_req, st, en, iptr = ops.plan_decode_items(kv_lens, hkv, target_ctas=64, min_chunk=256, window_left=window)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)
    max_items = len(item_req) + 3
    plan = ops.DecodePlan(t(pages), t(indptr), t(item_req), t(st), t(en), t(iptr),
                          torch.tensor([len(item_req)], dtype=torch.int32, device=DEV),
                          torch.empty(ops.decode_scratch_floats(max_items, hq, d), device=DEV),
                          max_items, r, 64, page, window_left=window)
    scale = 1 / math.sqrt(d)
    out = ops.paged_decode_attention(q, kv, plan, scale, softcap=softcap)
    qo = np.arange(r + 1, dtype=np.int32)
    want = ref.paged_attention(q, kv, qo, indptr, torch.from_numpy(pages).to(DEV), kv_lens, scale, window_left=window,
                               softcap=softcap)
    close(out, want, 2e-2)
    if softcap:     # the cap changes the result: the test would not pass without it
        plain = ref.paged_attention(q, kv, qo, indptr, torch.from_numpy(pages).to(DEV), kv_lens, scale, window_left=window)
        assert (plain.float() - want.float()).abs().max() > 0.05


@pytest.mark.parametrize("d,hq,hkv,softcap,rows", [(256, 8, 4, 0.0, 64), (256, 4, 4, 0.0, 64), (256, 8, 1, 1.5, 64), (128, 32, 8, 1.5, 64),
                                                   (64, 4, 2, 2.0, 64), (128, 32, 8, 1.5, 256), (128, 32, 16, 2.0, 256), (128, 8, 1, 1.5, 256),
                                                   (64, 16, 2, 2.0, 256)])
@pytest.mark.parametrize("mode", ["causal", "custom", "window"])
def test_paged_prefill_attention_head_dim_256_and_softcap(d, hq, hkv, softcap, rows, mode):
    """head_dim 256 on the 64-row kernel (the tcgen05 kernel stops at 128); soft-capped scores on both kernels (the
    tcgen05 one in its two-tile form)."""
    page = 16
    assert ops.prefill_tile_rows(hq, hkv, d, page, softcap=bool(softcap)) == (64 if d == 256 else 256)
    qlens = np.array([1, 5, 64, 130, 17, 700], dtype=np.int32)
    prev = np.array([40, 0, 0, 200, 31, 333], dtype=np.int32)
    kv_lens = qlens + prev
    r = len(qlens)
    kv, pages, indptr = make_paged(r, kv_lens, hkv, d, page, seed=21)
    qo = np.zeros(r + 1, dtype=np.int32)
    qo[1:] = np.cumsum(qlens)
    q = bf(int(qo[-1]), hq, d, seed=22)
    masks, window = None, -1
    if mode == "custom":
        rng = np.random.default_rng(5)
        masks = []
        for i in range(r):
            m = rng.random((qlens[i], kv_lens[i])) < 0.6
            m[:, 0] = True
            masks.append(m if i != 2 else None)
    if mode == "window":
        window = 37
    plan = ops.build_prefill_plan(ops.AttnBatch(qo, indptr, pages, kv_lens, masks, window), hq // hkv, page, DEV, tile_rows=rows)
    scale = 1 / math.sqrt(d)
    lse = torch.empty(int(qo[-1]), hq, device=DEV)
    out = ops.paged_prefill_attention(q, kv, plan, scale, lse_out=lse, softcap=softcap)
    ops.check_kernel_status(DEV)
    tmasks = None if masks is None else [None if m is None else torch.from_numpy(m) for m in masks]
    want, want_lse = ref.paged_attention(q, kv, qo, indptr, torch.from_numpy(pages).to(DEV), kv_lens, scale,
                                         masks=tmasks, window_left=window, return_lse=True, softcap=softcap)
    close(out, want, 2e-2)
    close(lse, want_lse, 2e-2)


@pytest.mark.parametrize("d,hq,hkv", [(128, 32, 8), (128, 4, 1), (64, 16, 2), (128, 16, 16), (128, 16, 1)])
def test_paged_decode_attention_shared_prefix(d, hq, hkv):
    """Forks of one context share their leading pages: the cascade plan reads those pages once per
    tile of members and must give what the plain per-request plan gives."""
    page = 16
    rng = np.random.default_rng(5)
    tables, kv_lens = [], []
    nxt = 0
    for g, (members, shared_pages) in enumerate([(8, 40), (3, 17), (11, 64)]):
        shared = list(range(nxt, nxt + shared_pages))
        nxt += shared_pages
        for b in range(members):
            own_n = int(rng.integers(1, 9))
            tables.append(shared + list(range(nxt, nxt + own_n)))
            nxt += own_n
            kv_lens.append(shared_pages * page + (own_n - 1) * page + int(rng.integers(1, page + 1)))
    for n in (1, 3, 70):                                   # requests that share nothing
        tables.append(list(range(nxt, nxt + n)))
        nxt += n
        kv_lens.append((n - 1) * page + int(rng.integers(1, page + 1)))
    order = rng.permutation(len(tables))
    tables, kv_lens = [tables[i] for i in order], np.array([kv_lens[i] for i in order], dtype=np.int32)
    r = len(tables)
    phys = rng.permutation(nxt + 7)[:nxt].astype(np.int32)          # logical -> physical page ids
    indptr = np.zeros(r + 1, dtype=np.int32)
    indptr[1:] = np.cumsum([len(t) for t in tables])
    pages = np.concatenate([phys[np.array(t)] for t in tables]).astype(np.int32)
    kv = bf(nxt + 7, 2, hkv, page, d, seed=71)
    q = bf(r, hq, d, seed=72)
    groups = ops.find_shared_prefixes(kv_lens, indptr, pages, page, min_shared_tokens=64)
    assert sorted(len(m) for m, _ in groups) == [3, 8, 11]
    assert sorted(st for _, st in groups) == [17 * page, 40 * page, 64 * page]
    cp = ops.plan_decode_cascade(kv_lens, groups, hkv, hq // hkv, target_ctas=64, max_items=4096, min_chunk=256)
    if hq // hkv == 16:               # one request's heads fill the 16-row tile: no shared items to make
        assert cp is None
        return
    assert cp is not None and cp.shared_tokens > 0
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)
    max_items = int(cp.req_slot_indptr[-1]) + 5
    status = ops.kernel_status(DEV)
    status.zero_()
    plan = ops.DecodePlan(t(pages), t(indptr), t(cp.item_req), t(cp.item_start), t(cp.item_end), t(cp.req_slot_indptr),
                          torch.tensor([len(cp.item_req)], dtype=torch.int32, device=DEV),
                          torch.empty(ops.decode_scratch_floats(max_items, hq, d), device=DEV), max_items, r, 64, page,
                          item_slot=t(cp.item_slot), item_tile=t(cp.item_tile), tile_members=t(cp.tile_members))
    scale = 1 / math.sqrt(d)
    out = ops.paged_decode_attention(q, kv, plan, scale)
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0
    qo = np.arange(r + 1, dtype=np.int32)
    want = ref.paged_attention(q, kv, qo, indptr, torch.from_numpy(pages).to(DEV), kv_lens, scale)
    close(out, want, 2e-2)
    # attention sinks merge the same way over shared and unshared slots
    sinks = torch.linspace(-1.0, 2.0, hq, device=DEV)
    sl2 = (sinks * 1.4426950408889634).float().contiguous()
    out = ops.paged_decode_attention(q, kv, plan, scale, sinks_log2=sl2)
    want = ref.paged_attention(q, kv, qo, indptr, torch.from_numpy(pages).to(DEV), kv_lens, scale, sinks=sinks)
    close(out, want, 2e-2)


def test_paged_decode_attention_clamps_work_count():
    """A work count in device memory larger than the scratch was sized for (a stale value on a graph
    replay, an embedder's mistake) must not write past the scratch: the kernel drops the extra items,
    reports PIE_ERR_BOUNDS and the requests whose items are all covered still come out right."""
    d, hq, hkv, page = 128, 32, 8, 16
    kv_lens = np.array([300, 17, 1000, 2305], dtype=np.int32)
    r = len(kv_lens)
    kv, pages, indptr = make_paged(r, kv_lens, hkv, d, page, seed=61)
    q = bf(r, hq, d, seed=62)
    item_req, st, en, iptr = ops.plan_decode_items(kv_lens, hkv, target_ctas=64, min_chunk=256)
    covered = int(iptr[2])                       # every item of requests 0 and 1
    assert covered < len(item_req) and iptr[3] > covered + 1
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)
    need = ops.decode_scratch_floats(covered, hq, d)
    big = torch.full((need + 65536,), 777.0, device=DEV)
    status = ops.kernel_status(DEV)
    status.zero_()
    plan = ops.DecodePlan(t(pages), t(indptr), t(item_req), t(st), t(en), t(iptr),
                          torch.tensor([len(item_req)], dtype=torch.int32, device=DEV), big, covered, r, 64, page)
    scale = 1 / math.sqrt(d)
    out = ops.paged_decode_attention(q, kv, plan, scale)
    torch.cuda.synchronize()
    assert int(status[0].item()) == 5               # PIE_ERR_BOUNDS
    with pytest.raises(ops._lib.KernelLibraryError):
        ops.check_kernel_status(DEV)
    assert int(status[0].item()) == 0
    assert bool((big[need:] == 777.0).all())     # nothing written past the scratch
    qo = np.arange(r + 1, dtype=np.int32)
    want = ref.paged_attention(q, kv, qo, indptr, torch.from_numpy(pages).to(DEV), kv_lens, scale)
    close(out[:2], want[:2], 2e-2)
    # an item that names a request outside the batch is skipped and reported as well
    bad = item_req.copy()
    bad[-1] = r + 5
    plan = ops.DecodePlan(t(pages), t(indptr), t(bad), t(st), t(en), t(iptr),
                          torch.tensor([len(item_req)], dtype=torch.int32, device=DEV),
                          torch.empty(ops.decode_scratch_floats(len(item_req), hq, d), device=DEV),
                          len(item_req), r, 64, page)
    out = ops.paged_decode_attention(q, kv, plan, scale)
    torch.cuda.synchronize()
    assert int(status[0].item()) == 5
    status.zero_()
    close(out[:3], want[:3], 2e-2)


@pytest.mark.parametrize("d,hq,hkv", [(128, 32, 8), (64, 16, 2)])
def test_attention_sinks_and_per_call_window(d, hq, hkv):
    """Per-head sink logits in the softmax denominator (decode: single-item and merged requests;
    prefill: both kernels) and a window given per call over a plan that covers the whole range."""
    page = 16
    sinks = torch.linspace(-2.0, 3.0, hq, device=DEV)
    sl2 = (sinks * 1.4426950408889634).float().contiguous()
    scale = 1 / math.sqrt(d)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)
    # decode
    kv_lens = np.array([1, 17, 300, 2305, 64], dtype=np.int32)
    r = len(kv_lens)
    kv, pages, indptr = make_paged(r, kv_lens, hkv, d, page, seed=51)
    q = bf(r, hq, d, seed=52)
    item_req, st, en, iptr = ops.plan_decode_items(kv_lens, hkv, target_ctas=64, min_chunk=256)
    max_items = len(item_req) + 3
    plan = ops.DecodePlan(t(pages), t(indptr), t(item_req), t(st), t(en), t(iptr),
                          torch.tensor([len(item_req)], dtype=torch.int32, device=DEV),
                          torch.empty(ops.decode_scratch_floats(max_items, hq, d), device=DEV), max_items, r, 64, page)
    qo = np.arange(r + 1, dtype=np.int32)
    for window in (-1, 40):
        out = ops.paged_decode_attention(q, kv, plan, scale, window_left=window, sinks_log2=sl2)
        want = ref.paged_attention(q, kv, qo, indptr, torch.from_numpy(pages).to(DEV), kv_lens, scale,
                                   window_left=window, sinks=sinks)
        close(out, want, 2e-2)
    # prefill
    qlens = np.array([5, 130, 300], dtype=np.int32)
    kv_lens = qlens + np.array([40, 0, 77], dtype=np.int32)
    kv, pages, indptr = make_paged(3, kv_lens, hkv, d, page, seed=53)
    qo = np.zeros(4, dtype=np.int32)
    qo[1:] = np.cumsum(qlens)
    q = bf(int(qo[-1]), hq, d, seed=54)
    batch = ops.AttnBatch(qo, indptr, pages, kv_lens, None, -1)
    for rows in [64, 128, 256]:
        plan = ops.build_prefill_plan(batch, hq // hkv, page, DEV, tile_rows=rows)
        for window in (-1, 33):
            out = ops.paged_prefill_attention(q, kv, plan, scale, window_left=window, sinks_log2=sl2)
            want = ref.paged_attention(q, kv, qo, indptr, torch.from_numpy(pages).to(DEV), kv_lens, scale,
                                       window_left=window, sinks=sinks)
            close(out, want, 2e-2)
    ops.check_kernel_status(DEV)


@pytest.mark.parametrize("window", [0, 15, 16, 100, 1000])
def test_paged_decode_attention_sliding_window(window):
    """Decode attention over the last window + 1 keys only: the plan starts at the 16-token boundary
    below the first visible key and the kernel masks the keys under it."""
    d, hq, hkv, page = 128, 32, 8, 16
    kv_lens = np.array([1, 15, 16, 17, 300, 1000, 2305, 64], dtype=np.int32)
    r = len(kv_lens)
    kv, pages, indptr = make_paged(r, kv_lens, hkv, d, page, seed=13)
    q = bf(r, hq, d, seed=14)
    item_req, st, en, iptr = ops.plan_decode_items(kv_lens, hkv, target_ctas=64, min_chunk=256, window_left=window)
    assert (st % 16 == 0).all() and (en[iptr[1:] - 1] == kv_lens).all()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)
    max_items = len(item_req) + 3
    plan = ops.DecodePlan(t(pages), t(indptr), t(item_req), t(st), t(en), t(iptr),
                          torch.tensor([len(item_req)], dtype=torch.int32, device=DEV),
                          torch.empty(ops.decode_scratch_floats(max_items, hq, d), device=DEV),
                          max_items, r, 64, page, window_left=window)
    scale = 1 / math.sqrt(d)
    out = ops.paged_decode_attention(q, kv, plan, scale)
    qo = np.arange(r + 1, dtype=np.int32)
    want = ref.paged_attention(q, kv, qo, indptr, torch.from_numpy(pages).to(DEV), kv_lens, scale, window_left=window)
    close(out, want, 2e-2)


@pytest.mark.parametrize("d,hq,hkv,rows", [(128, 32, 8, 64), (128, 8, 1, 64), (64, 4, 2, 64),
                                           (128, 32, 8, 128), (128, 8, 1, 128), (128, 4, 4, 128),
                                           (128, 32, 2, 128), (128, 8, 4, 128), (128, 32, 8, 256),
                                           (128, 8, 1, 256), (128, 4, 4, 256), (128, 32, 2, 256),
                                           (64, 4, 2, 128), (64, 16, 2, 256), (64, 64, 8, 256), (64, 8, 8, 128)])
@pytest.mark.parametrize("mode", ["causal", "custom", "window", "custom_window"])
def test_paged_prefill_attention(d, hq, hkv, rows, mode):
    """rows = 64: the mma.sync kernel; rows = 128 / 256: the tcgen05 kernel with one / two MMA
    tiles per CTA (head_dim 128, 16-token pages)."""
    page = 16
    if rows > 64:
        assert ops._lib.fn("pie_prefill_attn_tc_supported")(hq, hkv, d, page) == 1
    qlens = np.array([1, 5, 64, 130, 17, 700], dtype=np.int32)
    prev = np.array([40, 0, 0, 200, 31, 333], dtype=np.int32)
    kv_lens = qlens + prev
    r = len(qlens)
    kv, pages, indptr = make_paged(r, kv_lens, hkv, d, page, seed=21)
    qo = np.zeros(r + 1, dtype=np.int32)
    qo[1:] = np.cumsum(qlens)
    q = bf(int(qo[-1]), hq, d, seed=22)
    masks = None
    window = -1
    if mode in ("custom", "custom_window"):      # custom_window: a layer's window bounds the left side under a custom mask too
        rng = np.random.default_rng(5)
        masks = []
        for i in range(r):
            m = rng.random((qlens[i], kv_lens[i])) < 0.6
            m[:, 0] = True
            masks.append(m if i != 2 else None)
    if mode in ("window", "custom_window"):
        window = 37
    batch = ops.AttnBatch(qo, indptr, pages, kv_lens, masks, window)
    plan = ops.build_prefill_plan(batch, hq // hkv, page, DEV, tile_rows=rows)
    scale = 1 / math.sqrt(d)
    lse = torch.empty(int(qo[-1]), hq, device=DEV)
    out = ops.paged_prefill_attention(q, kv, plan, scale, lse_out=lse)
    ops.check_kernel_status(DEV)
    tmasks = None if masks is None else [None if m is None else torch.from_numpy(m) for m in masks]
    want, want_lse = ref.paged_attention(q, kv, qo, indptr, torch.from_numpy(pages).to(DEV), kv_lens, scale,
                                         masks=tmasks, window_left=window, return_lse=True)
    close(out, want, 2e-2)
    close(lse, want_lse, 2e-2)


@pytest.mark.parametrize("rows", [128, 256])
def test_prefill_tc_rescales_accumulator_when_scores_grow(rows):
    """Large score magnitudes make block maxima outgrow the lazily updated reference maximum, so
    the kernel's rescale of its TMEM accumulator runs in ordinary causal blocks too."""
    d, hq, hkv, page = 128, 8, 2, 16
    qlens = np.array([300, 77], dtype=np.int32)
    prev = np.array([500, 0], dtype=np.int32)
    kv_lens = qlens + prev
    kv, pages, indptr = make_paged(2, kv_lens, hkv, d, page, seed=41)
    qo = np.zeros(3, dtype=np.int32)
    qo[1:] = np.cumsum(qlens)
    q = bf(int(qo[-1]), hq, d, seed=42, scale=8.0)
    batch = ops.AttnBatch(qo, indptr, pages, kv_lens, None, -1)
    plan = ops.build_prefill_plan(batch, hq // hkv, page, DEV, tile_rows=rows)
    scale = 1 / math.sqrt(d)
    lse = torch.empty(int(qo[-1]), hq, device=DEV)
    out = ops.paged_prefill_attention(q, kv, plan, scale, lse_out=lse)
    ops.check_kernel_status(DEV)
    want, want_lse = ref.paged_attention(q, kv, qo, indptr, torch.from_numpy(pages).to(DEV), kv_lens, scale,
                                         return_lse=True)
    close(out, want, 3e-2)
    close(lse, want_lse, 5e-2, rtol=1e-2)


def test_row_stats():
    lg = bf(7, 4096, scale=3.0, seed=30)
    close(ops.row_stats(lg), ref.row_stats(lg), 2e-3, rtol=1e-3)


def _params(rows, t, k, p, mp, seed0=1):
    return (torch.full((rows,), t, device=DEV), torch.full((rows,), k, dtype=torch.int32, device=DEV),
            torch.full((rows,), p, device=DEV), torch.full((rows,), mp, device=DEV),
            torch.arange(seed0, seed0 + rows, dtype=torch.int64, device=DEV))


def test_sample_argmax_and_topk1():
    lg = bf(16, 32000, scale=2.0, seed=31)
    want = lg.float().argmax(-1).int()
    got = ops.sample(lg, *_params(16, 0.0, 0, 1.0, 0.0))
    assert torch.equal(got, want)
    got = ops.sample(lg, *_params(16, 1.0, 1, 1.0, 0.0))
    # top-k = 1 keeps every token tied with the maximum (bf16 ties are common)
    mx = lg.float().amax(-1)
    assert bool((lg.float()[torch.arange(16), got.long()] == mx).all())


@pytest.mark.parametrize("t,k,p,mp", [(1.0, 50, 1.0, 0.0), (0.8, 0, 0.9, 0.0), (1.0, 0, 1.0, 0.05), (0.7, 40, 0.95, 0.0)])
def test_sample_stays_in_kept_set(t, k, p, mp):
    rows, vocab = 64, 8192
    lg = bf(rows, vocab, scale=3.0, seed=32)
    got = ops.sample(lg, *_params(rows, t, k, p, mp)).cpu()
    lgc = lg.cpu()
    for r in range(rows):
        keep = ref.kept_set(lgc[r], t, k, p, mp)
        assert bool(keep[got[r]]), f"row {r}: token {int(got[r])} outside the kept set"


def test_sample_distribution_matches_softmax():
    vocab, draws = 64, 20000
    row = (torch.randn(vocab, generator=torch.Generator().manual_seed(3)) * 1.5).to(torch.bfloat16)
    lg = row.to(DEV).repeat(draws, 1).contiguous()
    got = ops.sample(lg, *_params(draws, 1.0, 0, 1.0, 0.0, seed0=1000)).cpu()
    freq = torch.bincount(got.long(), minlength=vocab).float() / draws
    p = torch.softmax(row.float(), -1)
    assert float((freq - p).abs().max()) < 0.02
    # same seeds -> same tokens (counter-based stream)
    again = ops.sample(lg, *_params(draws, 1.0, 0, 1.0, 0.0, seed0=1000)).cpu()
    assert torch.equal(got, again)


def test_sample_with_vocab_mask():
    rows, vocab = 8, 4096
    lg = bf(rows, vocab, scale=2.0, seed=33)
    runs = [[100, 50, 1000, 7]]           # allowed: [100,150) and [1150,1157)
    bits = ops.brle_expand(runs, vocab, DEV)
    mrow = torch.tensor([0, -1] * 4, dtype=torch.int32, device=DEV)
    got = ops.sample(lg, *_params(rows, 1.0, 0, 1.0, 0.0), mask_bits=bits, mask_row=mrow).cpu()
    for r in range(0, rows, 2):
        t = int(got[r])
        assert 100 <= t < 150 or 1150 <= t < 1157
    # greedy under a mask = arg-max over the allowed set
    got = ops.sample(lg, *_params(rows, 0.0, 0, 1.0, 0.0), mask_bits=bits, mask_row=mrow).cpu()
    allowed = torch.zeros(vocab, dtype=torch.bool)
    allowed[100:150] = True
    allowed[1150:1157] = True
    for r in range(0, rows, 2):
        want = int(lg[r].float().cpu().masked_fill(~allowed, float("-inf")).argmax())
        assert int(got[r]) == want


def test_fp8_block_dequant_and_gemm():
    """fp8 weights with per-row x 128-column scales: the dequant kernel equals the PyTorch
    expansion, and the fp8-weight GEMM (with each epilogue) equals the bf16 GEMM over it."""
    from pie_b200 import ops
    from pie_b200.ops import reference as ref
    torch.manual_seed(5)
    n, k, m = 1536, 2048, 200
    w = (torch.randn(n, k, device="cuda") * 0.05)
    q = ops.quantize_fp8_block(w)
    assert q.w8.dtype == torch.float8_e4m3fn and q.scale.shape == (n, k // 128)
    deq = ops.dequant_fp8(q)
    want = (q.w8.float() * q.scale.repeat_interleave(128, dim=1)).to(torch.bfloat16)
    assert torch.equal(deq, want)
    assert (deq.float() - w).abs().max() / w.abs().max() < 0.07
    x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
    r = (torch.randn(m, n, device="cuda") * 0.5).to(torch.bfloat16)
    full = x.float() @ deq.float().t()
    y = ops.gemm_fp8w(x, q, mode="dequant")
    assert (y.float() - full).abs().max() < 0.05 * full.abs().max()
    y = ops.gemm_fp8w(x, q, residual=r, epilogue=ops.EPI_RESIDUAL, mode="dequant")
    assert (y.float() - (full + r.float())).abs().max() < 0.05 * full.abs().max()
    y = ops.gemm_fp8w(x, q, epilogue=ops.EPI_SWIGLU, mode="dequant")
    assert (y.float() - ref.swiglu_interleaved(full)).abs().max() < 0.05 * full.abs().max()
    ops.check_kernel_status()


@pytest.mark.parametrize("m,n,k", [(64, 1536, 2048), (200, 1024, 5120), (512, 6400, 5120), (1000, 640, 3200), (130, 2016, 1024)])
@pytest.mark.parametrize("epi", ["store", "residual", "swiglu"])
def test_fp8_blockscaled_gemm_fused(m, n, k, epi):
    """fp8 x fp8 tcgen05 GEMM with 1x128 activation scales and per-row x 128 weight scales against
    the fp32 evaluation of the same quantised operands; and close to the unquantised product."""
    from pie_b200 import ops
    from pie_b200.ops import reference as ref
    torch.manual_seed(m + n)
    w = torch.randn(n, k, device="cuda") * 0.05
    x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
    r = (torch.randn(m, n, device="cuda") * 0.5).to(torch.bfloat16) if epi == "residual" else None
    q = ops.quantize_fp8_block(w)
    x8, sx = ops.quant_act_fp8(x)
    # the quantiser itself: dequantised activations within fp8 rounding of the input
    xd = x8.float() * sx.repeat_interleave(128, dim=1)[:, :k]
    assert (xd - x.float()).abs().max() <= 0.07 * x.float().abs().max()
    want = ops.gemm_fp8_reference(x8, sx, q)
    e = {"store": ops.EPI_STORE, "residual": ops.EPI_RESIDUAL, "swiglu": ops.EPI_SWIGLU}[epi]
    if epi == "residual":
        want = want + r.float()
    if epi == "swiglu":
        want = ref.swiglu_interleaved(want)
    y = ops.gemm_fp8w(x, q, residual=r, epilogue=e, mode="fused")
    torch.cuda.synchronize()
    ops.check_kernel_status()
    tol = 2e-2 * want.abs().max().item() + 1e-3 * k ** 0.5
    assert (y.float() - want).abs().max().item() <= tol
    if epi == "store":
        exact = x.float() @ w.t()
        rel = (y.float() - exact).norm() / exact.norm()
        assert rel < 0.06, rel


@pytest.mark.parametrize("k,p", [(0, 0.6), (5, 1.0), (8, 0.8), (0, 0.05)])
def test_sample_topk_topp_distribution_is_renormalised_kept_set(k, p):
    """Draws under top-k / top-p follow the softmax renormalised over the kept set (rejection
    rounds and the radix fallback for a small top-p must agree with the reference set)."""
    vocab, draws = 64, 20000
    row = (torch.randn(vocab, generator=torch.Generator().manual_seed(9)) * 1.5).to(torch.bfloat16)
    lg = row.to(DEV).repeat(draws, 1).contiguous()
    got = ops.sample(lg, *_params(draws, 1.0, k, p, 0.0, seed0=77)).cpu()
    keep = ref.kept_set(row, 1.0, k, p, 0.0)
    assert bool(keep[got.long()].all())
    probs = torch.softmax(row.float(), -1) * keep
    probs = probs / probs.sum()
    freq = torch.bincount(got.long(), minlength=vocab).float() / draws
    assert float((freq - probs).abs().max()) < 0.02


def test_bounded_peer_wait_times_out_and_reports_status():
    """A wait on a peer flag that nothing sets gives up after its bound, records
    PIE_ERR_WAIT_PEER (4) in the status word and returns; the context stays usable and
    `check_kernel_status` raises and clears the word."""
    import ctypes as C
    import time
    from pie_b200.ops import _lib
    wait = _lib.declare("pie_tp_wait_ag", [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p])
    flags = torch.zeros(8, dtype=torch.int32, device=DEV)          # never raised
    epoch = torch.ones(1, dtype=torch.int32, device=DEV)           # the kernel expects flags >= 1
    status = ops.kernel_status(DEV)
    status.zero_()
    t0 = time.time()
    _lib.check(wait(flags.data_ptr(), epoch.data_ptr(), 2, status.data_ptr(), _lib.stream_ptr()), "tp_wait_ag")
    torch.cuda.synchronize()
    assert time.time() - t0 < 10.0
    assert int(status[0].item()) == 4
    with pytest.raises(_lib.KernelLibraryError):
        ops.check_kernel_status(DEV)
    assert int(status[0].item()) == 0
    # the device still works
    x = torch.ones(1024, device=DEV)
    assert float(x.sum()) == 1024.0
    # and a wait whose flags are already up returns at once with a clean status
    flags.fill_(1)
    _lib.check(wait(flags.data_ptr(), epoch.data_ptr(), 2, status.data_ptr(), _lib.stream_ptr()), "tp_wait_ag")
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0


def test_index_validator_records_the_first_bad_entry_and_touches_nothing():
    """The `PIE_BOUNDS=1` check: entries outside [lo, hi) set PIE_ERR_BOUNDS with table and position; the
    status check raises with them and clears the block, and a clean table leaves it alone."""
    from pie_b200.ops import _lib
    ops.kernel_status(DEV).zero_()
    good = torch.arange(0, 1000, dtype=torch.int32, device=DEV)
    ops.validate_indices(good, 0, 1000, "kv_page_indices")
    torch.cuda.synchronize()
    ops.check_kernel_status(DEV)
    bad = good.clone()
    bad[637] = 1000
    ops.validate_indices(bad, 0, 1000, "kv_page_indices")
    torch.cuda.synchronize()
    with pytest.raises(_lib.KernelLibraryError, match=r"kv_page_indices\[637\]"):
        ops.check_kernel_status(DEV)
    ops.check_kernel_status(DEV)                              # cleared
    neg = good.clone()
    neg[3] = -1
    ops.validate_indices(neg, 0, 1000, "tokens")
    torch.cuda.synchronize()
    with pytest.raises(_lib.KernelLibraryError, match=r"tokens\[3\]"):
        ops.check_kernel_status(DEV)


@pytest.mark.parametrize("dk,dv,hk,hv", [(32, 32, 2, 4), (64, 64, 2, 2), (128, 128, 2, 4)])
def test_gdn_mixer_matches_reference_over_chunks(dk, dv, hk, hv):
    """Gated DeltaNet mixer kernels (short convolution with slot tails, token-serial delta rule, gated norm)
    against the fp32 reference: a ragged batch, then a second fire that continues from the cached state."""
    from types import SimpleNamespace
    from pie_b200.driver.recurrent import RecurrentStateCache
    from pie_b200.models.config import ModelConfig
    torch.manual_seed(dk + hv)
    cfg = ModelConfig(model_type="qwen3_5", num_hidden_layers=1, layer_types=["linear_attention"], linear_num_key_heads=hk,
                      linear_num_value_heads=hv, linear_key_head_dim=dk, linear_value_head_dim=dv)
    c, f = cfg.gdn_conv_channels, cfg.gdn_in_features
    lw_f = {"gdn_conv": torch.randn(c, 4) * 0.3, "gdn_A_log": torch.randn(hv) * 0.5, "gdn_dt_bias": torch.randn(hv) * 0.5,
            "gdn_norm": 1 + torch.randn(dv) * 0.1}
    lw_f = {k: v.to(torch.bfloat16).float() if k in ("gdn_conv", "gdn_norm") else v for k, v in lw_f.items()}
    lw_d = {k: (v.to(DEV).to(torch.bfloat16) if k in ("gdn_conv", "gdn_norm") else v.to(DEV)) for k, v in lw_f.items()}
    dev_cache, cpu_cache = RecurrentStateCache(cfg, 6, DEV), RecurrentStateCache(cfg, 6, "cpu")
    for lens, reset in (([5, 1, 37, 2], [1, 1, 1, 1]), ([1, 3, 1, 40], [0, 0, 0, 0]), ([2, 1, 1, 1], [1, 0, 0, 0])):
        qo = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        slots = np.asarray([4, 0, 2, 5], np.int32)
        mix = (torch.randn(int(qo[-1]), f) * 1.5).to(torch.bfloat16)
        want = ref.gdn_mixer(mix.float(), lw_f["gdn_conv"], lw_f["gdn_A_log"], lw_f["gdn_dt_bias"], lw_f["gdn_norm"], 1e-5,
                             hk, hv, dk, dv, qo.tolist(), cpu_cache.conv_state[0], cpu_cache.rec_state[0],
                             slots.tolist(), reset)
        got = ops.gdn_mixer(mix.to(DEV), lw_d, cfg, dev_cache.inputs(qo, slots, np.asarray(reset, np.int32)), 0)
        torch.cuda.synchronize()
        close(got.cpu(), want, 3e-2)
        assert torch.allclose(dev_cache.rec_state.cpu(), cpu_cache.rec_state, atol=2e-2, rtol=2e-2)
        assert torch.allclose(dev_cache.conv_state.cpu(), cpu_cache.conv_state, atol=1e-6)
    dev_cache.copy_slot(4, 1)
    torch.cuda.synchronize()
    assert torch.equal(dev_cache.rec_state[:, 1], dev_cache.rec_state[:, 4])
    assert torch.equal(dev_cache.conv_state[:, 1], dev_cache.conv_state[:, 4])


@pytest.mark.parametrize("heads,head_dim,state,groups", [(8, 32, 16, 2), (4, 64, 128, 1), (8, 64, 64, 4)])
def test_mamba2_mixer_matches_reference_over_chunks(heads, head_dim, state, groups):
    """Mamba-2 mixer (convolution with bias and slot tails, state-space update, gate + norm) against the fp32
    reference: a ragged batch, a second fire continuing from the cached state, and a reset."""
    from pie_b200.driver.recurrent import RecurrentStateCache
    from pie_b200.models.config import ModelConfig
    torch.manual_seed(heads + state)
    cfg = ModelConfig(model_type="mamba2_hybrid", num_hidden_layers=1, layer_types=["mamba2"], mamba_num_heads=heads,
                      mamba_head_dim=head_dim, ssm_state_size=state, mamba_n_groups=groups)
    c, f, inner = cfg.mamba_conv_channels, cfg.mamba_in_features, cfg.mamba_inner
    rb = lambda t: t.to(torch.bfloat16).float()
    lw_f = {"mamba_conv": rb(torch.randn(c, 4) * 0.3), "mamba_conv_bias": rb(torch.randn(c) * 0.1),
            "mamba_A_log": torch.randn(heads) * 0.5, "mamba_dt_bias": torch.randn(heads) * 0.5,
            "mamba_D": 1 + torch.randn(heads) * 0.2, "mamba_norm": rb(1 + torch.randn(inner) * 0.1)}
    bf = ("mamba_conv", "mamba_conv_bias", "mamba_norm")
    lw_d = {k: (v.to(DEV).to(torch.bfloat16) if k in bf else v.to(DEV)) for k, v in lw_f.items()}
    dev_cache, cpu_cache = RecurrentStateCache(cfg, 6, DEV), RecurrentStateCache(cfg, 6, "cpu")
    for lens, reset in (([5, 1, 37, 2], [1, 1, 1, 1]), ([1, 3, 1, 40], [0, 0, 0, 0]), ([2, 1, 1, 1], [1, 0, 0, 0])):
        qo = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        slots = np.asarray([4, 0, 2, 5], np.int32)
        mix = (torch.randn(int(qo[-1]), f) * 1.0).to(torch.bfloat16)
        want = ref.mamba2_mixer(mix.float(), lw_f["mamba_conv"], lw_f["mamba_conv_bias"], lw_f["mamba_A_log"],
                                lw_f["mamba_dt_bias"], lw_f["mamba_D"], lw_f["mamba_norm"], 1e-5, heads, head_dim, state,
                                groups, qo.tolist(), cpu_cache.conv_state[0], cpu_cache.rec_state[0], slots.tolist(), reset)
        got = ops.mamba2_mixer(mix.to(DEV), lw_d, cfg, dev_cache.inputs(qo, slots, np.asarray(reset, np.int32)), 0)
        torch.cuda.synchronize()
        close(got.cpu(), want, 3e-2)
        assert torch.allclose(dev_cache.rec_state.cpu(), cpu_cache.rec_state, atol=2e-2, rtol=2e-2)
        assert torch.allclose(dev_cache.conv_state.cpu(), cpu_cache.conv_state, atol=1e-6)
