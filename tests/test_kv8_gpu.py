"""fp8 (e4m3) KV pages with per-(token, head) scales: the writer, the page expander, decode attention
that reads the fp8 pages directly, and the driver end to end against a bf16-KV driver."""
import math

import numpy as np
import pytest
import torch

from pie_b200 import ops
from pie_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def bf(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).to(DEV)


def write_both(n_tokens, hq, hkv, d, page, seed):
    """The same tokens written into a bf16 layer and an fp8 layer (+ scales). Returns both and the slots."""
    pages = -(-n_tokens // page) + 2
    qkv = bf(n_tokens, (hq + 2 * hkv) * d, seed=seed, scale=2.0)
    qkv[:, hq * d: hq * d + 8] *= 30.0                       # a few outliers per K row: the scale must follow them
    pos = torch.arange(n_tokens, dtype=torch.int32, device=DEV)
    perm = torch.randperm(pages * page, generator=torch.Generator().manual_seed(seed))[:n_tokens]
    slots = perm.to(torch.int32).to(DEV)
    inv = ref.rope_inv_freq(d, 10000.0, None, DEV)
    kv16 = torch.zeros(pages + 1, 2, hkv, page, d, dtype=torch.bfloat16, device=DEV)
    kv8 = torch.zeros(pages + 1, 2, hkv, page, d, dtype=torch.uint8, device=DEV)
    sc = torch.zeros(pages + 1, 2, hkv, page, dtype=torch.float32, device=DEV)
    q16 = ops.qk_norm_rope_kvwrite(qkv, pos, slots, inv, None, None, kv16, hq, hkv, d, page, 1e-6)
    q8 = ops.qk_norm_rope_kvwrite(qkv, pos, slots, inv, None, None, kv8, hq, hkv, d, page, 1e-6, kv_scale=sc)
    assert torch.equal(q16, q8)
    return kv16, kv8, sc, slots, pages


@pytest.mark.parametrize("d,hq,hkv", [(128, 8, 2), (64, 4, 4)])
def test_fp8_kv_write_and_expand(d, hq, hkv):
    page = 16
    kv16, kv8, sc, slots, pages = write_both(75, hq, hkv, d, page, seed=1)
    all_pages = torch.arange(pages, dtype=torch.int32, device=DEV)
    dense = ops.dequant_kv_pages(kv8, sc, all_pages)
    assert dense.shape[0] == pages + 1 and float(dense[pages].abs().max()) == 0.0
    want, got = kv16[:pages].float(), dense[:pages].float()
    written = (sc[:pages] > 0)[..., None].expand_as(want)
    assert bool((got[~written] == 0).all())
    # e4m3 keeps 3 mantissa bits: relative error 2^-4 of the value, absolute floor one step of the row's smallest bucket
    row_max = want.abs().amax(-1, keepdim=True)
    err = (got - want).abs()
    assert bool((err <= 0.0626 * want.abs() + row_max / 448.0 * 0.002 + 1e-3)[written].all())
    # scales: max|x| / 448 per written row
    rows = sc[:pages] > 0
    assert torch.allclose(sc[:pages][rows], row_max.squeeze(-1)[rows] / 448.0, rtol=2e-2)


@pytest.mark.parametrize("d,hq,hkv", [(128, 32, 8), (128, 4, 1), (64, 16, 2), (128, 16, 16)])
@pytest.mark.parametrize("window", [-1, 70])
def test_fp8_kv_decode_attention(d, hq, hkv, window):
    page = 16
    kv_lens = np.array([1, 15, 16, 17, 300, 1000, 2305, 64], dtype=np.int32)
    r = len(kv_lens)
    npages = [-(-int(k) // page) for k in kv_lens]
    total = sum(npages) + 3
    g = torch.Generator().manual_seed(5)
    kvf = torch.randn(total, 2, hkv, page, d, generator=g) * 1.5
    kvf[:, 0, :, :, :4] *= 8.0                               # outlier channels in K
    amax = kvf.abs().amax(-1)
    sc = (amax / 448.0).clamp_min(1e-12).to(DEV)
    kv8 = (kvf.to(DEV) / sc[..., None]).to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
    kv8 = torch.cat([kv8, torch.zeros_like(kv8[:1])])        # the pad page
    sc = torch.cat([sc, torch.zeros_like(sc[:1])]).contiguous()
    pages = torch.randperm(total, generator=g)[:sum(npages)].numpy().astype(np.int32)
    indptr = np.zeros(r + 1, dtype=np.int32)
    indptr[1:] = np.cumsum(npages)
    q = bf(r, hq, d, seed=6)
    item_req, st, en, iptr = ops.plan_decode_items(kv_lens, hkv, target_ctas=64, min_chunk=256, window_left=window)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)
    max_items = len(item_req) + 3
    plan = ops.DecodePlan(t(pages), t(indptr), t(item_req), t(st), t(en), t(iptr),
                          torch.tensor([len(item_req)], dtype=torch.int32, device=DEV),
                          torch.empty(ops.decode_scratch_floats(max_items, hq, d), device=DEV),
                          max_items, r, 64, page, window_left=window)
    scale = 1 / math.sqrt(d)
    status = ops.kernel_status(DEV)
    status.zero_()
    out = ops.paged_decode_attention(q, kv8, plan, scale, kv_scale=sc)
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0
    # oracle: fp32 attention over the dequantised pages (the kernel's only extra rounding is P to f16)
    dense = ops.dequant_kv_pages(kv8, sc, torch.arange(total, dtype=torch.int32, device=DEV), pad_zero_page=False)
    exact = kv8[:total].view(torch.float8_e4m3fn).float() * sc[:total, ..., None]
    assert float((dense.float() - exact).abs().max()) <= 0.004 * float(exact.abs().max())     # bf16 rounding only
    qo = np.arange(r + 1, dtype=np.int32)
    want = ref.paged_attention(q, exact, qo, indptr, torch.from_numpy(pages).to(DEV), kv_lens, scale, window_left=window)
    assert float((out.float() - want.float()).abs().max()) <= 2e-2 * max(1.0, float(want.abs().max()))


def test_driver_with_fp8_kv_tracks_the_bf16_driver():
    from pie_b200.driver.executor import TorchDriver
    from pie_b200.driver.schema import SamplerKind, SamplerSpec
    from pie_b200.models.config import preset
    from pie_b200.models.weights import random_weights
    from pie_b200.runtime.scheduler import PendingRequest, fold
    cfg = preset("tiny-llama", hidden_size=512, intermediate_size=1408, num_attention_heads=8, num_key_value_heads=2,
                 head_dim=128, vocab_size=4096, num_hidden_layers=3, dtype="bfloat16")
    w = random_weights(cfg, "cuda", torch.bfloat16, seed=2, std=0.05)
    raw = SamplerSpec(SamplerKind.RAW_LOGITS)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, cfg.vocab_size, n).tolist() for n in (37, 150, 5)]
    pages, nxt = [], 0
    for p in prompts:
        k = -(-(len(p) + 8) // 16)
        pages.append(list(range(nxt, nxt + k)))
        nxt += k
    outs = {}
    for kvd in ("auto", "fp8_e4m3"):
        drv = TorchDriver(cfg, "cuda", weights=w, num_pages=64, page_size=16, max_requests=8, max_tokens=512, kv_dtype=kvd)
        assert (drv.kv.scale is not None) == (kvd == "fp8_e4m3")
        if kvd == "fp8_e4m3":
            assert drv.kv.data.dtype == torch.uint8 and not drv.cascade
        r1 = drv.fire_batch(fold([PendingRequest(i, p, list(range(len(p))), pg, 0, [(len(p) - 1, raw)])
                                  for i, (p, pg) in enumerate(zip(prompts, pages))], 16))
        toks = [int(np.frombuffer(s.logits, dtype=np.float32).argmax()) for s in r1.slots] if kvd == "auto" else outs["toks"]
        outs["toks"] = toks
        logits = [[np.frombuffer(s.logits, dtype=np.float32).copy() for s in r1.slots]]
        for step in range(2):
            r2 = drv.fire_batch(fold([PendingRequest(i, [t], [len(p) + step], pg, len(p) + step, [(0, raw)])
                                      for i, (t, p, pg) in enumerate(zip(toks, prompts, pages))], 16))
            logits.append([np.frombuffer(s.logits, dtype=np.float32).copy() for s in r2.slots])
        ops.check_kernel_status(drv.device)
        assert drv.stats["graph_replays"] == 2
        outs[kvd] = logits
    for a, b in zip(outs["auto"], outs["fp8_e4m3"]):
        for x, y in zip(a, b):
            cos = float(np.dot(x, y) / (np.linalg.norm(x) * np.linalg.norm(y)))
            assert cos > 0.995, cos
            assert int(y.argmax()) in np.argsort(x)[-3:]
