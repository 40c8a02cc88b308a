"""Mixture-of-experts kernels on the GPU: router top-k, alignment to 128-row tiles, grouped
tcgen05 GEMMs and the weighted combine, against a dense fp32 PyTorch evaluation."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(x, router, wgu, wd, k, renorm, residual):
    xf = x.float()
    probs = torch.softmax(xf @ router.float().t(), -1)
    w, ids = torch.topk(probs, k, -1)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    out = residual.float().clone()
    for e in range(wgu.shape[0]):
        sel = ids == e
        tok = sel.any(-1).nonzero()[:, 0]
        if tok.numel() == 0:
            continue
        gu = xf[tok] @ wgu[e].float().t()
        act = (torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]).to(torch.bfloat16).float()
        y = (act @ wd[e].float().t()).to(torch.bfloat16).float()
        out[tok] += y * (w[tok] * sel[tok]).sum(-1, keepdim=True)
    return out, ids, w


@pytest.mark.parametrize("n,h,inter,e,k", [(1, 256, 128, 8, 2), (37, 256, 128, 8, 2), (512, 2048, 768, 128, 8),
                                           (300, 2048, 768, 16, 8), (2048, 1024, 384, 64, 4)])
def test_moe_experts_matches_reference(n, h, inter, e, k):
    from pie_b200 import ops
    torch.manual_seed(n + e)
    dev = torch.device("cuda")
    x = (torch.randn(n, h, device=dev) * 0.5).to(torch.bfloat16)
    res = (torch.randn(n, h, device=dev) * 0.5).to(torch.bfloat16)
    router = (torch.randn(e, h, device=dev) * 0.05).to(torch.bfloat16)
    wgu = (torch.randn(e, 2 * inter, h, device=dev) * 0.03).to(torch.bfloat16)
    wd = (torch.randn(e, h, inter, device=dev) * 0.03).to(torch.bfloat16)
    logits = (x.float() @ router.float().t())            # fp32 logits: no bf16 ties in the top-k
    buf = ops.MoeBuffers(n, h, inter, e, k, dev)
    for _ in range(2):                                   # twice: the counters must come back to zero
        got = ops.moe_experts(x, logits, wgu, wd, k, True, buf, residual=res)
    torch.cuda.synchronize()
    ops.check_kernel_status(dev)
    want, ids, w = _reference(x, router, wgu, wd, k, True, res)
    assert torch.equal(torch.sort(buf.ids[:n].long(), -1).values, torch.sort(ids, -1).values)
    torch.testing.assert_close(torch.sort(buf.w[:n], -1).values, torch.sort(w, -1).values, rtol=1e-4, atol=1e-6)
    assert int(buf.counts.sum()) == 0 and int(buf.counts_out.sum()) == n * k
    err = (got.float() - want).abs().max().item()
    assert err < 0.06, err
    cos = torch.nn.functional.cosine_similarity(got.float().flatten(), want.flatten(), dim=0).item()
    assert cos > 0.9995, cos


def test_moe_block_in_cuda_graph_and_model():
    """tiny Qwen3-MoE through the driver: prefill + decode tokens equal the dense fp32 oracle's."""
    import numpy as np
    from pie_b200.driver.executor import TorchDriver
    from pie_b200.models.config import preset
    from pie_b200.models.transformer import dense_reference_forward
    from pie_b200.models.weights import random_weights
    from pie_b200.bench import harness
    from pie_b200.driver.schema import SamplerKind, SamplerSpec
    cfg = preset("tiny-qwen3-moe")
    dev = torch.device("cuda", 0)
    w = random_weights(cfg, dev, torch.bfloat16, seed=0)
    drv = TorchDriver(cfg, dev, weights=w, num_pages=256, page_size=16, max_requests=8, max_tokens=512)
    prompts = [np.random.default_rng(i).integers(0, cfg.vocab_size, 20 + 7 * i).tolist() for i in range(4)]
    sampler = SamplerSpec(SamplerKind.MULTINOMIAL, temperature=0.0)
    pages, first, _ = harness.prefill_contexts(drv, prompts, 8, sampler)

    def to_cpu(x):
        if torch.is_tensor(x):
            return x.float().cpu()
        if isinstance(x, dict):
            return {k_: to_cpu(v) for k_, v in x.items()}
        if isinstance(x, list):
            return [to_cpu(v) for v in x]
        return x

    wf = to_cpu(w)
    for i, p in enumerate(prompts):
        logits = dense_reference_forward(cfg, wf, torch.tensor(p))
        top2 = torch.topk(logits[-1].float(), 2).values
        if (top2[0] - top2[1]) > 0.05:                   # only compare when the oracle is not at a near tie
            assert int(first[i]) == int(torch.argmax(logits[-1])), i
