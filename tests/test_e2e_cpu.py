"""Config-1 plumbing run: tiny Llama (2 layers, hidden 256, 4q/2kv heads, d 64, FFN 688,
vocab 32000, fp32, N(0,0.02) weights from seed 0), one 32-token random prompt (seed 1),
page size 16, greedy decode of 64 tokens through the whole engine (inferlet -> SDK ->
inference service -> scheduler -> driver -> paged kernels' CPU path), checked
token-for-token against an independent dense fp32 forward."""
import json

import numpy as np
import pytest
import torch

from pie_b200.driver.executor import TorchDriver
from pie_b200.inferlets import install_all
from pie_b200.models.config import preset
from pie_b200.models.transformer import dense_reference_forward
from pie_b200.models.weights import random_weights
from pie_b200.runtime.engine import Engine, EngineConfig


def oracle_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    out = []
    for _ in range(n):
        logits = dense_reference_forward(cfg, w, torch.tensor(toks))
        t = int(torch.argmax(logits[-1]))
        out.append(t)
        toks.append(t)
    return out


def make_engine(policy="adaptive", depth=1, num_pages=64):
    cfg = preset("tiny-llama")
    w = random_weights(cfg, "cpu", torch.float32, seed=0)
    drv = TorchDriver(cfg, device="cpu", weights=w, num_pages=num_pages, page_size=16, max_requests=16,
                      max_tokens=256)
    eng = Engine(EngineConfig(batch_policy=policy, speculation_depth=depth))
    eng.add_model("tiny-llama", drv)
    install_all(eng)
    return eng, cfg, w


def test_text_completion_matches_dense_oracle():
    eng, cfg, w = make_engine()
    try:
        prompt = np.random.default_rng(1).integers(0, cfg.vocab_size, 32).tolist()
        res = eng.run("text-completion", {"prompt_tokens": prompt, "max_tokens": 64, "stop_tokens": []}, timeout=300)
        got = json.loads(res)["tokens"]
        want = oracle_greedy(cfg, w, prompt, 64)
        assert got == want
        st = eng.model_status()["models"]["tiny-llama"]
        assert st["kv_pages_used"] == 0       # everything released with the process
        assert eng.model("tiny-llama").schedulers[0].stats.get("decode_steps", 0) >= 63   # ran in the cohort
    finally:
        eng.shutdown()


def test_per_step_inferlet_claims_staged_passes():
    eng, cfg, w = make_engine()
    try:
        prompt = np.random.default_rng(1).integers(0, cfg.vocab_size, 32).tolist()
        res = eng.run("text-completion", {"prompt_tokens": prompt, "max_tokens": 24, "stop_tokens": [],
                                          "per_step": True}, timeout=300)
        assert json.loads(res)["tokens"] == oracle_greedy(cfg, w, prompt, 24)
        st = eng.model_status()["models"]["tiny-llama"]
        assert st["bypass_hits"] > 0          # the staged (speculative) passes were claimed
        assert st["kv_pages_used"] == 0
    finally:
        eng.shutdown()


def test_no_speculation_same_tokens():
    eng, cfg, w = make_engine(policy="greedy", depth=0)
    try:
        prompt = np.random.default_rng(1).integers(0, cfg.vocab_size, 32).tolist()
        res = eng.run("text-completion", {"prompt_tokens": prompt, "max_tokens": 16, "stop_tokens": [],
                                          "per_step": True}, timeout=300)
        assert json.loads(res)["tokens"] == oracle_greedy(cfg, w, prompt, 16)
    finally:
        eng.shutdown()


def test_concurrent_inferlets_batch_together():
    eng, cfg, w = make_engine()
    try:
        rng = np.random.default_rng(3)
        prompts = [rng.integers(0, cfg.vocab_size, int(n)).tolist() for n in (5, 17, 32, 40)]
        procs = [eng.launch("text-completion", {"prompt_tokens": p, "max_tokens": 12, "stop_tokens": []}) for p in prompts]
        outs = [json.loads(eng.wait(p, 300))["tokens"] for p in procs]
        for p, o in zip(prompts, outs):
            assert o == oracle_greedy(cfg, w, p, 12)
        st = eng.model_status()["models"]["tiny-llama"]
        assert st["total_requests"] > st["total_batches"]   # batches held more than one request
    finally:
        eng.shutdown()


def test_moe_model_matches_dense_oracle():
    """Qwen3-MoE style model (8 experts, top-2, qk-norm) through the engine on CPU."""
    cfg = preset("tiny-qwen3-moe")
    w = random_weights(cfg, "cpu", torch.float32, seed=0)
    drv = TorchDriver(cfg, device="cpu", weights=w, num_pages=64, page_size=16, max_requests=16, max_tokens=256)
    eng = Engine(EngineConfig())
    eng.add_model(cfg.name, drv)
    install_all(eng)
    try:
        prompt = np.random.default_rng(2).integers(0, cfg.vocab_size, 24).tolist()
        res = eng.run("text-completion", {"prompt_tokens": prompt, "max_tokens": 12, "stop_tokens": []}, timeout=300)
        assert json.loads(res)["tokens"] == oracle_greedy(cfg, w, prompt, 12)
    finally:
        eng.shutdown()


def test_seeded_sampling_same_stream_on_both_scheduler_paths():
    """A request that fixes its sampler seed gets the same tokens whether the runtime's cohort steps
    it or the inferlet drives one forward per token: both derive the per-draw seed from
    (seed, position of the sampled row)."""
    eng, cfg, w = make_engine()
    try:
        prompt = np.random.default_rng(5).integers(0, cfg.vocab_size, 20).tolist()
        args = {"prompt_tokens": prompt, "max_tokens": 12, "stop_tokens": [], "temperature": 1.0, "top_p": 0.95,
                "seed": 1234}
        a = json.loads(eng.run("text-completion", dict(args), timeout=300))["tokens"]
        b = json.loads(eng.run("text-completion", dict(args, per_step=True), timeout=300))["tokens"]
        c = json.loads(eng.run("text-completion", dict(args, seed=99), timeout=300))["tokens"]
        assert a == b and len(a) == 12
        assert a != c                      # and the seed matters
        assert len(set(a)) > 1             # the noise differs from step to step
    finally:
        eng.shutdown()


def test_samplers_on_one_row_share_one_logit_row():
    """Compact logit rows: several probes of the same token row cost one row of the vocabulary projection."""
    from pie_b200.driver.executor import TorchDriver
    from pie_b200.driver.schema import ForwardRequest, SamplerKind, SamplerSpec
    from pie_b200.models.config import preset
    drv = TorchDriver(preset("tiny-llama", num_hidden_layers=1), device="cpu", num_pages=8)
    i32 = lambda *a: np.asarray(a, dtype=np.int32)

    def fire(rows, samplers):
        return drv.fire_batch(ForwardRequest(
            tokens=i32(1, 2, 3, 4), positions=i32(0, 1, 2, 3), qo_indptr=i32(0, 4), kv_page_indices=i32(0),
            kv_page_indptr=i32(0, 1), kv_last_page_lens=i32(4), slot_req=i32(*([0] * len(rows))), slot_row=i32(*rows),
            slot_samplers=samplers))
    before = drv.stats.get("logit_rows", 0)
    r = fire([3, 1, 3, 3], [SamplerSpec.greedy(), SamplerSpec.greedy(), SamplerSpec(SamplerKind.DIST, top_k=3),
                            SamplerSpec(SamplerKind.ENTROPY)])
    assert drv.stats["logit_rows"] - before == 2                    # rows {1, 3}
    a = fire([3], [SamplerSpec.greedy()]).slots[0].token
    b = fire([1], [SamplerSpec.greedy()]).slots[0].token
    assert [r.slots[0].token, r.slots[1].token] == [a, b]
    assert r.slots[2].ids[0] == a and r.slots[3].kind == "entropy"


def test_bounds_check_mode_names_the_bad_table_and_entry(monkeypatch):
    """`PIE_BOUNDS=1`: a fire whose index tables point outside their ranges fails before any kernel runs."""
    from pie_b200.driver.executor import TorchDriver
    from pie_b200.driver.schema import ForwardRequest, SamplerSpec
    from pie_b200.models.config import preset
    monkeypatch.setenv("PIE_BOUNDS", "1")
    drv = TorchDriver(preset("tiny-llama", num_hidden_layers=1), device="cpu", num_pages=8)
    assert drv.bounds_check
    i32 = lambda *a: np.asarray(a, dtype=np.int32)

    def req(**kw):
        base = dict(tokens=i32(1, 2, 3), positions=i32(0, 1, 2), qo_indptr=i32(0, 3), kv_page_indices=i32(2),
                    kv_page_indptr=i32(0, 1), kv_last_page_lens=i32(3), slot_req=i32(0), slot_row=i32(2),
                    slot_samplers=[SamplerSpec()])
        base.update(kw)
        return ForwardRequest(**base)
    assert drv.fire_batch(req()).slots[0].kind == "token"
    with pytest.raises(IndexError, match=r"kv_page_indices\[0\] = 8"):
        drv.fire_batch(req(kv_page_indices=i32(8)))                  # pages 0..7 exist
    with pytest.raises(IndexError, match=r"tokens\[1\]"):
        drv.fire_batch(req(tokens=i32(1, 1 << 20, 3)))
    with pytest.raises(IndexError, match=r"logit_rows\[0\] = 3"):
        drv.fire_batch(req(slot_row=i32(3)))
    assert drv.fire_batch(req()).slots[0].kind == "token"           # the driver is still usable


def test_system_speculation_gives_the_same_greedy_tokens_in_fewer_passes():
    """Runtime-side prompt-look-up drafting: a repetitive context lets the runtime propose the continuation,
    verify it in one pass and hand several tokens to the generator step; the output is the plain greedy output."""
    cfg = preset("tiny-llama")
    w = random_weights(cfg, "cpu", torch.float32, seed=0)
    prompt = [11, 12, 13, 14, 15, 16] * 6

    def run(k):
        drv = TorchDriver(cfg, device="cpu", weights=w, num_pages=64, page_size=16, max_requests=8, max_tokens=256)
        eng = Engine(EngineConfig(system_spec_tokens=k))
        eng.add_model("m", drv)
        install_all(eng)
        try:
            out = json.loads(eng.run("text-completion-bench", {"prompt_tokens": prompt, "max_tokens": 24, "per_step": True,
                                                               "temperature": 0.0}, 300))
            st = dict(eng.models["m"].inference.stats)
            fires = drv.stats["fires"]
            eng.models["m"].ctxm.audit()
        finally:
            eng.shutdown()
        return out, st, fires
    base, st0, fires0 = run(0)
    spec, st4, fires4 = run(4)
    assert st0["system_spec_proposed"] == 0 and st4["system_spec_proposed"] > 0
    assert spec["n_tokens"] == base["n_tokens"] == 24
    # token-level equality through the text-completion inferlet (it returns the tokens)
    def toks(k):
        drv = TorchDriver(cfg, device="cpu", weights=w, num_pages=64, page_size=16, max_requests=8, max_tokens=256)
        eng = Engine(EngineConfig(system_spec_tokens=k))
        eng.add_model("m", drv)
        install_all(eng)
        try:
            return json.loads(eng.run("text-completion", {"prompt_tokens": prompt, "max_tokens": 24, "temperature": 0.0,
                                                          "stop_tokens": [], "per_step": True}, 300))["tokens"]
        finally:
            eng.shutdown()
    assert toks(4) == toks(0)
    if st4["system_spec_accepted"] > 0:
        assert fires4 < fires0                     # accepted drafts save forward passes


def test_probe_slots_of_every_kind_in_one_fire_are_batched_correctly():
    """Two distributions with different temperatures and widths, two label sets of different sizes, raw logits and an
    entropy in one fire: each slot's payload equals the plain computation on its own row."""
    import numpy as np
    import torch
    from pie_b200.driver.executor import TorchDriver
    from pie_b200.driver.schema import SamplerKind, SamplerSpec
    from pie_b200.models.config import preset
    from pie_b200.models.transformer import dense_reference_forward
    from pie_b200.models.weights import random_weights
    from pie_b200.runtime.scheduler import PendingRequest, fold
    cfg = preset("tiny-llama")
    w = random_weights(cfg, "cpu", torch.float32, seed=1)
    drv = TorchDriver(cfg, "cpu", weights=w, num_pages=16, page_size=16, max_requests=4, max_tokens=64)
    toks = list(range(10, 30))
    specs = [(3, SamplerSpec(SamplerKind.DIST, temperature=0.7, top_k=5)), (19, SamplerSpec(SamplerKind.DIST, temperature=0.0, top_k=0)),
             (7, SamplerSpec(SamplerKind.LOGPROBS, labels=(1, 2, 3))), (19, SamplerSpec(SamplerKind.LOGPROBS, labels=(31999,))),
             (12, SamplerSpec(SamplerKind.RAW_LOGITS)), (19, SamplerSpec(SamplerKind.ENTROPY)), (3, SamplerSpec(SamplerKind.ENTROPY))]
    resp = drv.fire_batch(fold([PendingRequest(0, toks, list(range(20)), [0, 1], 0, specs)], 16))
    want = dense_reference_forward(cfg, w, torch.tensor(toks))
    s = resp.slots
    p = torch.softmax(want[3] / 0.7, -1)
    pv, pi = torch.topk(p, 5)
    assert s[0].ids == pi.tolist() and np.allclose(s[0].probs, pv.numpy(), atol=1e-5)
    pv, pi = torch.topk(torch.softmax(want[19], -1), 32)
    assert s[1].ids == pi.tolist() and np.allclose(s[1].probs, pv.numpy(), atol=1e-5)
    assert np.allclose(s[2].logprobs, torch.log_softmax(want[7], -1)[[1, 2, 3]].numpy(), atol=1e-4)
    assert np.allclose(s[3].logprobs, torch.log_softmax(want[19], -1)[[31999]].numpy(), atol=1e-4)
    assert np.allclose(np.frombuffer(s[4].logits, dtype=np.float32), want[12].numpy(), atol=1e-4)
    ent = lambda r: float(-(torch.softmax(r, -1) * torch.log_softmax(r, -1)).sum())
    assert abs(s[5].entropy - ent(want[19])) < 1e-3 and abs(s[6].entropy - ent(want[3])) < 1e-3
