"""Gated DeltaNet hybrid family (linear-attention layers with a recurrent-state cache between full-attention
layers): the cached, chunked, batched path against an independent dense oracle; recurrent-state slots through
the runtime (fork copies, eviction and truncation replay the lineage). CPU driver; the CUDA kernels have their
own test in test_kernels_gpu.py."""
import json

import numpy as np
import pytest
import torch

from pie_b200.driver.executor import TorchDriver
from pie_b200.driver.schema import ForwardRequest, SamplerKind, SamplerSpec
from pie_b200.inferlets import install_all
from pie_b200.models.config import preset
from pie_b200.models.transformer import dense_reference_forward
from pie_b200.models.weights import random_weights
from pie_b200.runtime.engine import Engine, EngineConfig
from pie_b200.runtime.rs_cache import RsState
from pie_b200.runtime.tokenizer import ByteTokenizer


def model(seed=3):
    cfg = preset("tiny-qwen3.5")
    cfg.dtype = "float32"
    return cfg, random_weights(cfg, "cpu", torch.float32, seed=seed)


def oracle_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(dense_reference_forward(cfg, w, torch.tensor(toks))[-1].argmax()))
    return toks[len(prompt):]


def test_driver_matches_dense_oracle_over_chunks_batches_and_slots():
    cfg, w = model()
    drv = TorchDriver(cfg, "cpu", weights=w, num_pages=32, page_size=16, max_requests=4, max_tokens=128)
    assert drv.capabilities().rs_cache_slots >= 4 and not drv.use_graphs
    i32 = lambda *a: np.asarray(a, dtype=np.int32)
    raw = SamplerSpec(SamplerKind.RAW_LOGITS)
    a = list(range(50, 71))
    b = list(range(900, 907))
    wa = dense_reference_forward(cfg, w, torch.tensor(a)).numpy()
    wb = dense_reference_forward(cfg, w, torch.tensor(b)).numpy()

    def fire(parts):
        """parts: [(tokens, start, page ids, slot, reset)] -> last-row logits of every request"""
        toks, pos, qo, pages, pptr, last, rows = [], [], [0], [], [0], [], []
        for tk, start, pg, _, _ in parts:
            toks += tk
            pos += list(range(start, start + len(tk)))
            qo.append(qo[-1] + len(tk))
            kv = start + len(tk)
            pages += pg[:-(-kv // 16)]
            pptr.append(len(pages))
            last.append((kv - 1) % 16 + 1)
            rows.append(qo[-1] - 1)
        req = ForwardRequest(tokens=i32(*toks), positions=i32(*pos), qo_indptr=i32(*qo), kv_page_indices=i32(*pages),
                             kv_page_indptr=i32(*pptr), kv_last_page_lens=i32(*last), slot_req=i32(*range(len(parts))),
                             slot_row=i32(*rows), slot_samplers=[raw] * len(parts),
                             rs_slots=i32(*[p[3] for p in parts]), rs_reset=i32(*[p[4] for p in parts]))
        return [np.frombuffer(s.logits, dtype=np.float32) for s in drv.fire_batch(req).slots]
    pa, pb = [0, 1], [5]
    # two requests prefilled in one fire, different lengths, different slots
    la, lb = fire([(a[:9], 0, pa, 2, 1), (b[:4], 0, pb, 0, 1)])
    assert np.abs(la - wa[8]).max() < 1e-4 and np.abs(lb - wb[3]).max() < 1e-4
    # second chunk of one, single decode token of the other (shorter than the convolution's reach)
    la, lb = fire([(a[9:20], 9, pa, 2, 0), (b[4:5], 4, pb, 0, 0)])
    assert np.abs(la - wa[19]).max() < 1e-4 and np.abs(lb - wb[4]).max() < 1e-4
    la, lb = fire([(a[20:], 20, pa, 2, 0), (b[5:7], 5, pb, 0, 0)])
    assert np.abs(la - wa[20]).max() < 1e-4 and np.abs(lb - wb[6]).max() < 1e-4
    # a slot copy carries the state: continue `b` from a copy of its slot
    drv.copy_rs(0, 3)
    (lc,) = fire([([42], 7, pb, 3, 0)])
    wc = dense_reference_forward(cfg, w, torch.tensor(b + [42])).numpy()[-1]
    assert np.abs(lc - wc).max() < 1e-4
    # reset really starts over: the same slot reused for a new sequence
    (ld,) = fire([(a[:5], 0, [7], 2, 1)])
    assert np.abs(ld - wa[4]).max() < 1e-4
    with pytest.raises(ValueError, match="recurrent-state slot"):
        drv.fire_batch(ForwardRequest(tokens=i32(1), positions=i32(0), qo_indptr=i32(0, 1), kv_page_indices=i32(0),
                                      kv_page_indptr=i32(0, 1), kv_last_page_lens=i32(1), slot_req=i32(0),
                                      slot_row=i32(0), slot_samplers=[raw]))


@pytest.fixture()
def eng():
    cfg, w = model()
    drv = TorchDriver(cfg, "cpu", weights=w, num_pages=64, page_size=16, max_requests=8, max_tokens=64, rs_slots=3)
    e = Engine(EngineConfig())
    e.add_model("hybrid", drv, tokenizer=ByteTokenizer(cfg.vocab_size))
    install_all(e)
    yield e, cfg, w
    e.shutdown()


def test_engine_generates_the_oracle_tokens_with_chunked_prefill(eng):
    e, cfg, w = eng
    prompt = list(range(100, 190))                       # 90 tokens > max_tokens 64: two prefill chunks
    out = json.loads(e.run("text-completion", {"prompt_tokens": prompt, "max_tokens": 6, "temperature": 0.0,
                                               "stop_tokens": []}, 300))
    assert out["tokens"] == oracle_greedy(cfg, w, prompt, 6)
    entry = e.models["hybrid"]
    assert entry.inference.cohorts == [] and entry.schedulers[0].stats["chunked_requests"] >= 1
    assert entry.ctxm.rs[0].slot_of == {} and len(entry.ctxm.rs[0].free) == 3        # the slot went back


def test_fork_copies_the_state_and_lost_state_is_replayed(eng):
    e, cfg, w = eng
    from pie_b200.sdk import Context, Model, Sampler
    prompt = list(range(300, 321))

    async def prog(args):
        m = Model.load("hybrid")
        ctx = Context(m)
        ctx.append(prompt)
        first = await ctx.generate(Sampler.argmax(), max_tokens=3).stop([]).collect_tokens()
        child = ctx.fork()
        a = await child.generate(Sampler.argmax(), max_tokens=3).stop([]).collect_tokens()
        b = await ctx.generate(Sampler.argmax(), max_tokens=3).stop([]).collect_tokens()
        # lose the parent's recurrent state: the next pass must rebuild it from the lineage
        cm = ctx._entry.ctxm
        cm.rs[0].invalidate(ctx.id)
        c = await ctx.generate(Sampler.argmax(), max_tokens=2).stop([]).collect_tokens()
        replayed = cm.counters["replayed_tokens"]
        # roll two tokens back: a recurrent state cannot be rolled back either
        ctx.truncate(2)
        state_after_truncate = cm.rs[0].state_of(ctx.id).name
        ctx._buffer[:] = [(first + b + c)[5]]          # KV now ends after 5 generated tokens: feed the 6th again
        d = await ctx.generate(Sampler.argmax(), max_tokens=2).stop([]).collect_tokens()
        child.release()
        ctx.release()
        return json.dumps({"first": first, "a": a, "b": b, "c": c, "d": d, "replayed": replayed,
                           "state": state_after_truncate})
    e.register_program("t", prog)
    r = json.loads(e.run("t", {}, 300))
    want = oracle_greedy(cfg, w, prompt, 8)
    assert r["first"] == want[:3] and r["a"] == want[3:6] and r["b"] == want[3:6]      # fork and parent agree
    assert r["c"] == want[6:8] and r["replayed"] >= len(prompt) + 5
    assert r["state"] == RsState.MISSING.name and r["d"] == want[6:8]
    rec = e.models["hybrid"].ctxm.rs[0]
    assert rec.slot_of == {} and len(rec.free) == 3


def test_more_contexts_than_slots_take_turns(eng):
    """Three slots, five concurrent generations: a context that loses its slot replays when it runs again."""
    e, cfg, w = eng
    prompts = [list(range(400 + 10 * i, 400 + 10 * i + 12)) for i in range(5)]
    pids = [e.launch("text-completion", {"prompt_tokens": p, "max_tokens": 5, "temperature": 0.0, "stop_tokens": [],
                                         "per_step": True}) for p in prompts]
    outs = [json.loads(e.wait(p, 300))["tokens"] for p in pids]
    assert outs == [oracle_greedy(cfg, w, p, 5) for p in prompts]


def test_checkpoint_round_trip_through_hugging_face_names(tmp_path):
    """Export under the checkpoint's names (projections grouped by key head, conv1d [C, 1, K]) and load back:
    the runtime layout is restored and the loaded model gives the oracle's logits."""
    from pie_b200.models import loader
    cfg, w = model(seed=9)
    loader.export_hf_checkpoint(cfg, w, tmp_path)
    from safetensors import safe_open
    with safe_open(str(tmp_path / "model.safetensors"), "pt") as f:
        names = set(f.keys())
        assert "model.layers.0.linear_attn.in_proj_qkvz.weight" in names
        assert list(f.get_tensor("model.layers.0.linear_attn.conv1d.weight").shape) == [cfg.gdn_conv_channels, 1, 4]
        assert "model.layers.3.self_attn.q_proj.weight" in names and "model.layers.3.linear_attn.A_log" not in names
    cfg2, w2 = loader.load_checkpoint(tmp_path, "cpu", dtype="float32")
    assert cfg2.model_type == "qwen3_5" and cfg2.linear_layers == [0, 1, 2] and cfg2.linear_num_value_heads == 4
    for key in ("w_gdn_in", "gdn_conv", "gdn_A_log", "gdn_dt_bias", "gdn_norm", "w_gdn_out", "w_gate_up"):
        assert torch.equal(w2["layers"][1][key], w["layers"][1][key]), key
    toks = torch.arange(7, 30)
    assert torch.allclose(dense_reference_forward(cfg2, w2, toks), dense_reference_forward(cfg, w, toks), atol=1e-5)
