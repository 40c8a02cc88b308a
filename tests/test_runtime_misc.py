"""Small runtime components: sandbox policies, program manager, telemetry, recurrent-state slot
pool, memory planner, parity harness, model path resolution."""
import json
import os

import numpy as np
import pytest

from pie_b200.runtime.policy import FsPolicy, NetworkPolicy, PolicyError
from pie_b200.runtime.program import Manifest, ProgramError, ProgramStore, content_hash
from pie_b200.runtime.rs_cache import RS_FLAG_RESET, RsCache, RsState
from pie_b200.runtime.telemetry import Telemetry


def test_fs_policy_scratch_and_escape(tmp_path):
    pol = FsPolicy("scratch", str(tmp_path))
    s = pol.make_scratch("proc-1")
    assert os.path.isdir(s)
    assert FsPolicy.resolve(s, "a/b.txt").startswith(s)
    with pytest.raises(PolicyError):
        FsPolicy.resolve(s, "../other")
    with pytest.raises(PolicyError):
        FsPolicy.resolve(None, "x")
    FsPolicy.drop_scratch(s)
    assert not os.path.exists(s)
    assert FsPolicy("none").make_scratch("p") is None


def test_network_policy_cidr_and_ports():
    pol = NetworkPolicy(["10.0.0.0/8", "192.168.1.5:443", "[2001:db8::]/32:8080"])
    assert pol.check("10.1.2.3", 80) == ("10.1.2.3", 80)
    assert pol.check("192.168.1.5", 443)
    with pytest.raises(PolicyError):
        pol.check("192.168.1.5", 80)
    with pytest.raises(PolicyError):
        pol.check("8.8.8.8", 53)
    assert pol.check("2001:db8::1", 8080)
    with pytest.raises(PolicyError):
        NetworkPolicy([]).check("127.0.0.1", 1)
    assert NetworkPolicy.allow_all().check("127.0.0.1", 1)


MANIFEST = '''
[package]
name = "echo-upper"
version = "1.2.0"
description = "upper-cases its input"

[parameters]
text = { type = "string", default = "hi" }
times = { type = "int", default = 1 }
'''
SOURCE = '''
async def main(args):
    return (args["text"].upper() + " ") * args["times"]
'''


def test_program_store_install_resolve_and_run(tmp_path):
    from pie_b200.runtime.engine import Engine, EngineConfig
    eng = Engine(EngineConfig())
    try:
        store = ProgramStore(eng, str(tmp_path))
        m = Manifest.parse(MANIFEST)
        h = store.install(SOURCE, m)
        assert h == content_hash(SOURCE.encode())
        with pytest.raises(ProgramError):
            store.install(SOURCE, m, expected_hash="00")
        assert eng.run("echo-upper", {"times": "2"}, timeout=30) == "HI HI "
        assert eng.run("echo-upper@1.2.0", {"text": "a"}, timeout=30) == "A "
        m2 = Manifest.parse(MANIFEST.replace("1.2.0", "1.10.0"))
        store.install(SOURCE.replace(".upper()", ".lower()"), m2)
        assert store.latest("echo-upper") == "1.10.0"
        assert store.resolve("echo-upper", "^1.2.0").version == "1.10.0"
        assert store.resolve("echo-upper", "2.0.0") is None
        assert eng.run("echo-upper", {"text": "ABC"}, timeout=30) == "abc "
        # a fresh store finds both versions in the disk cache
        eng2 = Engine(EngineConfig())
        try:
            assert ProgramStore(eng2, str(tmp_path)).load_cache() == ["echo-upper@1.2.0", "echo-upper@1.10.0"]
            assert eng2.run("echo-upper", {"text": "Q"}, timeout=30) == "q "
        finally:
            eng2.shutdown()
        dep = Manifest.parse('[package]\nname = "needs"\nversion = "0.1.0"\n[dependencies]\nmissing = "1.0.0"\n')
        with pytest.raises(ProgramError):
            store.install(SOURCE, dep)
    finally:
        eng.shutdown()


def test_manifest_validation():
    with pytest.raises(ProgramError):
        Manifest.parse('[package]\nname = "Bad Name"\nversion = "1.0.0"\n')
    with pytest.raises(ProgramError):
        Manifest.parse('[package]\nname = "ok"\nversion = "one"\n')
    with pytest.raises(ProgramError):
        Manifest.parse('[package]\nname = "ok"\nversion = "1.0.0"\n[surprise]\nx = 1\n')
    m = Manifest.parse(MANIFEST)
    assert Manifest.parse(m.to_toml()).parameters == m.parameters
    with pytest.raises(ProgramError):
        m.check_input({"times": "many"})


def test_telemetry_prometheus_and_spans(tmp_path):
    path = tmp_path / "spans.jsonl"
    t = Telemetry("pie", True, str(path))
    t.incr("fires")
    t.incr("fires", 2)
    t.gauge("kv_pages_used", 12)
    with t.probe("fold"):
        pass
    t.record_probe_us("driver_forward", 1500)
    with t.span("fire_batch", requests=3):
        pass
    with pytest.raises(ValueError):
        with t.span("bad"):
            raise ValueError("x")
    text = t.prometheus()
    assert "pie_fires_total 3" in text and "pie_kv_pages_used 12" in text and "pie_probe_fold_seconds_count 1" in text
    snap = t.snapshot()
    assert abs(snap["probes"]["driver_forward"]["mean_us"] - 1500) < 1e-6
    t.close()
    spans = [json.loads(l) for l in path.read_text().splitlines()]
    assert [s["name"] for s in spans] == ["fire_batch", "bad"]
    assert spans[0]["status"]["code"] == "OK" and spans[1]["status"]["code"] == "ERROR"
    off = Telemetry(enabled=False)
    off.incr("x")
    assert off.prometheus() == "\n"


def test_rs_cache_states():
    assert RsCache(0).state_of(1) == RsState.UNSUPPORTED
    c = RsCache(2)
    assert c.acquire(7) == 0 and c.state_of(7) == RsState.EMPTY
    assert c.flags_for_pass(7) == RS_FLAG_RESET and c.state_of(7) == RsState.RESIDENT
    assert c.flags_for_pass(7) == 0
    assert c.fork(7, 8) == (0, 1) and c.state_of(8) == RsState.RESIDENT
    assert c.acquire(9) is None                     # pool exhausted
    c.invalidate(8)
    assert c.flags_for_pass(8) == RS_FLAG_RESET
    c.release(7)
    assert c.state_of(7) == RsState.MISSING and c.acquire(9) == 0
    c.forget(7)
    assert c.state_of(7) == RsState.EMPTY


def test_memory_planner_profiles():
    from pie_b200.driver.memory_planner import kv_bytes_per_page, plan
    from pie_b200.models.config import preset
    cfg = preset("llama-3.1-8b")
    assert kv_bytes_per_page(cfg, 16) == 32 * 2 * 8 * 16 * 128 * 2
    free = 160 << 30
    auto = plan(cfg, free)
    assert auto.profile == "throughput" and auto.kv_pages * 16 >= 512 * 2048
    lat = plan(cfg, free, profile="latency")
    assert lat.max_requests == 64 and lat.kv_pages > auto.kv_pages * 0.9
    small = plan(cfg, 24 << 30)
    assert small.profile in ("balanced", "capacity") and small.kv_bytes + small.arena_bytes <= 0.9 * (24 << 30)
    tp8 = plan(cfg, free, tp=8)
    assert tp8.kv_pages > 7 * auto.kv_pages
    with pytest.raises(ValueError):
        plan(cfg, free, profile="nope")


def test_parity_harness_prefill_vs_decode_after_prefill():
    from pie_b200 import parity
    toks = list(range(5, 40))
    a = parity.run("tiny-llama", toks)
    b = parity.run("tiny-llama", toks, decode_after_prefill=True)
    rep = parity.compare(a, b)
    assert rep["cos"] > 0.9999 and rep["argmax_equal"]


def test_hf_resolve(tmp_path, monkeypatch):
    from pie_b200.server.hf import resolve_model
    snap = tmp_path / "hub" / "models--org--tiny" / "snapshots" / "abc123"
    snap.mkdir(parents=True)
    refs = tmp_path / "hub" / "models--org--tiny" / "refs"
    refs.mkdir()
    (refs / "main").write_text("abc123")
    monkeypatch.setenv("HF_HOME", str(tmp_path))
    monkeypatch.delenv("HF_HUB_CACHE", raising=False)
    assert resolve_model("org/tiny") == snap
    assert resolve_model("org/tiny@main") == snap
    assert resolve_model(str(tmp_path)) == tmp_path
    with pytest.raises(FileNotFoundError):
        resolve_model("org/absent")


def test_harmony_and_kimi_chat_templates():
    from pie_b200.runtime import instruct as I
    g = I.for_arch("gpt_oss")
    text = g.format("system", "Be brief", True) + g.format("system", "Use tools", False) + g.format("user", "hi", False) + g.cue_text()
    assert text == ("<|start|>system<|message|>Be brief<|end|><|start|>developer<|message|>Use tools<|end|>"
                    "<|start|>user<|message|>hi<|end|><|start|>assistant")
    assert g.format("assistant", "ok", False) == "<|start|>assistant<|channel|>final<|message|>ok<|end|>"
    assert set(g.stop_strings) == {"<|return|>", "<|call|>"} and g.seal_text() == "<|return|>"
    decl = g.equip([{"name": "get_weather", "description": "weather", "parameters": {"type": "object"}}])
    assert "type get_weather = (_: {\"type\": \"object\"}) => any;" in decl and "namespace functions" in decl
    assert g.answer("get_weather", "{}").startswith("<|start|>functions.get_weather to=assistant")
    k = I.for_arch("kimi")
    assert k.format("user", "hi", False) + k.cue_text() == "<|im_user|>user<|im_middle|>hi<|im_end|><|im_assistant|>assistant<|im_middle|>"


def test_attention_plans_on_the_host():
    """Decode work items cover each request's visible key range exactly once in 16-token aligned
    chunks (also under a sliding window); prefill tiles come out heaviest first."""
    import numpy as np
    from pie_b200 import ops
    kv = np.array([1, 15, 16, 17, 300, 1000, 2305, 64])
    for window in (-1, 0, 100):
        req, st, en, iptr = ops.plan_decode_items(kv, 8, target_ctas=64, min_chunk=256, window_left=window)
        assert iptr[0] == 0 and iptr[-1] == len(req)
        for r, kl in enumerate(kv):
            a, b = iptr[r], iptr[r + 1]
            assert b > a and (req[a:b] == r).all()
            lo = 0 if window < 0 else max(0, kl - 1 - window) // 16 * 16
            assert st[a] == lo and en[b - 1] == kl and (st[a:b] % 16 == 0).all()
            assert (st[a + 1:b] == en[a:b - 1]).all()        # contiguous, no overlap
    # a cap on the number of items coarsens the chunks instead of dropping work
    req, st, en, iptr = ops.plan_decode_items(kv, 8, target_ctas=4096, max_items=10, min_chunk=16)
    assert len(req) <= 10 and en[iptr[1:] - 1].tolist() == kv.tolist()
    qo = np.array([0, 5, 300, 1000])
    lens = np.array([45, 295, 2000])
    tr, tq = ops.plan_prefill_tiles(qo, 4, 256, lens)
    work = [lens[r] - (qo[r + 1] - qo[r]) + min(q + 64, qo[r + 1] - qo[r]) for r, q in zip(tr, tq)]
    assert work == sorted(work, reverse=True) and len(tr) == 1 + 5 + 11
    tr0, tq0 = ops.plan_prefill_tiles(qo, 4, 256)
    assert sorted(zip(tr.tolist(), tq.tolist())) == sorted(zip(tr0.tolist(), tq0.tolist()))


def test_reasoning_decoder_splits_harmony_channels():
    from pie_b200.runtime import instruct as I
    g = I.for_arch("gpt_oss")
    stream = ("<|channel|>analysis<|message|>think hard<|end|><|start|>assistant<|channel|>final<|message|>"
              "The answer is 4.<|return|>")
    for step in (1, 3, 7, len(stream)):
        dec = I.ReasoningDecoder(g)
        ev = []
        for i in range(0, len(stream), step):
            ev += dec.feed(stream[i:i + step])
        ev += dec.flush()
        think = "".join(e.text for e in ev if e.kind == "thinking")
        answer = "".join(e.text for e in ev if e.kind == "delta")
        assert think == "think hard" and answer == "The answer is 4.", (step, think, answer)
        assert sum(e.kind == "thinking_done" for e in ev) == 1
    # the plain <think> family is unchanged
    dec = I.ReasoningDecoder(I.for_arch("qwen3"))
    ev = dec.feed("<think>a</think>b") + dec.flush()
    got = [(e.kind, e.text) for e in ev if e.text or e.kind == "thinking_done"]
    assert got == [("thinking", "a"), ("thinking_done", ""), ("delta", "b")]


def test_precapture_is_a_no_op_without_cuda_graphs():
    import torch
    from pie_b200.driver.executor import TorchDriver, graph_buckets
    from pie_b200.models.config import preset
    drv = TorchDriver(preset("tiny-llama"), "cpu", num_pages=8, page_size=16, max_requests=4, max_tokens=64)
    assert drv.precapture_graphs() == 0 and not drv.graphs
    b = graph_buckets(512)
    assert b[:5] == [1, 2, 4, 8, 16] and b[-1] == 512 and b == sorted(set(b)) and 64 in b and 256 in b


def test_driver_config_carries_the_memory_profile():
    """`[model.driver] memory_profile` reaches the driver, which then takes its forward limits from
    the planner (on a CPU driver the page count is fixed, the limits still follow the profile's)."""
    from pie_b200.server import config as cfgmod
    cfg = cfgmod.parse('[[model]]\nname = "m"\npreset = "tiny-llama"\n[model.driver]\ntype = "cpu"\nmemory_profile = "latency"\n')
    assert cfg.model[0].driver.memory_profile == "latency"
    from pie_b200.driver.memory_planner import PROFILES, arena_bytes, plan
    from pie_b200.models.config import preset
    c = preset("llama-3.1-8b")
    p = plan(c, 100 << 30, 1.0, "latency")
    assert (p.max_requests, p.max_tokens) == (PROFILES["latency"]["max_requests"], PROFILES["latency"]["max_tokens"])
    assert p.kv_bytes + p.arena_bytes <= (100 << 30) and p.arena_bytes == arena_bytes(c, p.max_tokens, p.max_requests)


def test_determinism_ledger_cases_repeat_and_match_when_asked():
    """Greedy output is repeatable run to run; with PIE_CHECK_LEDGER=1 it must also equal the
    committed ledger (exact-token regression guard for refactors on the reference machine)."""
    import json
    import os
    from pie_b200.bench import determinism
    name, prog, args = determinism.CASES[0]
    h1, h2 = determinism.run_case(name, prog, args), determinism.run_case(name, prog, args)
    assert h1 == h2 and len(h1) == 64
    ledger = json.loads(determinism.LEDGER.read_text())
    assert set(ledger["cases"]) == {f"{n}/{p}" for n, p, _ in determinism.CASES}
    if os.environ.get("PIE_CHECK_LEDGER") == "1":
        assert ledger["cases"][f"{name}/{prog}"] == h1


def test_ragged_brle_expansion_on_the_cpu_path():
    """Rows of different lengths expand back to back, each to ceil(bits / 32) words, with zeros past the last run."""
    import numpy as np
    from pie_b200 import ops
    from pie_b200.runtime import brle
    rows, bits = [[3, 2, 1], [0, 40], [10], [0, 5, 2, 7], []], [6, 40, 10, 70, 33]
    words, offs = ops.brle_expand_ragged(rows, bits, "cpu")
    assert offs.tolist() == [0, 1, 3, 4, 7, 9] and words.numel() == 9
    for i, (r, n) in enumerate(zip(rows, bits)):
        got = np.unpackbits(words[offs[i]:offs[i + 1]].numpy().view(np.uint8), bitorder="little")[:n].astype(bool)
        assert np.array_equal(got, brle.decode(r, n)), i
    empty, offs0 = ops.brle_expand_ragged([], [], "cpu")
    assert empty.numel() == 0 and offs0.tolist() == [0]
