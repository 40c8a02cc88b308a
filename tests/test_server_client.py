"""Server, client, CLI, config, auth, workflows, daemon over the dummy / mock drivers (CPU)."""
import json
import tempfile
import time
import urllib.request

import pytest

from pie_b200.client.client import ClientError, PieClient
from pie_b200.driver.mock import CounterBehavior, MockDriver
from pie_b200.inferlets import install_all
from pie_b200.runtime.engine import Engine, EngineConfig
from pie_b200.server import config as cfgmod
from pie_b200.server.auth import Authenticator, UserStore, generate_ed25519
from pie_b200.server.server import PieServer


@pytest.fixture()
def stack(tmp_path):
    eng = Engine(EngineConfig(watchdog_interval_s=0.1))
    eng.add_model("mock", MockDriver(CounterBehavior(), total_pages=256))
    install_all(eng)
    users = UserStore(str(tmp_path / "users.json"))
    key, pub = generate_ed25519()
    users.add("alice", pub)
    auth = Authenticator(True, users)
    srv = PieServer(eng, "127.0.0.1", 0, auth, str(tmp_path / "programs"), allow_program_upload=True)
    srv.bad_token_delay_scale = 0.01
    port = srv.start()
    yield eng, srv, auth, key, f"ws://127.0.0.1:{port}"
    srv.stop()
    eng.shutdown()


def test_auth_launch_events_query(stack):
    eng, srv, auth, key, uri = stack
    c = PieClient(uri)
    assert c.ping() == "pong"
    with pytest.raises(ClientError):
        c.query("model_status")                       # not authenticated yet
    with pytest.raises(ClientError):
        c.auth_by_token("wrong")
    c.auth_with_key("alice", key)
    p = c.launch_process("text-completion", {"prompt_tokens": [5, 6], "max_tokens": 4, "stop_tokens": []})
    assert json.loads(p.wait(30))["tokens"] == [7, 8, 9, 10]
    st = c.model_status()
    assert st["models"]["mock"]["kv_pages_used"] == 0 and st["models"]["mock"]["total_batches"] > 0
    assert "text-completion" in c.query("programs")
    c.close()
    c2 = PieClient(uri)
    c2.auth_by_token(auth.internal_token)
    res = c2.run_processes("text-completion", [{"prompt_tokens": [i], "max_tokens": 2, "stop_tokens": []} for i in range(3)])
    assert [json.loads(r["value"])["tokens"] for r in res] == [[1, 2], [2, 3], [3, 4]]
    c2.close()


PROGRAM = b'''
from pie_b200.sdk import runtime, session, messaging

async def main(args):
    runtime.print_out("hello ", args["who"])
    session.send("ready")
    msg = await session.receive()
    data = await session.receive_file()
    messaging.push("q", msg)
    got = await messaging.pull("q")
    return got + ":" + str(len(data))
'''


def test_upload_program_signal_file_and_disk_cache(stack, tmp_path):
    eng, srv, auth, key, uri = stack
    c = PieClient(uri)
    c.auth_by_token(auth.internal_token)
    name = c.install_program(PROGRAM, '[package]\nname = "echo-test"\nversion = "0.2.0"\n')
    assert name == "echo-test" and c.program_exists("echo-test")
    p = c.launch_process("echo-test", {"who": "world"})
    seen = []
    while True:
        ev, val = p.recv(10)
        seen.append((ev, val))
        if ev == "message" and val == "ready":
            p.signal("ping")
            p.transfer_file(b"x" * 300000)            # two chunks
        if ev in ("return", "error"):
            break
    assert ("stdout", "hello  world") in seen or ("stdout", "hello world") in seen
    assert seen[-1] == ("return", "ping:300000")
    assert (tmp_path / "programs" / "echo-test" / "0.2.0.py").exists()
    c.close()


def test_upload_refused_unless_enabled(tmp_path):
    """Uploaded programs are unsandboxed Python: a server accepts them only with allow_program_upload."""
    eng = Engine(EngineConfig(watchdog_interval_s=0.1))
    eng.add_model("mock", MockDriver(CounterBehavior(), total_pages=64))
    install_all(eng)
    # a program cached by an earlier (opted-in) run must not be executed by a server that did not opt in
    cached = tmp_path / "programs" / "evil"
    cached.mkdir(parents=True)
    marker = tmp_path / "ran"
    (cached / "0.1.0.py").write_text(f"open({str(marker)!r}, 'w').write('x')\nasync def main(a):\n    return 1\n")
    (cached / "0.1.0.toml").write_text('[package]\nname = "evil"\nversion = "0.1.0"\n')
    srv = PieServer(eng, "127.0.0.1", 0, Authenticator(False), str(tmp_path / "programs"))
    port = srv.start()
    try:
        assert not marker.exists() and "evil" not in eng.programs
        c = PieClient(f"ws://127.0.0.1:{port}")
        with pytest.raises(ClientError, match="uploads disabled"):
            c.install_program(PROGRAM, '[package]\nname = "echo-test"\nversion = "0.2.0"\n')
        assert not c.program_exists("echo-test")
        c.close()
    finally:
        srv.stop()
        eng.shutdown()


def test_workflow_and_daemon(stack):
    eng, srv, auth, key, uri = stack
    c = PieClient(uri)
    c.auth_by_token(auth.internal_token)
    tc = lambda toks, n: {"op": "process", "program": "text-completion",
                          "input": {"prompt_tokens": toks, "max_tokens": n, "stop_tokens": []}}
    spec = {"op": "pipe", "steps": [
        {"op": "fork", "branches": [tc([1], 2), tc([10], 2)]},
        {"op": "map", "over": "$prev", "body": {"op": "value", "value": "$item.tokens"}},
        {"op": "fold", "over": "$prev", "init": 0, "body": {"op": "value", "value": {"len": "$item"}}},
        {"op": "cond", "if": {"eq": ["$prev", 2]}, "then": {"op": "value", "value": "two"},
         "else": {"op": "value", "value": "other"}}]}
    assert c.submit_workflow(spec).wait(30) == "two"
    port = c.launch_daemon("text-completion", 0, {"prompt_tokens": [3], "max_tokens": 2, "stop_tokens": []})
    body = urllib.request.urlopen(f"http://127.0.0.1:{port}/anything", timeout=10).read()
    assert json.loads(body)["tokens"] == [4, 5]
    c.close()


def test_config_parse_validate_topology(tmp_path):
    text = '''
[server]
port = 9001
[auth]
enabled = false
[[model]]
name = "a"
preset = "llama-3.1-8b"
[model.driver]
device = [0, 1, 2, 3]
tensor_parallel_size = 2
[[model]]
name = "b"
preset = "tiny-llama"
[model.driver]
type = "dummy"
'''
    cfg = cfgmod.parse(text)
    assert cfg.server.port == 9001 and not cfg.auth.enabled and len(cfg.model) == 2
    assert cfgmod.calculate_topology([0, 1, 2, 3], 2) == [[0, 1], [2, 3]]
    assert cfgmod.parse(cfgmod.dumps(cfg)).model[0].driver.tensor_parallel_size == 2      # round trip
    for bad in ("[server]\nbogus = 1\n", "[nope]\n", text.replace("device = [0, 1, 2, 3]", "device = [0, 1, 2]"),
                text + "[model.driver]\n", '[[model]]\nname="x"\npreset="tiny-llama"\n[model.driver]\nmax_num_seqs = 4\n'):
        with pytest.raises((cfgmod.ConfigError, Exception)):
            cfgmod.parse(bad)
    with pytest.raises(cfgmod.ConfigError):
        cfgmod.parse(text.replace('type = "dummy"', 'device = [3]'))       # device 3 claimed twice
    cfgmod.set_key(cfg, "model.1.driver.kv_page_size", "32")
    assert cfg.model[1].driver.kv_page_size == 32
    # KV page format and media encoders are driver keys
    fp8 = cfgmod.parse(text.replace("tensor_parallel_size = 2", 'tensor_parallel_size = 2\nkv_dtype = "fp8_e4m3"\nvision = "tiny-vit"'))
    assert fp8.model[0].driver.kv_dtype == "fp8_e4m3" and fp8.model[0].driver.vision == "tiny-vit" and fp8.model[1].driver.kv_dtype == "auto"
    with pytest.raises(cfgmod.ConfigError, match="kv_dtype"):
        cfgmod.parse(text.replace("tensor_parallel_size = 2", 'tensor_parallel_size = 2\nkv_dtype = "int4"'))
    with pytest.raises(cfgmod.ConfigError, match="cuda_native"):
        cfgmod.parse(text.replace('type = "dummy"', 'type = "dummy"\nkv_dtype = "fp8_e4m3"'))


def test_cli_smoke_run_and_monitor(capsys):
    from pie_b200.server import cli
    from pie_b200.server.monitor import run_monitor
    assert cli.main(["smoke"]) == 0
    assert '"tokens"' in capsys.readouterr().out
    assert cli._trailing_to_json(["--prompt", "hi", "--max_tokens", "4", "--flag"]) == {"prompt": "hi", "max_tokens": 4, "flag": True}
    eng = Engine(EngineConfig())
    eng.add_model("mock", MockDriver())
    import io
    buf = io.StringIO()
    run_monitor(eng, period=0.01, out=buf, iterations=2)
    assert "kv 0/" in buf.getvalue()
    eng.shutdown()


def test_embedded_server_and_client_cli(tmp_path, capsys):
    from pie_b200.client import cli as client_cli
    from pie_b200.server.embed import Server
    toml = (f'[server]\nallow_program_upload = true\n[runtime]\nprogram_dir = "{tmp_path}/programs"\n'
            f'[telemetry]\nenabled = true\n[auth]\nenabled = false\n'
            '[[model]]\nname = "dummy"\npreset = "tiny-llama"\n[model.driver]\ntype = "dummy"\n')
    with Server.from_text(toml) as srv:
        uri = srv.uri
        assert client_cli.main(["--uri", uri, "ping"]) == 0
        assert client_cli.main(["--uri", uri, "submit", "helloworld"]) == 0
        out = capsys.readouterr().out
        assert "Hello, world!" in out and "Hello from instance" in out
        src = tmp_path / "main.py"
        src.write_text("async def main(a):\n    return 'v=' + str((a or {}).get('x'))\n")
        man = tmp_path / "Pie.toml"
        man.write_text('[package]\nname = "cli-demo"\nversion = "0.1.0"\n')
        assert client_cli.main(["--uri", uri, "install", str(src), str(man)]) == 0
        assert client_cli.main(["--uri", uri, "submit", "cli-demo", "--x", "5"]) == 0
        assert "v=5" in capsys.readouterr().out
        assert client_cli.main(["--uri", uri, "status"]) == 0
        assert '"models"' in capsys.readouterr().out
        assert "pie_b200_uptime_seconds" in srv.engine.metrics_text()


def test_cli_runs_a_gguf_model_with_its_own_tokenizer(tmp_path, capsys):
    """`pie run --model-path file.gguf --driver cpu`: configuration, weights and the byte-level BPE
    tokenizer all come from the one GGUF file; text goes in, text comes out."""
    import json
    import torch
    tokenizers = pytest.importorskip("tokenizers")
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    from pie_b200.models import gguf
    from pie_b200.models.config import preset
    from pie_b200.models.weights import random_weights
    from pie_b200.server import cli

    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    tok.decoder = decoders.ByteLevel()
    tok.train_from_iterator(["the quick brown fox jumps over the lazy dog " * 4, "hello world hello pie"],
                            trainers.BpeTrainer(vocab_size=320, special_tokens=["<|eot|>"],
                                                initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    tj = json.loads(tok.to_str())
    vocab = tj["model"]["vocab"]
    tokens = [None] * len(vocab)
    for t, i in vocab.items():
        tokens[i] = t
    merges = [m if isinstance(m, str) else " ".join(m) for m in tj["model"]["merges"]]
    cfg = preset("tiny-llama", vocab_size=len(tokens), hidden_size=64, intermediate_size=128, num_attention_heads=2,
                 num_key_value_heads=1, head_dim=32, num_hidden_layers=1)
    w = random_weights(cfg, "cpu", torch.float32, seed=3, std=0.05)
    d, hq, hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    lw = w["layers"][0]
    q, k, v = lw["wqkv"].split([hq * d, hkv * d, hkv * d], 0)
    tensors = {"token_embd.weight": (w["embed"], gguf.T_F32), "output_norm.weight": (w["final_norm"], gguf.T_F32),
               "output.weight": (w["lm_head"], gguf.T_F32), "blk.0.attn_norm.weight": (lw["ln1"], gguf.T_F32),
               "blk.0.ffn_norm.weight": (lw["ln2"], gguf.T_F32),
               "blk.0.attn_q.weight": (gguf.permute_rotary(q, hq), gguf.T_F32),
               "blk.0.attn_k.weight": (gguf.permute_rotary(k, hkv), gguf.T_F32), "blk.0.attn_v.weight": (v, gguf.T_F32),
               "blk.0.attn_output.weight": (lw["wo"], gguf.T_F32), "blk.0.ffn_gate.weight": (lw["w_gate_up"][0::2], gguf.T_F32),
               "blk.0.ffn_up.weight": (lw["w_gate_up"][1::2], gguf.T_F32), "blk.0.ffn_down.weight": (lw["w_down"], gguf.T_F32)}
    meta = {"general.architecture": "llama", "general.name": "tiny-gguf", "llama.embedding_length": cfg.hidden_size,
            "llama.block_count": 1, "llama.attention.head_count": hq, "llama.attention.head_count_kv": hkv,
            "llama.feed_forward_length": cfg.intermediate_size, "llama.context_length": 512,
            "llama.attention.key_length": d, "llama.rope.freq_base": float(cfg.rope_theta),
            "llama.attention.layer_norm_rms_epsilon": float(cfg.rms_norm_eps), "tokenizer.ggml.model": "gpt2",
            "tokenizer.ggml.tokens": tokens, "tokenizer.ggml.merges": merges,
            "tokenizer.ggml.eos_token_id": vocab["<|eot|>"]}
    path = tmp_path / "tiny.gguf"
    gguf.write_gguf(path, meta, tensors)
    capsys.readouterr()
    rc = cli.main(["run", "--model-path", str(path), "--driver", "cpu", "text-completion", "--",
                   "--prompt", "hello world", "--max_tokens", "6", "--temperature", "0", "--return_tokens"])
    out = capsys.readouterr().out
    assert rc == 0, out
    res = json.loads([l for l in out.strip().splitlines() if l.startswith("{")][-1])
    assert 1 <= len(res["tokens"]) <= 6 and all(0 <= t < len(tokens) for t in res["tokens"])
    # the prompt was tokenised with the file's vocabulary: the same ids as the source tokenizer gives
    from pie_b200.runtime.tokenizer import load_gguf_tokenizer
    assert load_gguf_tokenizer(path).encode("hello world") == tok.encode("hello world").ids


def test_client_cli_config_file_and_key_auth(stack, tmp_path, capsys, monkeypatch):
    """`pie-client config init | update | show`, and a command that authenticates with the configured key."""
    from cryptography.hazmat.primitives import serialization
    from pie_b200.client import cli
    eng, srv, auth, key, uri = stack
    monkeypatch.setenv("HOME", str(tmp_path))
    conf = tmp_path / "client.toml"
    monkeypatch.setenv("PIE_B200_CLIENT_CONFIG", str(conf))
    assert cli.main(["config", "show"]) == 1
    assert cli.main(["config", "init"]) == 0
    assert cli.main(["config", "init"]) == 1                      # refuses to overwrite without --force
    assert cli.load_config()["enable_auth"] is False             # no key under ~/.ssh
    assert cli.main(["config", "update"]) == 1
    kp = tmp_path / "id_test"
    kp.write_bytes(key.private_bytes(serialization.Encoding.PEM, serialization.PrivateFormat.OpenSSH,
                                     serialization.NoEncryption()))
    kp.chmod(0o600)
    port = int(uri.rsplit(":", 1)[1])
    assert cli.main(["config", "update", "--port", str(port), "--username", "alice", "--private-key-path", str(kp),
                     "--enable-auth", "true"]) == 0
    assert cli.load_config() == {"host": "127.0.0.1", "port": port, "username": "alice", "private_key_path": str(kp),
                                 "enable_auth": True}
    capsys.readouterr()
    assert cli.main(["config", "show"]) == 0
    assert 'username = "alice"' in capsys.readouterr().out
    assert cli.main(["status"]) == 0                               # needs authentication: done with the key
    assert "mock" in capsys.readouterr().out
    assert cli.main(["submit", "text-completion", "--prompt_tokens", "[5, 6]", "--max_tokens", "3", "--stop_tokens", "[]"]) == 0
    assert json.loads(capsys.readouterr().out)["tokens"] == [7, 8, 9]
    assert cli.main(["config", "update", "--enable-auth", "false"]) == 0
    assert cli.main(["status"]) == 1                               # the server still wants authentication


def test_client_cli_interrupt_terminates_its_own_process_and_only_detaches_from_others():
    from pie_b200.client import cli as client_cli

    class Handle:
        def __init__(self):
            self.terminated = 0

        def recv(self, timeout=None):
            raise KeyboardInterrupt

        def terminate(self):
            self.terminated += 1
            return True
    own, other = Handle(), Handle()
    assert client_cli._stream(own) == 130 and own.terminated == 1
    assert client_cli._stream(other, owner=False) == 130 and other.terminated == 0
