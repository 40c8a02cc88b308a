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
    srv = PieServer(eng, "127.0.0.1", 0, auth, str(tmp_path / "programs"))
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
    toml = (f'[runtime]\nprogram_dir = "{tmp_path}/programs"\n[telemetry]\nenabled = true\n[auth]\nenabled = false\n'
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
