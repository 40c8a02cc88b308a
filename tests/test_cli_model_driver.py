"""`pie model list | download | remove` against a local stand-in for the model hub, and the
`pie driver` subcommand tree with its persisted knobs (server/src/cli/model_cmd.rs, driver_cmd.rs)."""
import http.server
import json
import threading

import pytest

from pie_b200.server import cli, config as cfgmod, hf

FILES = {"config.json": json.dumps({"model_type": "llama", "hidden_size": 8}).encode(),
         "tokenizer.json": b"{}", "model-00001-of-00001.safetensors": b"\x00" * 4096,
         "model.safetensors.index.json": b"{}", "pytorch_model.bin": b"\x01" * 100, "README.md": b"hi"}


class _Hub(http.server.BaseHTTPRequestHandler):
    def log_message(self, *a):
        pass

    def do_GET(self):
        if self.path == "/api/models/acme/tiny/revision/main":
            body = json.dumps({"sha": "abc123", "siblings": [{"rfilename": n} for n in FILES]}).encode()
        elif self.path.startswith("/acme/tiny/resolve/abc123/") and self.path.rsplit("/", 1)[1] in FILES:
            body = FILES[self.path.rsplit("/", 1)[1]]
        else:
            self.send_error(404)
            return
        self.send_response(200)
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        self.wfile.write(body)


@pytest.fixture
def hub(monkeypatch, tmp_path):
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), _Hub)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    monkeypatch.setenv("HF_ENDPOINT", f"http://127.0.0.1:{srv.server_address[1]}")
    monkeypatch.setenv("HF_HUB_CACHE", str(tmp_path / "hub"))
    monkeypatch.delenv("HF_TOKEN", raising=False)
    yield tmp_path / "hub"
    srv.shutdown()


def test_model_download_list_remove(hub, capsys):
    assert cli.main(["model", "download", "acme/tiny"]) == 0
    snap = hub / "models--acme--tiny" / "snapshots" / "abc123"
    got = sorted(p.name for p in snap.iterdir())
    assert got == ["config.json", "model-00001-of-00001.safetensors", "model.safetensors.index.json", "tokenizer.json"]
    assert (hub / "models--acme--tiny" / "refs" / "main").read_text() == "abc123"
    assert hf.resolve_model("acme/tiny") == snap
    assert hf.list_cached() == [("acme/tiny", True, "llama", sum(len(FILES[n]) for n in got) + len("abc123"))]
    cli.main(["model", "list"])
    assert "acme/tiny" in capsys.readouterr().out
    assert cli.main(["model", "download", "acme/tiny", "--all"]) == 0          # adds the rest, keeps complete files
    assert (snap / "pytorch_model.bin").is_file() and (snap / "README.md").is_file()
    assert cli.main(["model", "remove", "acme/tiny", "--yes"]) == 0
    assert hf.list_cached() == []
    with pytest.raises(FileNotFoundError):
        hf.remove("acme/tiny")


def test_unsupported_architecture_is_flagged(hub):
    d = hub / "models--acme--odd" / "snapshots" / "r1"
    d.mkdir(parents=True)
    (d / "config.json").write_text(json.dumps({"model_type": "mamba"}))
    assert hf.list_cached()[0][1:3] == (False, "unsupported type: mamba")


def test_driver_knobs_persist_and_become_defaults(monkeypatch, tmp_path, capsys):
    monkeypatch.setenv("PIE_B200_CONFIG", str(tmp_path / "config.toml"))
    assert cli.main(["driver", "list"]) == 0
    assert "cuda_native" in capsys.readouterr().out
    assert cli.main(["driver", "cuda-native", "set", "kv_page_size", "32"]) == 0
    assert cli.main(["driver", "cuda-native", "set", "memory_profile", "throughput"]) == 0
    assert cli.main(["driver", "cuda-native", "show"]) == 0
    out = capsys.readouterr().out
    assert "kv_page_size" in out and "drivers.toml" in out
    with pytest.raises(SystemExit):
        cli.main(["driver", "cuda-native", "set", "no_such_knob", "1"])
    (tmp_path / "config.toml").write_text('[[model]]\nname = "m"\npreset = "tiny-llama"\n\n'
                                          '[[model]]\nname = "n"\npreset = "tiny-llama"\n[model.driver]\ntype = "cpu"\nkv_page_size = 48\n')
    cfg = cfgmod.load()
    assert cfg.model[0].driver.kv_page_size == 32 and cfg.model[0].driver.memory_profile == "throughput"
    assert cfg.model[1].driver.kv_page_size == 48 and cfg.model[1].driver.memory_profile == ""
    assert cli.main(["driver", "cuda-native", "unset", "kv_page_size"]) == 0
    assert cfgmod.load().model[0].driver.kv_page_size == 16
    assert cli.main(["driver", "list"]) == 0
    assert "used by: m" in capsys.readouterr().out
    assert cli.main(["driver", "cuda-native", "install"]) == 0
    assert "pie_b200._build" in capsys.readouterr().out


def test_new_build_publish_and_fetch_round_trip(tmp_path, monkeypatch, capsys):
    """`pie new` -> `pie build` (package zip) -> `pie publish` to a registry -> an engine fetches it on first launch."""
    import json as _json
    from pie_b200.driver.mock import CounterBehavior, MockDriver
    from pie_b200.runtime.engine import Engine, EngineConfig
    from pie_b200.runtime.program import ProgramStore
    store = {}

    class Registry(http.server.BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_PUT(self):
            store[self.path] = (self.rfile.read(int(self.headers["Content-Length"])), self.headers.get("X-Content-Hash"))
            self.send_response(201)
            self.send_header("Content-Length", "0")
            self.end_headers()

        def do_GET(self):
            key = self.path[:-len("/download")]
            if key.endswith("/latest"):
                key = sorted(k for k in store if k.startswith(key[:-len("latest")]))[-1] if store else key
            if key not in store:
                self.send_error(404)
                return
            blob, h = store[key]
            self.send_response(200)
            self.send_header("Content-Length", str(len(blob)))
            self.send_header("X-Content-Hash", h)
            self.end_headers()
            self.wfile.write(blob)
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), Registry)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    url = f"http://127.0.0.1:{srv.server_address[1]}"
    monkeypatch.chdir(tmp_path)
    assert cli.main(["new", "my-bot"]) == 0
    (tmp_path / "my-bot" / "main.py").write_text("async def main(args):\n    return 'bot:' + str(args.get('q'))\n")
    assert cli.main(["build", "my-bot"]) == 0
    assert (tmp_path / "my-bot" / "dist" / "my-bot-0.1.0.zip").exists() and "content hash" in capsys.readouterr().out
    (tmp_path / "broken").mkdir()
    (tmp_path / "broken" / "main.py").write_text("def main(x):\n    return 1\n")
    (tmp_path / "broken" / "Pie.toml").write_text('[package]\nname = "broken"\nversion = "0.1.0"\n')
    with pytest.raises(SystemExit, match="async def main"):
        cli.main(["build", "broken"])
    assert cli.main(["publish", "my-bot", "--registry", url]) == 0
    assert list(store) == ["/api/v1/inferlets/my-bot/0.1.0"]
    eng = Engine(EngineConfig())
    eng.add_model("mock", MockDriver(CounterBehavior(), total_pages=16))
    try:
        eng.program_resolver = ProgramStore(eng, str(tmp_path / "cache"), url).ensure
        assert eng.run("my-bot", {"q": 3}, 30) == "bot:3"
    finally:
        eng.shutdown()
        srv.shutdown()
