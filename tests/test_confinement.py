"""Uploaded programs run under the audit-hook confinement (runtime/policy.py): files outside the scratch
directory, sockets outside the allow list, process spawns, ctypes and threads are refused - also when the
program bypasses the SDK and imports os / socket itself - while programs shipped with the package and the
engine's own work on an inferlet's behalf are untouched. Counterpart of the sandbox role of
runtime/src/instance.rs:89-125 (WASI preopens and socket allow lists)."""
import http.server
import json
import os
import threading

import pytest

from pie_b200.driver.mock import CounterBehavior, MockDriver
from pie_b200.inferlets import install_all
from pie_b200.runtime import policy
from pie_b200.runtime.engine import Engine, EngineConfig
from pie_b200.runtime.program import Manifest, ProgramStore


@pytest.fixture()
def eng(tmp_path):
    e = Engine(EngineConfig(scratch_root=str(tmp_path / "scratch"), network_allow=("127.0.0.1/32",)))
    e.add_model("mock", MockDriver(CounterBehavior(), total_pages=64))
    install_all(e)
    e.store = ProgramStore(e, str(tmp_path / "programs"))
    yield e
    e.shutdown()


def install(e, name, body):
    src = "import json\nfrom pie_b200.sdk import runtime, io as pio\n\nasync def main(args):\n" + "".join(
        "    " + line + "\n" for line in body.strip("\n").splitlines())
    e.store.install(src, Manifest(name=name, version="0.1.0"))
    return name


def run(e, name, args=None):
    return json.loads(e.run(name, args or {}, 30))


def test_direct_file_access_is_limited_to_the_scratch_directory(eng, tmp_path):
    secret = tmp_path / "secret.txt"
    secret.write_text("top secret")
    install(eng, "files", f'''
import os
out = {{}}
for label, fn in (("read", lambda: open({str(secret)!r}).read()),
                  ("write", lambda: open({str(tmp_path / "dropped.txt")!r}, "w").write("x")),
                  ("listdir", lambda: os.listdir({str(tmp_path)!r})),
                  ("remove", lambda: os.remove({str(secret)!r})),
                  ("os_open", lambda: os.open({str(secret)!r}, os.O_RDONLY))):
    try:
        fn()
        out[label] = "allowed"
    except PermissionError as e:
        out[label] = "denied"
d = pio.scratch_dir()
with open(os.path.join(d, "note.txt"), "w") as f:
    f.write("mine")
out["scratch"] = open(os.path.join(d, "note.txt")).read()
out["listed"] = os.listdir(d)
import colorsys                                     # importing from the standard library keeps working
out["import"] = colorsys.rgb_to_hsv(1, 0, 0)[2]
return json.dumps(out)
''')
    r = run(eng, "files")
    assert {k: r[k] for k in ("read", "write", "listdir", "remove", "os_open")} == {
        "read": "denied", "write": "denied", "listdir": "denied", "remove": "denied", "os_open": "denied"}
    assert r["scratch"] == "mine" and r["listed"] == ["note.txt"] and r["import"] == 1
    assert secret.read_text() == "top secret" and not (tmp_path / "dropped.txt").exists()
    assert ("files", "open") in policy.denied_events


def test_processes_threads_ctypes_and_foreign_sockets_are_refused(eng):
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), http.server.SimpleHTTPRequestHandler)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    port = srv.server_address[1]
    install(eng, "doors", f'''
import os, socket, subprocess, threading
out = {{}}
def attempt(label, fn):
    try:
        fn()
        out[label] = "allowed"
    except PermissionError:
        out[label] = "denied"
    except Exception as e:
        out[label] = type(e).__name__
attempt("popen", lambda: subprocess.run(["true"]))
attempt("system", lambda: os.system("true"))
attempt("thread", lambda: threading.Thread(target=lambda: None).start())
def dl():
    import ctypes
    ctypes.CDLL("libc.so.6")
attempt("ctypes", dl)
attempt("connect_allowed", lambda: socket.create_connection(("127.0.0.1", {port}), timeout=5).close())
attempt("connect_denied", lambda: socket.create_connection(("10.255.255.1", 80), timeout=0.2))
attempt("bind", lambda: socket.socket().bind(("127.0.0.1", 0)))
return json.dumps(out)
''')
    r = run(eng, "doors")
    srv.shutdown()
    assert r == {"popen": "denied", "system": "denied", "thread": "denied", "ctypes": "denied",
                 "connect_allowed": "allowed", "connect_denied": "denied", "bind": "denied"}


def test_module_body_of_an_upload_is_confined_too(eng, tmp_path):
    marker = tmp_path / "import_time.txt"
    src = f"open({str(marker)!r}, 'w').write('ran')\nasync def main(args):\n    return 'x'\n"
    with pytest.raises(PermissionError):
        eng.store.install(src, Manifest(name="evil", version="0.1.0"))
    assert not marker.exists() and "evil" not in eng.programs


def test_shipped_programs_and_engine_work_for_an_inferlet_are_not_confined(eng, tmp_path):
    # a program registered by the package itself may do what it wants
    async def trusted_main(args):
        (tmp_path / "trusted.txt").write_text("ok")
        return "done"
    eng.register_program("trusted", trusted_main)
    assert eng.run("trusted", {}, 30) == "done" and (tmp_path / "trusted.txt").read_text() == "ok"
    # an uploaded program that installs and launches a child: the store writes to its directory on its behalf
    child = "async def main(args):\\n    return 'child says hi'\\n"
    install(eng, "parent", f'''
import asyncio
from pie_b200.sdk import host
from pie_b200.runtime.program import Manifest
from pie_b200.inferlets.text_completion import main as text_completion
eng = host.engine()
eng.store.install("{child}", Manifest(name="kid", version="0.1.0"))
p = eng.launch("kid", {{}})
while not p.finished:
    await asyncio.sleep(0.01)
gen = json.loads(await text_completion({{"prompt_tokens": [1, 2, 3], "max_tokens": 4, "stop_tokens": []}}))
return json.dumps({{"kid": p.result, "generated": len(gen["tokens"])}})
''')
    r = run(eng, "parent")
    assert r == {"kid": "child says hi", "generated": 4}
    assert (tmp_path / "programs" / "kid" / "0.1.0.py").exists() and "kid" in eng.confined_programs


def test_programs_are_fetched_from_the_registry_on_first_use(tmp_path):
    """`launch` of a program that is neither registered nor cached downloads it from the registry
    (runtime/src/program/repository.rs:19-45): zip of Pie.toml + main.py, hash header checked, cached on disk,
    and the fetched program runs confined like any other upload."""
    import io
    import zipfile
    from pie_b200.runtime.program import ProgramError, content_hash
    src = "async def main(args):\n    return 'from the registry: ' + str(args.get('x'))\n"
    buf = io.BytesIO()
    with zipfile.ZipFile(buf, "w") as z:
        z.writestr("Pie.toml", '[package]\nname = "remote-hello"\nversion = "1.2.0"\n')
        z.writestr("main.py", src)
    hits = []

    class Registry(http.server.BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_GET(self):
            hits.append(self.path)
            if self.path in ("/api/v1/inferlets/remote-hello/latest/download", "/api/v1/inferlets/remote-hello/1.2.0/download"):
                self.send_response(200)
                self.send_header("Content-Length", str(len(buf.getvalue())))
                self.send_header("X-Content-Hash", "bad" if "tampered" in self.headers.get("User-Agent", "") else
                                 content_hash(src.encode()))
                self.end_headers()
                self.wfile.write(buf.getvalue())
            else:
                self.send_error(404)
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), Registry)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    e = Engine(EngineConfig())
    e.add_model("mock", MockDriver(CounterBehavior(), total_pages=64))
    try:
        store = ProgramStore(e, str(tmp_path / "programs"), f"http://127.0.0.1:{srv.server_address[1]}")
        e.program_resolver = store.ensure
        assert e.run("remote-hello", {"x": 7}, 30) == "from the registry: 7"
        assert e.run("remote-hello@1.2.0", {"x": 8}, 30) == "from the registry: 8"
        assert hits == ["/api/v1/inferlets/remote-hello/latest/download"]            # fetched once, then local
        assert (tmp_path / "programs" / "remote-hello" / "1.2.0.py").read_text() == src
        assert "remote-hello" in e.confined_programs
        with pytest.raises(ProgramError, match="404"):
            store.fetch("no-such-program")
        with pytest.raises(ProgramError, match="bad program reference"):
            store.fetch("../etc/passwd")
        with pytest.raises(ProgramError, match="registry has no"):
            e.launch("no-such-program")
    finally:
        e.shutdown()
        srv.shutdown()
