"""`pie` command line (python -m pie_b200 ...). Subcommands follow the reference CLI
(server/src/cli.rs:50-142): serve, run, config {init,show,set}, auth {add,remove,list,keygen},
model {list,download,remove}, inferlet {list}, driver {list, <type> install|doctor|show|set|unset},
new, build, publish, monitor, doctor, check, smoke.

`pie run <inferlet> [-- --key value ...]` boots a one-shot engine, connects a client over the
WebSocket like any other client, launches the inferlet with the trailing `--key value` pairs as
its JSON input, relays its output and shuts down (server/src/cli/run_cmd.rs:26-120).
"""
from __future__ import annotations

import argparse
import json
import logging
import sys
import textwrap
import time
from pathlib import Path

from . import config as cfgmod


def _trailing_to_json(rest):
    out, i = {}, 0
    while i < len(rest):
        k = rest[i]
        if not k.startswith("--"):
            raise SystemExit(f"expected --key, got {k!r}")
        v = rest[i + 1] if i + 1 < len(rest) and not rest[i + 1].startswith("--") else "true"
        i += 2 if v != "true" or (i + 1 < len(rest) and rest[i + 1] == "true") else 1
        try:
            out[k[2:].replace("-", "_")] = json.loads(v)
        except json.JSONDecodeError:
            out[k[2:].replace("-", "_")] = v
    return out


def _load(args) -> cfgmod.Config:
    if getattr(args, "config", None):
        return cfgmod.load(args.config)
    p = cfgmod.default_path()
    cfg = cfgmod.load(p) if p.exists() else cfgmod.default_config()
    if getattr(args, "driver", None):
        for m in cfg.model:
            m.driver.type = args.driver
    if getattr(args, "preset", None):
        cfg.model = [cfgmod.ModelSection(name=args.preset, preset=args.preset, driver=cfg.model[0].driver if cfg.model
                                         else cfgmod.DriverConfig())]
    if getattr(args, "model_path", None):
        cfg.model = [cfgmod.ModelSection(name=Path(args.model_path).name, path=args.model_path,
                                         driver=cfg.model[0].driver if cfg.model else cfgmod.DriverConfig())]
    for key in ("vision", "audio"):
        if getattr(args, key, None):
            for m in cfg.model:
                setattr(m.driver, key, getattr(args, key))
    cfgmod.validate(cfg)
    return cfg


def cmd_serve(args) -> int:
    from .serve import start_engine
    cfg = _load(args)
    if args.port is not None:
        cfg.server.port = args.port
    if args.no_auth:
        cfg.auth.enabled = False
    h = start_engine(cfg)
    if h is None:
        return 0
    print(f"pie_b200 serving on {h.uri}")
    if cfg.auth.enabled:
        print(f"internal token: {h.auth.internal_token}")
    if args.monitor:
        from .monitor import run_monitor
        threading = __import__("threading")
        threading.Thread(target=run_monitor, args=(h.engine,), daemon=True).start()
    h.wait_then_shutdown()
    return 0


def cmd_run(args) -> int:
    from ..client.client import PieClient
    from .serve import start_engine
    cfg = _load(args)
    cfg.server.port = 0
    h = start_engine(cfg)
    if h is None:
        return 0
    rc = 0
    try:
        c = PieClient(h.uri)
        if cfg.auth.enabled:
            c.auth_by_token(h.auth.internal_token)
        name = args.inferlet
        if Path(name).suffix == ".py" and Path(name).exists():
            src = Path(name).read_bytes()
            name = Path(name).stem.replace("_", "-")
            c.install_program(src, f'[package]\nname = "{name}"\nversion = "0.1.0"\n')
        proc = c.launch_process(name, _trailing_to_json(args.rest))
        while True:
            ev, val = proc.recv(timeout=args.timeout)
            if ev == "stdout":
                print(val, end="", flush=True)
            elif ev == "stderr":
                print(val, end="", file=sys.stderr, flush=True)
            elif ev == "message":
                print(f"[message] {val}")
            elif ev == "return":
                print(val)
                break
            elif ev == "error":
                print(f"error: {val}", file=sys.stderr)
                rc = 1
                break
        c.close()
    finally:
        h.shutdown()
    return rc


def cmd_config(args) -> int:
    p = Path(args.config).expanduser() if args.config else cfgmod.default_path()
    if args.action == "init":
        if p.exists() and not args.force:
            raise SystemExit(f"{p} exists (use --force)")
        p.parent.mkdir(parents=True, exist_ok=True)
        p.write_text(cfgmod.dumps(cfgmod.default_config()))
        print(f"wrote {p}")
    elif args.action == "show":
        print(cfgmod.dumps(cfgmod.load(p) if p.exists() else cfgmod.default_config()))
    elif args.action == "set":
        cfg = cfgmod.load(p) if p.exists() else cfgmod.default_config()
        cfgmod.set_key(cfg, args.key, args.value)
        p.parent.mkdir(parents=True, exist_ok=True)
        p.write_text(cfgmod.dumps(cfg))
        print(f"{args.key} = {args.value}")
    return 0


def cmd_auth(args) -> int:
    from .auth import UserStore, generate_ed25519
    cfg = _load(args)
    store = UserStore(cfg.auth.authorized_users)
    if args.action == "add":
        store.add(args.username, Path(args.pubkey).expanduser().read_text() if Path(args.pubkey).expanduser().exists()
                  else args.pubkey)
        print(f"added key for {args.username}")
    elif args.action == "remove":
        print("removed" if store.remove(args.username) else "no such user")
    elif args.action == "list":
        for u, ks in store.users.items():
            print(f"{u}: {len(ks)} key(s)")
    elif args.action == "keygen":
        from cryptography.hazmat.primitives import serialization
        k, pub = generate_ed25519()
        out = Path(args.pubkey or "pie_ed25519").expanduser()
        out.write_bytes(k.private_bytes(serialization.Encoding.PEM, serialization.PrivateFormat.OpenSSH,
                                        serialization.NoEncryption()))
        out.with_suffix(".pub").write_text(pub + "\n")
        print(f"wrote {out} and {out.with_suffix('.pub')}")
    return 0


def _human(n: int) -> str:
    for unit in ("B", "KiB", "MiB", "GiB", "TiB"):
        if n < 1024 or unit == "TiB":
            return f"{n:.1f} {unit}" if unit != "B" else f"{n} B"
        n /= 1024.0


def cmd_model(args) -> int:
    """`pie model list | download <org/name> [--revision R] [--all] | remove <org/name> [--yes]`
    (server/src/cli/model_cmd.rs:20-254)."""
    from ..models.config import PRESETS
    from . import hf
    if args.action == "download":
        if not args.repo:
            raise SystemExit("usage: pie model download <org/name>")
        snap = hf.download(args.repo, args.revision, args.all, progress=hf.progress_bar())
        print(f"{args.repo} -> {snap}")
        return 0
    if args.action == "remove":
        if not args.repo:
            raise SystemExit("usage: pie model remove <org/name>")
        if not args.yes and input(f"remove {args.repo} from {hf.hf_cache_root()}? [y/N] ").strip().lower() != "y":
            return 1
        print(f"freed {_human(hf.remove(args.repo))}")
        return 0
    cached = hf.list_cached()
    if cached:
        print(f"cached under {hf.hf_cache_root()}:")
        for repo, ok, why, size in cached:
            print(f"  {'ok ' if ok else '-- '} {repo:44s} {why:28s} {_human(size):>10s}")
    print("presets (random-init, for benchmarks and tests):")
    for name, kw in PRESETS.items():
        print(f"  {name:18s} {kw['model_type']:10s} layers={kw['num_hidden_layers']:3d} hidden={kw['hidden_size']:5d} "
              f"heads={kw['num_attention_heads']}/{kw['num_key_value_heads']} vocab={kw['vocab_size']}")
    return 0


def cmd_inferlet(args) -> int:
    import importlib
    import pkgutil
    from .. import inferlets
    for m in pkgutil.iter_modules(inferlets.__path__):
        mod = importlib.import_module(f"pie_b200.inferlets.{m.name}")
        if hasattr(mod, "main"):
            doc = (mod.__doc__ or "").strip().splitlines()
            print(f"{getattr(mod, 'NAME', m.name.replace('_', '-')):28s} {doc[0] if doc else ''}")
    return 0


DRIVER_TYPES = {
    "cuda_native": "B200 driver: tcgen05 / TMA kernels, CUDA graphs, fused tensor parallelism (in-tree libpie_kernels.so)",
    "cpu": "plain PyTorch fp32 driver on the host: numerics oracle and tests",
    "dummy": "no model: uniform random tokens, for control-plane and scheduler tests",
}


def _drivers_toml() -> Path:
    return cfgmod.default_path().parent / "drivers.toml"


def _read_driver_knobs() -> dict:
    import tomllib
    p = _drivers_toml()
    return tomllib.loads(p.read_text()) if p.exists() else {}


def _write_driver_knobs(d: dict) -> None:
    p = _drivers_toml()
    p.parent.mkdir(parents=True, exist_ok=True)
    out = []
    for typ, kv in sorted(d.items()):
        if kv:
            out.append(f"[{typ}]")
            out += [f"{k} = {cfgmod._fmt(v)}" for k, v in sorted(kv.items())]
            out.append("")
    p.write_text("\n".join(out))


def cmd_driver(args) -> int:
    """`pie driver list [--config F]` and `pie driver <type> install|doctor|show|set K V|unset K`
    (server/src/cli/driver_cmd.rs:41-130). The drivers are in-tree, so `install` is the kernel build
    and the persisted knobs (`drivers.toml` beside the config) are defaults of `[model.driver]` keys."""
    import dataclasses
    typ = args.type.replace("-", "_")
    if typ == "list":
        used = {}
        if args.config or cfgmod.default_path().exists():
            for m in cfgmod.load(args.config).model:
                used.setdefault(m.driver.type, []).append(m.name)
        for t, doc in DRIVER_TYPES.items():
            print(f"{t:12s} {doc}" + (f"   [used by: {', '.join(used[t])}]" if t in used else ""))
        return 0
    if typ not in DRIVER_TYPES:
        raise SystemExit(f"unknown driver {args.type!r}; known: {', '.join(DRIVER_TYPES)}")
    knobs = _read_driver_knobs()
    mine = knobs.setdefault(typ, {})
    valid = {f.name: f for f in dataclasses.fields(cfgmod.DriverConfig) if f.name != "type"}
    act = args.action or "show"
    if act == "install":
        cmd = [sys.executable, "-m", "pie_b200._build"]
        print(" ".join(cmd) + "    # builds libpie_kernels.so (sm_100a) and the host module in-tree")
        if args.run and typ == "cuda_native":
            import subprocess
            return subprocess.call(cmd)
        return 0
    if act == "doctor":
        if typ == "cuda_native":
            return cmd_doctor(args)
        print(f"{typ}: no native dependencies")
        return 0
    if act == "show":
        print(f"[{typ}]  ({_drivers_toml()})")
        for k, f in valid.items():
            src = "drivers.toml" if k in mine else "default"
            v = mine.get(k, f.default if f.default is not dataclasses.MISSING else f.default_factory())
            print(f"  {k:24s} {cfgmod._fmt(v):16s} {src}")
        return 0
    if act in ("set", "unset"):
        if not args.key or args.key not in valid:
            raise SystemExit(f"unknown knob {args.key!r}; known: {', '.join(valid)}")
        if act == "unset":
            mine.pop(args.key, None)
        else:
            if args.value is None:
                raise SystemExit("usage: pie driver <type> set <key> <value>")
            try:
                v = json.loads(args.value)
            except json.JSONDecodeError:
                v = args.value
            probe = cfgmod.DriverConfig(**{**mine, args.key: v, "type": typ})
            cfgmod.validate(cfgmod.Config(model=[cfgmod.ModelSection(name="probe", preset="tiny-llama", driver=probe)]))
            mine[args.key] = v
        _write_driver_knobs(knobs)
        return 0
    raise SystemExit(f"unknown action {act!r}")


TEMPLATE = '''"""{name}: describe what this inferlet does."""
from pie_b200.sdk import Context, Model, Sampler, runtime

NAME = "{name}"


async def main(args):
    model = Model.load(runtime.models()[0])
    ctx = Context(model)
    ctx.system("You are a helpful assistant.").user(args.get("prompt", "Hello")).cue()
    text = await ctx.generate(Sampler.top_p(0.6, 0.95), max_tokens=int(args.get("max_tokens", 128))).collect_text()
    ctx.release()
    return text
'''


def cmd_new(args) -> int:
    d = Path(args.name)
    d.mkdir(parents=True, exist_ok=False)
    (d / "main.py").write_text(TEMPLATE.format(name=args.name))
    (d / "Pie.toml").write_text(f'[package]\nname = "{args.name}"\nversion = "0.1.0"\n\n[runtime]\nlanguage = "python"\n')
    print(f"created {d}/main.py and {d}/Pie.toml")
    return 0


def _package(path: str):
    """(manifest, main.py source, zip bytes) of an inferlet directory (or a single source file beside a Pie.toml)."""
    import ast
    import io
    import zipfile
    from ..runtime.program import Manifest
    p = Path(path)
    d = p if p.is_dir() else p.parent
    src = (d / "main.py") if p.is_dir() else p
    toml = d / "Pie.toml"
    if not src.exists() or not toml.exists():
        raise SystemExit(f"{d}: need main.py and Pie.toml")
    source = src.read_text()
    tree = ast.parse(source)
    if not any(isinstance(n, ast.AsyncFunctionDef) and n.name == "main" for n in tree.body):
        raise SystemExit("missing `async def main(input)`")
    manifest = Manifest.parse(toml.read_text())
    manifest.validate()
    buf = io.BytesIO()
    with zipfile.ZipFile(buf, "w", zipfile.ZIP_DEFLATED) as z:
        z.writestr("Pie.toml", toml.read_text())
        z.writestr("main.py", source)
    return manifest, source, buf.getvalue()


def cmd_build(args) -> int:
    """`pie build <dir> [--out DIR]`: check the program (it parses, defines `async def main`, the manifest is valid)
    and write the package the registry serves: `<out>/<name>-<version>.zip` holding Pie.toml and main.py
    (the role of the reference's `bakery build`, sdk/tools/bakery/src/bakery/build.py)."""
    from ..runtime.program import content_hash
    manifest, source, blob = _package(args.path)
    out = Path(args.out or (Path(args.path) if Path(args.path).is_dir() else Path(args.path).parent) / "dist")
    out.mkdir(parents=True, exist_ok=True)
    target = out / f"{manifest.name}-{manifest.version}.zip"
    target.write_bytes(blob)
    print(f"ok: {target} ({len(blob)} bytes, content hash {content_hash(source.encode())})")
    return 0


def cmd_publish(args) -> int:
    """`pie publish <dir> --registry URL [--token T]`: upload the package to a registry
    (`PUT <registry>/api/v1/inferlets/<name>/<version>`; `bakery publish` in the reference)."""
    import urllib.error
    import urllib.request
    from ..runtime.program import content_hash
    manifest, source, blob = _package(args.path)
    url = f"{args.registry.rstrip('/')}/api/v1/inferlets/{manifest.name}/{manifest.version}"
    req = urllib.request.Request(url, data=blob, method="PUT", headers={
        "Content-Type": "application/zip", "X-Content-Hash": content_hash(source.encode())})
    if args.token:
        req.add_header("Authorization", f"Bearer {args.token}")
    try:
        with urllib.request.urlopen(req, timeout=60) as r:
            print(f"published {manifest.name}@{manifest.version} ({r.status})")
    except urllib.error.HTTPError as e:
        print(f"registry refused {manifest.name}@{manifest.version}: {e.code} {e.reason}", file=sys.stderr)
        return 1
    return 0


def cmd_doctor(args) -> int:
    import shutil
    import torch
    from ..ops import _lib
    print(f"python        {sys.version.split()[0]}")
    print(f"torch         {torch.__version__} cuda={torch.cuda.is_available()} devices={torch.cuda.device_count()}")
    print(f"nvcc          {shutil.which('nvcc') or 'not found'}")
    print(f"kernel lib    {'present' if _lib.lib_path().exists() else 'missing (python -m pie_b200._build)'}")
    try:
        from .._C import pie_host  # noqa: F401
        print("host module   present")
    except ImportError:
        print("host module   missing (python -m pie_b200._build)")
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        print(f"gpu {i}         {p.name} sm_{p.major}{p.minor} {p.total_memory >> 30} GiB {p.multi_processor_count} SMs")
    return 0


def cmd_monitor(args) -> int:
    """`pie monitor [--uri ws://host:port] [--token T]`: the dashboard of a running engine, over its status query."""
    from ..client.client import PieClient
    from .monitor import run_monitor
    c = PieClient(args.uri)
    try:
        if args.token:
            c.auth_by_token(args.token)
        run_monitor(c.model_status, period=args.period, iterations=args.iterations)
    except KeyboardInterrupt:
        pass
    finally:
        c.close()
    return 0


def cmd_check(args) -> int:
    try:
        cfg = cfgmod.load(args.config) if args.config else (
            cfgmod.load(cfgmod.default_path()) if cfgmod.default_path().exists() else cfgmod.default_config())
        print(f"config ok: {len(cfg.model)} model(s)")
        return 0
    except Exception as e:  # noqa: BLE001
        print(f"config error: {e}", file=sys.stderr)
        return 1


def cmd_smoke(args) -> int:
    """Boot a dummy-driver engine, run text-completion through the WebSocket path."""
    args.config, args.driver, args.preset, args.model_path = None, "dummy", "tiny-llama", None
    args.inferlet, args.rest, args.timeout = "text-completion", ["--prompt_tokens", "[1,2,3]", "--max_tokens", "4"], 60
    return cmd_run(args)


def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(name)s %(levelname)s %(message)s")
    ap = argparse.ArgumentParser(prog="pie", description="pie_b200: programmable LLM serving on B200")
    sub = ap.add_subparsers(dest="cmd", required=True)

    def common(p):
        p.add_argument("--config")
        p.add_argument("--driver", choices=["cuda_native", "cpu", "dummy"])
        p.add_argument("--preset")
        p.add_argument("--model-path")
        p.add_argument("--vision", help='vision encoder: "checkpoint" (the tower of --model-path) or a preset such as tiny-vit')
        p.add_argument("--audio", help='audio encoder: "checkpoint" or a preset such as tiny-audio')

    p = sub.add_parser("serve"); common(p)
    p.add_argument("--port", type=int); p.add_argument("--no-auth", action="store_true")
    p.add_argument("--monitor", action="store_true"); p.set_defaults(fn=cmd_serve)
    p = sub.add_parser("run"); common(p)
    p.add_argument("inferlet"); p.add_argument("--timeout", type=float, default=600.0)
    p.add_argument("rest", nargs=argparse.REMAINDER); p.set_defaults(fn=cmd_run)
    p = sub.add_parser("config"); p.add_argument("action", choices=["init", "show", "set"])
    p.add_argument("key", nargs="?"); p.add_argument("value", nargs="?")
    p.add_argument("--config"); p.add_argument("--force", action="store_true"); p.set_defaults(fn=cmd_config)
    p = sub.add_parser("auth"); common(p); p.add_argument("action", choices=["add", "remove", "list", "keygen"])
    p.add_argument("username", nargs="?"); p.add_argument("pubkey", nargs="?"); p.set_defaults(fn=cmd_auth)
    p = sub.add_parser("model"); p.add_argument("action", choices=["list", "download", "remove"], nargs="?", default="list")
    p.add_argument("repo", nargs="?"); p.add_argument("--revision", default="main")
    p.add_argument("--all", action="store_true", help="every file of the repository, not only what the loader reads")
    p.add_argument("--yes", action="store_true"); p.set_defaults(fn=cmd_model)
    p = sub.add_parser("inferlet"); p.add_argument("action", choices=["list"], nargs="?", default="list"); p.set_defaults(fn=cmd_inferlet)
    p = sub.add_parser("driver"); p.add_argument("type", help="list | cuda-native | cpu | dummy")
    p.add_argument("action", nargs="?", choices=["install", "doctor", "show", "set", "unset"])
    p.add_argument("key", nargs="?"); p.add_argument("value", nargs="?")
    p.add_argument("--config"); p.add_argument("--run", action="store_true"); p.set_defaults(fn=cmd_driver)
    p = sub.add_parser("new"); p.add_argument("name"); p.set_defaults(fn=cmd_new)
    p = sub.add_parser("build"); p.add_argument("path"); p.add_argument("--out"); p.set_defaults(fn=cmd_build)
    p = sub.add_parser("publish"); p.add_argument("path"); p.add_argument("--registry", required=True)
    p.add_argument("--token", default=""); p.set_defaults(fn=cmd_publish)
    p = sub.add_parser("monitor"); p.add_argument("--uri", default="ws://127.0.0.1:8080"); p.add_argument("--token", default="")
    p.add_argument("--period", type=float, default=1.0); p.add_argument("--iterations", type=int, default=-1)
    p.set_defaults(fn=cmd_monitor)
    p = sub.add_parser("doctor"); p.set_defaults(fn=cmd_doctor)
    p = sub.add_parser("check"); p.add_argument("--config"); p.set_defaults(fn=cmd_check)
    p = sub.add_parser("smoke"); p.set_defaults(fn=cmd_smoke)
    args = ap.parse_args(argv)
    if getattr(args, "rest", None) and args.rest and args.rest[0] == "--":
        args.rest = args.rest[1:]
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
