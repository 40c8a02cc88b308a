"""`pie-client`: talk to a running engine from the shell.

    python -m pie_b200.client.cli [--uri ws://127.0.0.1:8080] [--token T] <command>
        ping
        submit <inferlet> [--input JSON | --key value ...] [--detach]
        attach <process-id>
        abort <process-id>
        list
        install <source.py> <Pie.toml> [--no-force]
        status
        config init [--force] | show | update [--host H] [--port P] [--username U]
                                              [--private-key-path K] [--enable-auth true|false]

Connection settings come from, in order: the command line, the client configuration file
(`~/.pie_b200/client.toml`, or `$PIE_B200_CLIENT_CONFIG`, or `--config`), the defaults. With
`enable_auth = true` the client proves its identity with the private key before the command runs.

Counterpart of client/python/src/pie_client_cli (submit/attach/abort/list/ping/install, config.py,
engine.py).
"""
from __future__ import annotations

import argparse
import getpass
import json
import os
import sys
import tomllib
from pathlib import Path

from .client import ClientError, PieClient


def _kv_to_json(rest):
    out, i = {}, 0
    while i < len(rest):
        k = rest[i]
        if not k.startswith("--"):
            raise SystemExit(f"unexpected argument {k!r} (want --key value)")
        v = rest[i + 1] if i + 1 < len(rest) and not rest[i + 1].startswith("--") else "true"
        i += 2 if v != "true" or (i + 1 < len(rest) and rest[i + 1] == "true") else 1
        try:
            out[k[2:].replace("-", "_")] = json.loads(v)
        except json.JSONDecodeError:
            out[k[2:].replace("-", "_")] = v
    return out


def _stream(handle, out=None, owner: bool = True) -> int:
    """Print a process' events until it returns. Ctrl-C ends the process when this client launched it (`owner`) and only
    stops listening when it attached to somebody's; either way the exit code is 130."""
    out = out or sys.stdout
    while True:
        try:
            ev, val = handle.recv(timeout=3600)
        except KeyboardInterrupt:
            if owner:
                try:
                    sys.stderr.write("interrupted: process terminated\n" if handle.terminate() else "interrupted\n")
                except Exception:  # noqa: BLE001 - the connection may be the thing that broke
                    sys.stderr.write("interrupted\n")
            else:
                sys.stderr.write("detached\n")
            return 130
        if ev == "stdout":
            out.write(val)
            out.flush()
        elif ev == "stderr":
            sys.stderr.write(val)
        elif ev == "message":
            out.write(f"[message] {val}\n")
        elif ev == "return":
            out.write(val + ("\n" if val and not val.endswith("\n") else ""))
            return 0
        elif ev == "error":
            sys.stderr.write(f"error: {val}\n")
            return 1


CONFIG_KEYS = ("host", "port", "username", "private_key_path", "enable_auth")


def config_path(custom=None) -> Path:
    return Path(custom or os.environ.get("PIE_B200_CLIENT_CONFIG", "~/.pie_b200/client.toml")).expanduser()


def load_config(custom=None) -> dict:
    p = config_path(custom)
    return {k: v for k, v in tomllib.loads(p.read_text()).items() if k in CONFIG_KEYS} if p.exists() else {}


def save_config(cfg: dict, custom=None) -> Path:
    p = config_path(custom)
    p.parent.mkdir(parents=True, exist_ok=True)
    fmt = lambda v: ("true" if v else "false") if isinstance(v, bool) else (str(v) if isinstance(v, int) else json.dumps(v))
    p.write_text("".join(f"{k} = {fmt(cfg[k])}\n" for k in CONFIG_KEYS if cfg.get(k) is not None))
    return p


def find_ssh_key():
    for name in ("id_ed25519", "id_rsa", "id_ecdsa"):
        if (Path.home() / ".ssh" / name).exists():
            return f"~/.ssh/{name}"
    return None


def _check_key(path: str) -> bool:
    """Warn (never fail) about a private key that is missing, world-readable or unparsable."""
    p = Path(path).expanduser()
    if not p.exists():
        print(f"warning: private key {p} not found", file=sys.stderr)
        return False
    if os.name == "posix" and p.stat().st_mode & 0o077:
        print(f"warning: private key {p} is readable by others (chmod 600)", file=sys.stderr)
        return False
    try:
        from ..server.auth import load_private_key
        load_private_key(str(p))
        return True
    except Exception as e:  # noqa: BLE001
        print(f"warning: cannot parse private key {p}: {e}", file=sys.stderr)
        return False


def cmd_config(a) -> int:
    if a.action == "init":
        p = config_path(a.config)
        if p.exists() and not a.force:
            print(f"{p} exists (use --force to overwrite)", file=sys.stderr)
            return 1
        key = find_ssh_key()
        cfg = {"host": "127.0.0.1", "port": 8080, "username": getpass.getuser(), "private_key_path": key or "",
               "enable_auth": bool(key)}
        if key:
            _check_key(key)
        print(f"wrote {save_config(cfg, a.config)}")
        return 0
    if a.action == "show":
        p = config_path(a.config)
        if not p.exists():
            print(f"no configuration at {p} (run `config init`)", file=sys.stderr)
            return 1
        print(f"# {p}\n{p.read_text()}", end="")
        return 0
    cfg = load_config(a.config)
    changed = False
    for k in CONFIG_KEYS:
        v = getattr(a, k, None)
        if v is not None:
            cfg[k] = v
            changed = True
    if not changed:
        print("nothing to update: give at least one of --host --port --username --private-key-path --enable-auth",
              file=sys.stderr)
        return 1
    if cfg.get("private_key_path") and a.private_key_path is not None:
        _check_key(cfg["private_key_path"])
    print(f"updated {save_config(cfg, a.config)}")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pie-client")
    ap.add_argument("--uri", default=None)
    ap.add_argument("--token", default="")
    ap.add_argument("--config", default=None, help="client configuration file")
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("ping")
    sub.add_parser("list")
    sub.add_parser("status")
    p = sub.add_parser("submit")
    p.add_argument("inferlet")
    p.add_argument("--input", default=None)
    p.add_argument("--detach", action="store_true")
    p = sub.add_parser("attach")
    p.add_argument("pid")
    p = sub.add_parser("abort")
    p.add_argument("pid")
    p = sub.add_parser("install")
    p.add_argument("source")
    p.add_argument("manifest")
    p.add_argument("--no-force", action="store_true")
    p = sub.add_parser("config")
    p.add_argument("action", choices=["init", "show", "update"])
    p.add_argument("--force", action="store_true")
    p.add_argument("--host"); p.add_argument("--port", type=int); p.add_argument("--username")
    p.add_argument("--private-key-path", dest="private_key_path")
    p.add_argument("--enable-auth", dest="enable_auth", type=lambda v: v.lower() in ("1", "true", "yes"))
    a, rest = ap.parse_known_args(argv)
    if a.cmd == "config":
        return cmd_config(a)
    cfg = load_config(a.config)
    if a.uri is None:
        a.uri = f"ws://{cfg.get('host', '127.0.0.1')}:{cfg.get('port', 8080)}"
    try:
        c = PieClient(a.uri)
    except Exception as e:  # noqa: BLE001
        print(f"cannot connect to {a.uri}: {e}", file=sys.stderr)
        return 2
    try:
        if a.token:
            c.auth_by_token(a.token)
        elif cfg.get("enable_auth") and cfg.get("private_key_path"):
            from ..server.auth import load_private_key
            c.auth_with_key(cfg.get("username") or getpass.getuser(),
                            load_private_key(str(Path(cfg["private_key_path"]).expanduser())))
        if a.cmd == "ping":
            print(c.ping())
        elif a.cmd == "list":
            for p in c.list_processes():
                print(json.dumps(p))
        elif a.cmd == "status":
            print(json.dumps(c.model_status(), indent=1))
        elif a.cmd == "submit":
            value = json.loads(a.input) if a.input is not None else (_kv_to_json(rest) if rest else None)
            h = c.launch_process(a.inferlet, value)
            if a.detach:
                print(h.pid)
                return 0
            return _stream(h)
        elif a.cmd == "attach":
            return _stream(c.attach_process(a.pid), owner=False)
        elif a.cmd == "abort":
            h = c.attach_process(a.pid)
            print("terminated" if h.terminate() else "not running")
        elif a.cmd == "install":
            name = c.install_program(Path(a.source).read_bytes(), Path(a.manifest).read_text(), force=not a.no_force)
            print(f"installed {name}")
        return 0
    except ClientError as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    finally:
        c.close()


if __name__ == "__main__":
    sys.exit(main())
