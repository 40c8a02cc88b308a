"""`pie-client`: talk to a running engine from the shell.

    python -m pie_b200.client.cli [--uri ws://127.0.0.1:8080] [--token T] <command>
        ping
        submit <inferlet> [--input JSON | --key value ...] [--detach]
        attach <process-id>
        abort <process-id>
        list
        install <source.py> <Pie.toml> [--no-force]
        status

Counterpart of client/python/src/pie_client_cli (submit/attach/abort/list/ping/install).
"""
from __future__ import annotations

import argparse
import json
import sys
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


def _stream(handle, out=sys.stdout) -> int:
    while True:
        ev, val = handle.recv(timeout=3600)
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


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pie-client")
    ap.add_argument("--uri", default="ws://127.0.0.1:8080")
    ap.add_argument("--token", default="")
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
    a, rest = ap.parse_known_args(argv)
    try:
        c = PieClient(a.uri)
    except Exception as e:  # noqa: BLE001
        print(f"cannot connect to {a.uri}: {e}", file=sys.stderr)
        return 2
    try:
        if a.token:
            c.auth_by_token(a.token)
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
            return _stream(c.attach_process(a.pid))
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
