"""Sandbox policies of an inferlet process: what it may touch outside the engine.

FsPolicy     - "scratch" (a private directory that dies with the process) or "none"
NetworkPolicy - allowlist of CIDR[:port] rules; empty list = no outbound network

Inferlets here are native Python, so the policies are enforced at the SDK's doors
(`sdk.runtime.scratch_dir`, `sdk.http`) and, for programs that were uploaded rather than shipped with
the package, by an interpreter audit hook (second half of this file), not by a wasm sandbox.
Counterpart of runtime/src/policy.rs:1-45 and its use in runtime/src/instance.rs:89-125.
"""
from __future__ import annotations

import ipaddress
import os
import shutil
import socket
import tempfile
from dataclasses import dataclass, field
from typing import List, Optional, Tuple


class PolicyError(PermissionError):
    pass


@dataclass
class FsPolicy:
    mode: str = "scratch"           # "scratch" | "none"
    root: Optional[str] = None      # parent of the per-process scratch directories

    def __post_init__(self):
        if self.mode not in ("scratch", "none"):
            raise ValueError(f"unknown filesystem policy {self.mode!r}")

    def make_scratch(self, process_id: str) -> Optional[str]:
        if self.mode == "none":
            return None
        base = self.root or os.path.join(tempfile.gettempdir(), "pie_b200_scratch")
        path = os.path.join(base, process_id)
        with trusted():
            os.makedirs(path, exist_ok=True)
        return path

    @staticmethod
    def drop_scratch(path: Optional[str]) -> None:
        with trusted():
            if path and os.path.isdir(path):
                shutil.rmtree(path, ignore_errors=True)

    @staticmethod
    def resolve(scratch: Optional[str], relative: str) -> str:
        """Path inside the scratch directory; anything that escapes it is refused."""
        if scratch is None:
            raise PolicyError("this process has no filesystem access")
        full = os.path.realpath(os.path.join(scratch, relative.lstrip("/")))
        root = os.path.realpath(scratch)
        if full != root and not full.startswith(root + os.sep):
            raise PolicyError(f"path {relative!r} escapes the scratch directory")
        return full


@dataclass
class NetRule:
    net: "ipaddress._BaseNetwork"
    port: Optional[int] = None

    @staticmethod
    def parse(text: str) -> "NetRule":
        text = text.strip()
        port = None
        host = text
        if text.startswith("["):                       # [v6]/len:port
            end = text.index("]")
            host, rest = text[1:end], text[end + 1:]
            if rest.startswith("/"):
                pre, _, p = rest[1:].partition(":")
                host = f"{host}/{pre}"
                port = int(p) if p else None
            elif rest.startswith(":"):
                port = int(rest[1:])
        elif text.count(":") == 1:
            host, p = text.split(":")
            port = int(p)
        return NetRule(ipaddress.ip_network(host, strict=False), port)

    def allows(self, addr, port: int) -> bool:
        return addr.version == self.net.version and addr in self.net and (self.port is None or self.port == port)


@dataclass
class NetworkPolicy:
    allow: List[str] = field(default_factory=list)
    rules: List[NetRule] = field(init=False, default_factory=list)

    def __post_init__(self):
        self.rules = [NetRule.parse(r) for r in self.allow]

    @staticmethod
    def allow_all() -> "NetworkPolicy":
        return NetworkPolicy(["0.0.0.0/0", "::/0"])

    def check(self, host: str, port: int) -> Tuple[str, int]:
        """Resolve `host` and return the first address the policy allows; raise otherwise."""
        try:
            addrs = [ipaddress.ip_address(host)]
        except ValueError:
            try:
                infos = socket.getaddrinfo(host, port, type=socket.SOCK_STREAM)
            except OSError as e:
                raise PolicyError(f"cannot resolve {host}: {e}") from None
            addrs = [ipaddress.ip_address(i[4][0]) for i in infos]
        for a in addrs:
            if any(r.allows(a, port) for r in self.rules):
                return str(a), port
        raise PolicyError(f"network policy denies {host}:{port}")


# ------------------------------------------------------------------------------ confinement of uploaded programs
# Programs that ship with the package are trusted. A program that arrived through the server (upload, disk cache,
# registry) runs in the same interpreter, so the policies above are also enforced from inside the interpreter: an
# audit hook sees every file open, socket connect / bind, process spawn, dynamic library load and thread start,
# and refuses those that the policy of the running process does not allow - whether the program went through
# the SDK's doors or imported `os` / `socket` / `ctypes` itself. The scope is a context variable, so it follows the
# inferlet's asyncio task and nothing else. This closes the interpreter's own doors; it is not a defence against
# code that attacks the interpreter it shares with the engine (the reference's wasm sandbox has no equivalent here).
import contextlib
import contextvars
import sys


@dataclass
class Confinement:
    """What the code running in this scope may touch."""
    name: str = ""
    scratch: Optional[str] = None                    # writable (and readable) directory, None = no file access
    network: Optional[NetworkPolicy] = None          # None = no outbound network
    process: Optional[object] = None                 # the Process, for a scratch directory created later

    def scratch_root(self) -> Optional[str]:
        if self.process is not None:
            return getattr(self.process, "scratch_dir", None)
        return self.scratch


_scope: "contextvars.ContextVar[Optional[Confinement]]" = contextvars.ContextVar("pie_confinement", default=None)
_hook_installed = False
_read_roots: Optional[Tuple[str, ...]] = None
denied_events: List[Tuple[str, str]] = []            # (program, event) of what was refused, newest last (bounded)


@contextlib.contextmanager
def confine(c: Confinement):
    install_audit_hook()
    tok = _scope.set(c)
    try:
        yield c
    finally:
        _scope.reset(tok)


@contextlib.contextmanager
def trusted():
    """Engine code that works on behalf of a confined program (program store, adapter files, scratch set-up)."""
    tok = _scope.set(None)
    try:
        yield
    finally:
        _scope.reset(tok)


def _roots() -> Tuple[str, ...]:
    global _read_roots
    if _read_roots is None:
        cand = {sys.prefix, sys.base_prefix, sys.exec_prefix, os.path.dirname(os.__file__)}
        cand.update(p for p in sys.path if p and os.path.isdir(p))
        _read_roots = tuple(sorted({os.path.realpath(p) for p in cand}))
    return _read_roots


def _inside(path, roots) -> bool:
    try:
        full = os.path.realpath(os.fspath(path))
    except TypeError:
        return False
    if isinstance(full, bytes):
        full = os.fsdecode(full)
    return any(full == r or full.startswith(r + os.sep) for r in roots if r)


def _deny(c: Confinement, event: str, what: str):
    denied_events.append((c.name, event))
    del denied_events[:-256]
    raise PolicyError(f"{event} denied for program {c.name or '?'}: {what}")


_WRITE_FLAGS = os.O_WRONLY | os.O_RDWR | os.O_APPEND | os.O_CREAT | os.O_TRUNC
_PATH_EVENTS = {"os.remove": 0, "os.rename": None, "os.mkdir": 0, "os.rmdir": 0, "os.chmod": 0, "os.chown": 0,
                "os.truncate": 0, "os.link": None, "os.symlink": None, "shutil.rmtree": 0, "shutil.copyfile": None,
                "shutil.move": None, "shutil.copytree": None, "os.utime": 0, "tempfile.mkstemp": None,
                "tempfile.mkdtemp": None}
_SPAWN_EVENTS = {"subprocess.Popen", "os.system", "os.exec", "os.posix_spawn", "os.spawn", "os.fork", "os.forkpty",
                 "os.startfile", "pty.spawn", "os.kill", "os.killpg", "ctypes.dlopen", "ctypes.dlsym", "ctypes.cdata",
                 "ctypes.call_function", "_thread.start_new_thread", "socket.bind", "sys.addaudithook", "os.putenv",
                 "os.unsetenv", "signal.pthread_kill", "syslog.syslog", "webbrowser.open", "mmap.__new__"}


def _audit(event: str, args) -> None:
    c = _scope.get()
    if c is None:
        return
    if event == "open":
        path, mode, flags = (list(args) + [None, None])[:3]
        if isinstance(path, int):
            return                                   # an already open descriptor
        writing = bool((flags or 0) & _WRITE_FLAGS) or (isinstance(mode, str) and any(ch in mode for ch in "wax+"))
        scratch = c.scratch_root()
        if scratch and _inside(path, (os.path.realpath(scratch),)):
            return
        if not writing and _inside(path, _roots()):
            return                                   # the interpreter's own files: imports must keep working
        _deny(c, event, f"{path!r} ({'write' if writing else 'read'}) is outside the scratch directory")
    elif event == "socket.connect":
        addr = args[1]
        if isinstance(addr, tuple) and len(addr) >= 2 and c.network is not None:
            try:
                ip = ipaddress.ip_address(addr[0])
                if any(r.allows(ip, int(addr[1])) for r in c.network.rules):
                    return
            except ValueError:
                pass
        _deny(c, event, f"{addr!r} is not on the network allow list")
    elif event in ("socket.getaddrinfo", "socket.gethostbyname"):
        if c.network is None or not c.network.rules:
            _deny(c, event, "this program has no network access")
    elif event in _SPAWN_EVENTS:
        _deny(c, event, "not available to uploaded programs")
    elif event in _PATH_EVENTS or event in ("os.listdir", "os.scandir", "glob.glob"):
        scratch = c.scratch_root()
        roots = (os.path.realpath(scratch),) if scratch else ()
        paths = [a for a in args[:2] if isinstance(a, (str, bytes, os.PathLike))] if _PATH_EVENTS.get(event, 0) is None \
            else [a for a in args[:1] if isinstance(a, (str, bytes, os.PathLike))]
        for p in paths:
            if not _inside(p, roots):
                _deny(c, event, f"{p!r} is outside the scratch directory")


def install_audit_hook() -> None:
    """Idempotent. An audit hook cannot be removed; outside a confined scope it costs one context-variable read."""
    global _hook_installed
    if not _hook_installed:
        _hook_installed = True
        _roots()
        sys.addaudithook(_audit)
