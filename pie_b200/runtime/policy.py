"""Sandbox policies of an inferlet process: what it may touch outside the engine.

FsPolicy     - "scratch" (a private directory that dies with the process) or "none"
NetworkPolicy - allowlist of CIDR[:port] rules; empty list = no outbound network

Inferlets here are native Python, so the policies are enforced at the SDK's doors
(`sdk.runtime.scratch_dir`, `sdk.http`), not by a wasm sandbox.
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
        os.makedirs(path, exist_ok=True)
        return path

    @staticmethod
    def drop_scratch(path: Optional[str]) -> None:
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
