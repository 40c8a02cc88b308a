"""Filesystem scratch space and outbound HTTP for inferlets, both behind the process's policies.

    path = io.scratch_path("notes.txt")          # inside the private scratch directory
    io.write_text("notes.txt", "hello"); io.read_text("notes.txt")
    resp = await io.http_fetch("http://10.0.0.5:8080/x", method="POST", body=b"...")

Counterpart of the wasi:filesystem `/scratch` preopen and wasi:http outgoing handler that the
reference links into every instance (runtime/src/instance.rs:89-125, runtime/src/linker.rs:101-222).
"""
from __future__ import annotations

import asyncio
import os
import urllib.error
import urllib.parse
import urllib.request
from dataclasses import dataclass
from typing import Dict, Optional

from ..runtime.policy import FsPolicy, PolicyError
from . import host


def scratch_dir() -> str:
    return host.proc().scratch()


def scratch_path(relative: str) -> str:
    return FsPolicy.resolve(scratch_dir(), relative)


def write_text(relative: str, text: str) -> None:
    p = scratch_path(relative)
    os.makedirs(os.path.dirname(p), exist_ok=True)
    with open(p, "w") as f:
        f.write(text)


def read_text(relative: str) -> str:
    with open(scratch_path(relative)) as f:
        return f.read()


def write_bytes(relative: str, data: bytes) -> None:
    p = scratch_path(relative)
    os.makedirs(os.path.dirname(p), exist_ok=True)
    with open(p, "wb") as f:
        f.write(data)


def read_bytes(relative: str) -> bytes:
    with open(scratch_path(relative), "rb") as f:
        return f.read()


def listdir(relative: str = "") -> list:
    return sorted(os.listdir(scratch_path(relative) if relative else scratch_dir()))


@dataclass
class HttpResponse:
    status: int
    headers: Dict[str, str]
    body: bytes

    def text(self) -> str:
        return self.body.decode("utf-8", errors="replace")


async def http_fetch(url: str, method: str = "GET", headers: Optional[Dict[str, str]] = None,
                     body: Optional[bytes] = None, timeout: float = 30.0) -> HttpResponse:
    """HTTP request to a destination the process's network policy allows."""
    u = urllib.parse.urlsplit(url)
    if u.scheme not in ("http", "https"):
        raise PolicyError(f"scheme {u.scheme!r} is not allowed")
    pol = host.proc().network_policy
    if pol is None:
        raise PolicyError("this process has no network access")
    pol.check(u.hostname or "", u.port or (443 if u.scheme == "https" else 80))

    def do():
        req = urllib.request.Request(url, data=body, method=method, headers=headers or {})
        try:
            with urllib.request.urlopen(req, timeout=timeout) as r:   # noqa: S310 - scheme checked above
                return HttpResponse(r.status, dict(r.headers.items()), r.read())
        except urllib.error.HTTPError as e:
            return HttpResponse(e.code, dict(e.headers.items()), e.read())

    return await asyncio.get_running_loop().run_in_executor(None, do)
