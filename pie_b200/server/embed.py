"""Embedding the engine in a Python program (benches, tests, notebooks):

    from pie_b200.server.embed import Server
    with Server.from_toml("pie.toml") as srv:            # or Server(config_object)
        client = srv.connect()
        print(client.launch_process("text-completion", {"prompt": "hi"}).wait())

Counterpart of sdk/python-server (`pie.server.Server`, `pie.config`).
"""
from __future__ import annotations

from typing import Optional

from .config import Config, load as load_config, parse as parse_config
from .serve import EngineHandle, start_engine


class Server:
    def __init__(self, config: Config, port: Optional[int] = 0):
        self.config, self._port = config, port
        self.handle: Optional[EngineHandle] = None

    @classmethod
    def from_toml(cls, path: str, port: Optional[int] = 0) -> "Server":
        return cls(load_config(path), port)

    @classmethod
    def from_text(cls, toml_text: str, port: Optional[int] = 0) -> "Server":
        return cls(parse_config(toml_text), port)

    def start(self) -> "Server":
        self.handle = start_engine(self.config, serve=True, port=self._port)
        return self

    @property
    def engine(self):
        return self.handle.engine

    @property
    def uri(self) -> str:
        return self.handle.uri

    def connect(self):
        from ..client.client import PieClient
        c = PieClient(self.uri)
        if self.config.auth.enabled:
            c.auth_by_token(self.handle.auth.internal_token)
        return c

    def stop(self) -> None:
        if self.handle is not None:
            self.handle.shutdown()
            self.handle = None

    def __enter__(self) -> "Server":
        return self.start()

    def __exit__(self, *exc) -> None:
        self.stop()
