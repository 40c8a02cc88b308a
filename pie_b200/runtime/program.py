"""Program manager: installs inferlet programs (source + manifest), keeps a disk cache
`<dir>/<name>/<version>.py` + `.toml`, checks content hashes, resolves `name@version`, and
registers entry points with the engine. With a registry URL, a program that is neither registered nor
in the cache is downloaded on first use (`<registry>/api/v1/inferlets/<name>/<version>/download`: a zip
of `Pie.toml` and `main.py`, its content hash in the `X-Content-Hash` header when the registry sends one).

Manifest (`Pie.toml`):
    [package]      name, version, description, authors
    [runtime]      (reserved)
    [parameters]   name -> {type, default, description}   (validated on launch)
    [dependencies] name -> version                         (other programs that must be installed)

Counterpart of runtime/src/program.rs:1-45, program/manifest.rs:12-45, program/repository.rs:19-45.
"""
from __future__ import annotations

import asyncio
import hashlib
import os
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Tuple

try:
    import tomllib
except ImportError:  # pragma: no cover
    tomllib = None


class ProgramError(RuntimeError):
    pass


_NAME = re.compile(r"^[a-z0-9][a-z0-9_-]{0,63}$")
_VERSION = re.compile(r"^\d+\.\d+\.\d+([-+][0-9A-Za-z.-]+)?$")


@dataclass
class Manifest:
    name: str
    version: str = "0.1.0"
    description: str = ""
    authors: List[str] = field(default_factory=list)
    parameters: Dict[str, dict] = field(default_factory=dict)
    dependencies: Dict[str, str] = field(default_factory=dict)
    runtime: Dict[str, Any] = field(default_factory=dict)

    @staticmethod
    def parse(text: str) -> "Manifest":
        if tomllib is None:
            raise ProgramError("tomllib unavailable")
        try:
            doc = tomllib.loads(text)
        except Exception as e:  # noqa: BLE001
            raise ProgramError(f"bad manifest: {e}") from None
        pkg = doc.get("package") or {}
        unknown = set(doc) - {"package", "runtime", "parameters", "dependencies"}
        if unknown:
            raise ProgramError(f"unknown manifest sections {sorted(unknown)}")
        m = Manifest(name=str(pkg.get("name", "")), version=str(pkg.get("version", "0.1.0")),
                     description=str(pkg.get("description", "")), authors=list(pkg.get("authors", [])),
                     parameters=dict(doc.get("parameters") or {}), dependencies=dict(doc.get("dependencies") or {}),
                     runtime=dict(doc.get("runtime") or {}))
        m.validate()
        return m

    def validate(self) -> None:
        if not _NAME.match(self.name):
            raise ProgramError(f"bad program name {self.name!r}")
        if not _VERSION.match(self.version):
            raise ProgramError(f"bad version {self.version!r} (want MAJOR.MINOR.PATCH)")
        for p, spec in self.parameters.items():
            if not isinstance(spec, dict) or spec.get("type", "string") not in ("string", "int", "float", "bool", "json"):
                raise ProgramError(f"parameter {p}: bad spec")

    def to_toml(self) -> str:
        out = ["[package]", f'name = "{self.name}"', f'version = "{self.version}"']
        if self.description:
            out.append(f'description = "{self.description}"')
        if self.authors:
            out.append("authors = [" + ", ".join(f'"{a}"' for a in self.authors) + "]")
        if self.parameters:
            out.append("\n[parameters]")
            for k, spec in self.parameters.items():
                items = ", ".join(f'{a} = {_toml_value(b)}' for a, b in spec.items())
                out.append(f"{k} = {{ {items} }}")
        if self.dependencies:
            out.append("\n[dependencies]")
            out += [f'{k} = "{v}"' for k, v in self.dependencies.items()]
        return "\n".join(out) + "\n"

    def check_input(self, value: Any) -> Any:
        """Fill defaults and check the types of declared parameters of a dict input."""
        if not self.parameters or not isinstance(value, (dict, type(None))):
            return value
        out = dict(value or {})
        casts = {"string": str, "int": int, "float": float, "bool": bool}
        for k, spec in self.parameters.items():
            if k not in out:
                if "default" in spec:
                    out[k] = spec["default"]
                elif spec.get("required"):
                    raise ProgramError(f"missing required parameter {k!r}")
                continue
            t = spec.get("type", "string")
            if t in casts:
                try:
                    out[k] = casts[t](out[k])
                except (TypeError, ValueError):
                    raise ProgramError(f"parameter {k!r}: expected {t}") from None
        return out


def _toml_value(v) -> str:
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, (int, float)):
        return str(v)
    return '"' + str(v).replace('"', '\\"') + '"'


def content_hash(data: bytes) -> str:
    return hashlib.blake2b(data, digest_size=32).hexdigest()


def compile_program(name: str, source: str) -> Callable:
    """Run the module body of an uploaded program (confined: it may import, nothing else) and return `main`."""
    from .policy import Confinement, confine
    ns: Dict[str, Any] = {"__name__": f"pie_program_{name.replace('-', '_')}"}
    with confine(Confinement(name)):
        exec(compile(source, f"<inferlet {name}>", "exec"), ns)   # noqa: S102 - programs are the product's plugins
    if "main" not in ns or not asyncio.iscoroutinefunction(ns["main"]):
        raise ProgramError("an inferlet must define `async def main(input)`")
    return ns["main"]


def _vkey(v: str) -> Tuple:
    core = re.split(r"[-+]", v)[0]
    return tuple(int(x) for x in core.split("."))


class ProgramStore:
    """Disk cache + in-memory registry of installed programs."""

    def __init__(self, engine=None, directory: Optional[str] = None, registry_url: str = ""):
        self.engine = engine
        self.dir = Path(directory) if directory else None
        self.registry_url = registry_url
        self.installed: Dict[str, Dict[str, Manifest]] = {}     # name -> version -> manifest
        if self.dir:
            self.dir.mkdir(parents=True, exist_ok=True)

    # ---- install
    def install(self, source: str, manifest: Manifest, expected_hash: str = "", persist: bool = True) -> str:
        manifest.validate()
        data = source.encode("utf-8")
        h = content_hash(data)
        if expected_hash and expected_hash != h:
            raise ProgramError(f"hash mismatch for {manifest.name}: got {h}")
        for dep, ver in manifest.dependencies.items():
            if self.resolve(dep, ver) is None:
                raise ProgramError(f"{manifest.name} needs {dep}@{ver}, which is not installed")
        entry = compile_program(manifest.name, source)
        if self.dir and persist:
            from .policy import trusted
            with trusted():                        # an inferlet may install a child program: the store writes for it
                d = self.dir / manifest.name
                d.mkdir(parents=True, exist_ok=True)
                (d / f"{manifest.version}.py").write_bytes(data)
                (d / f"{manifest.version}.toml").write_text(manifest.to_toml())
        self.installed.setdefault(manifest.name, {})[manifest.version] = manifest
        if self.engine is not None:
            wrapped = self._wrap(entry, manifest)
            self.engine.register_program(f"{manifest.name}@{manifest.version}", wrapped, manifest, confined=True)
            if manifest.version == self.latest(manifest.name):
                self.engine.register_program(manifest.name, wrapped, manifest, confined=True)
        return h

    @staticmethod
    def _wrap(entry: Callable, manifest: Manifest) -> Callable:
        if not manifest.parameters:
            return entry

        async def main(value):
            return await entry(manifest.check_input(value))
        return main

    def fetch(self, name: str, version: str = "latest", timeout: float = 30.0) -> str:
        """Download `name@version` from the registry and install it; returns `name@version` as installed."""
        import io
        import urllib.error
        import urllib.request
        import zipfile
        if not self.registry_url:
            raise ProgramError(f"program {name!r} is not installed and no registry is configured")
        if not re.fullmatch(r"[A-Za-z0-9][A-Za-z0-9_.-]*", name) or not re.fullmatch(r"[A-Za-z0-9_.+^*-]+", version):
            raise ProgramError(f"bad program reference {name}@{version}")
        url = f"{self.registry_url.rstrip('/')}/api/v1/inferlets/{name}/{version}/download"
        from .policy import trusted
        with trusted():                         # an inferlet may launch a program the engine has to fetch first
            try:
                with urllib.request.urlopen(urllib.request.Request(url, headers={"User-Agent": "pie_b200"}),
                                            timeout=timeout) as r:
                    blob, want = r.read(), r.headers.get("X-Content-Hash", "")
            except urllib.error.HTTPError as e:
                raise ProgramError(f"registry has no {name}@{version} ({e.code})") from None
            except OSError as e:
                raise ProgramError(f"registry {self.registry_url} unreachable: {e}") from None
        try:
            with zipfile.ZipFile(io.BytesIO(blob)) as z:
                manifest = Manifest.parse(z.read("Pie.toml").decode("utf-8"))
                source = z.read("main.py").decode("utf-8")
        except (zipfile.BadZipFile, KeyError) as e:
            raise ProgramError(f"registry sent a bad package for {name}@{version}: {e}") from None
        if manifest.name != name:
            raise ProgramError(f"registry sent {manifest.name!r} for {name!r}")
        self.install(source, manifest, expected_hash=want)
        return f"{manifest.name}@{manifest.version}"

    def ensure(self, ref: str) -> bool:
        """Make `name[@version]` launchable: already registered, or fetched from the registry now."""
        name, _, version = ref.partition("@")
        if self.resolve(name, version) is not None:
            return True
        if not self.registry_url:
            return False
        self.fetch(name, version or "latest")
        return True

    def install_dir(self, path: str) -> str:
        """Install from a directory holding Pie.toml and main.py (or <name>.py)."""
        p = Path(path)
        manifest = Manifest.parse((p / "Pie.toml").read_text())
        src = p / "main.py"
        if not src.exists():
            src = p / f"{manifest.name.replace('-', '_')}.py"
        return self.install(src.read_text(), manifest)

    def load_cache(self) -> List[str]:
        """Register every program found in the disk cache."""
        names = []
        if not self.dir:
            return names
        for d in sorted(self.dir.iterdir()):
            if not d.is_dir():
                continue
            for toml in sorted(d.glob("*.toml"), key=lambda t: _vkey(t.stem)):
                src = toml.with_suffix(".py")
                if src.exists():
                    self.install(src.read_text(), Manifest.parse(toml.read_text()), persist=False)
                    names.append(f"{d.name}@{toml.stem}")
        return names

    # ---- lookup
    def latest(self, name: str) -> Optional[str]:
        vs = self.installed.get(name)
        return max(vs, key=_vkey) if vs else None

    def resolve(self, name: str, version: str = "") -> Optional[Manifest]:
        vs = self.installed.get(name)
        if not vs:
            return None
        if not version or version in ("*", "latest"):
            return vs[self.latest(name)]
        if version.startswith("^"):
            want = _vkey(version[1:])
            ok = [v for v in vs if _vkey(v)[0] == want[0] and _vkey(v) >= want]
            return vs[max(ok, key=_vkey)] if ok else None
        return vs.get(version)

    def list(self) -> List[str]:
        return [f"{n}@{v}" for n, vs in sorted(self.installed.items()) for v in sorted(vs, key=_vkey)]
