"""Resolve a model reference to a local directory: a path, or `org/name[@revision]` looked up in
the Hugging Face cache layout (`$HF_HOME/hub/models--org--name/snapshots/<rev>/`). Resolving never downloads; a missing snapshot
is an error that says where it was looked for. `pie model list | download | remove` manage that cache:
`download` fetches the runtime files of a repository (config, tokenizer, `*.safetensors` and their
index) from `$HF_ENDPOINT` (default https://huggingface.co) into the same layout.
Counterpart of server/src/hf.rs, server/src/cli/model_cmd.rs:20-254 and
driver/cuda/src/hf_snapshot.cpp.
"""
from __future__ import annotations

import fnmatch
import json
import os
import shutil
import sys
import time
import urllib.request
from pathlib import Path
from typing import Callable, List, Optional, Tuple


def hf_cache_root() -> Path:
    if os.environ.get("HF_HUB_CACHE"):
        return Path(os.environ["HF_HUB_CACHE"])
    home = os.environ.get("HF_HOME") or os.path.join(os.path.expanduser("~"), ".cache", "huggingface")
    return Path(home) / "hub"


def resolve_snapshot(repo: str, revision: Optional[str] = None, cache: Optional[Path] = None) -> Optional[Path]:
    root = (cache or hf_cache_root()) / ("models--" + repo.replace("/", "--"))
    snaps = root / "snapshots"
    if not snaps.is_dir():
        return None
    if revision:
        ref = root / "refs" / revision
        if ref.is_file():
            revision = ref.read_text().strip()
        cand = snaps / revision
        return cand if cand.is_dir() else None
    ref = root / "refs" / "main"
    if ref.is_file() and (snaps / ref.read_text().strip()).is_dir():
        return snaps / ref.read_text().strip()
    dirs = sorted((d for d in snaps.iterdir() if d.is_dir()), key=lambda d: d.stat().st_mtime)
    return dirs[-1] if dirs else None


def resolve_model(ref: str) -> Path:
    p = Path(ref).expanduser()
    if p.is_dir():
        return p
    repo, _, rev = ref.partition("@")
    snap = resolve_snapshot(repo, rev or None) if repo.count("/") == 1 else None
    if snap is None:
        raise FileNotFoundError(f"model {ref!r}: not a directory and no snapshot under {hf_cache_root()} "
                                f"(downloads are not performed; place the files there or pass a path)")
    return snap


# ----------------------------------------------------------------------------- cache management
RUNTIME_PATTERNS = ("config.json", "generation_config.json", "tokenizer.json", "tokenizer_config.json", "tokenizer.model",
                    "special_tokens_map.json", "vocab.json", "merges.txt", "chat_template.jinja",
                    "*.safetensors", "*.safetensors.index.json")


def _dir_size(p: Path) -> int:
    seen, total = set(), 0
    for f in p.rglob("*"):
        if f.is_file():
            st = f.stat()                                 # snapshots may link into blobs/: count an inode once
            if (st.st_dev, st.st_ino) not in seen:
                seen.add((st.st_dev, st.st_ino))
                total += st.st_size
    return total


def list_cached(cache: Optional[Path] = None) -> List[Tuple[str, bool, str, int]]:
    """[(repo id, supported, architecture or reason, bytes)] for every `models--*` directory of the cache."""
    from ..models.config import SUPPORTED_MODEL_TYPES
    root = cache or hf_cache_root()
    out = []
    if not root.is_dir():
        return out
    for d in sorted(root.iterdir()):
        if not (d.is_dir() and d.name.startswith("models--")):
            continue
        repo = d.name[len("models--"):].replace("--", "/", 1)
        snap = resolve_snapshot(repo, cache=root)
        ok, why = False, "no config"
        if snap is not None and (snap / "config.json").is_file():
            try:
                mt = json.loads((snap / "config.json").read_text()).get("model_type", "")
                ok, why = (True, mt) if mt in SUPPORTED_MODEL_TYPES else (False, f"unsupported type: {mt}")
            except (OSError, ValueError):
                pass
        out.append((repo, ok, why, _dir_size(d)))
    return out


def _endpoint() -> str:
    return os.environ.get("HF_ENDPOINT", "https://huggingface.co").rstrip("/")


def _open(url: str):
    req = urllib.request.Request(url, headers={"User-Agent": "pie_b200"})
    tok = os.environ.get("HF_TOKEN")
    if tok:
        req.add_header("Authorization", f"Bearer {tok}")
    return urllib.request.urlopen(req, timeout=60)


def download(repo: str, revision: str = "main", all_files: bool = False, cache: Optional[Path] = None,
             progress: Optional[Callable[[str, int, int], None]] = None) -> Path:
    """Fetch a snapshot of `org/name` into the cache; files already complete are kept. Returns the snapshot dir."""
    if repo.count("/") != 1:
        raise ValueError(f"expected org/name, got {repo!r}")
    root = (cache or hf_cache_root()) / ("models--" + repo.replace("/", "--"))
    with _open(f"{_endpoint()}/api/models/{repo}/revision/{revision}") as r:
        info = json.load(r)
    sha = info.get("sha") or revision
    files = [s["rfilename"] for s in info.get("siblings", [])]
    if not all_files:
        files = [f for f in files if any(fnmatch.fnmatch(f, p) for p in RUNTIME_PATTERNS)]
    if not files:
        raise FileNotFoundError(f"{repo}@{revision}: no files to download")
    snap = root / "snapshots" / sha
    for i, name in enumerate(files):
        dst = snap / name
        dst.parent.mkdir(parents=True, exist_ok=True)
        with _open(f"{_endpoint()}/{repo}/resolve/{sha}/{name}") as r:
            size = int(r.headers.get("Content-Length") or 0)
            if dst.is_file() and size and dst.stat().st_size == size:
                continue
            tmp = dst.with_name(dst.name + ".part")
            done = 0
            with open(tmp, "wb") as f:
                while True:
                    chunk = r.read(1 << 22)
                    if not chunk:
                        break
                    f.write(chunk)
                    done += len(chunk)
                    if progress:
                        progress(name, done, size)
            os.replace(tmp, dst)
    (root / "refs").mkdir(parents=True, exist_ok=True)
    (root / "refs" / revision).write_text(sha)
    return snap


def remove(repo: str, cache: Optional[Path] = None) -> int:
    """Delete a cached repository; returns the bytes freed."""
    d = (cache or hf_cache_root()) / ("models--" + repo.replace("/", "--"))
    if not d.is_dir():
        raise FileNotFoundError(f"{repo}: not in {d.parent}")
    n = _dir_size(d)
    shutil.rmtree(d)
    return n


def progress_bar():
    """A one-line terminal progress callback for `download`; silent when stderr is not a terminal."""
    last = [0.0]

    def cb(name: str, done: int, total: int) -> None:
        if not sys.stderr.isatty() or time.monotonic() - last[0] < 0.1 and done != total:
            return
        last[0] = time.monotonic()
        pct = f"{100.0 * done / total:5.1f}%" if total else f"{done >> 20} MiB"
        sys.stderr.write(f"\r{name[:48]:48s} {pct}")
        if done == total:
            sys.stderr.write("\n")
    return cb
