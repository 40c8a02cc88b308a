"""Resolve a model reference to a local directory: a path, or `org/name[@revision]` looked up in
the Hugging Face cache layout (`$HF_HOME/hub/models--org--name/snapshots/<rev>/`). Nothing is
downloaded; a missing snapshot is an error that says where it was looked for.
Counterpart of server/src/hf.rs and driver/cuda/src/hf_snapshot.cpp.
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import Optional


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
