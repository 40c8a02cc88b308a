"""In-tree build of the native libraries.

Two shared objects are produced under ``pie_b200/_C``:

* ``libpie_kernels.so`` - every ``.cu`` under ``csrc/kernels`` compiled by nvcc for
  sm_100a (``-gencode arch=compute_100a,code=sm_100a``); plain C ABI, loaded with ctypes.
* ``pie_host*.so`` - the C++ host runtime under ``csrc/host`` (page store, BRLE,
  batch accumulator, tokenizer, grammar engine) as a pybind11 module.

nvcc cross-compiles without a GPU, so the build works on a CPU-only machine.
Objects are rebuilt only when their source (or a header beside it) is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OUT = ROOT / "_C"
KERNEL_LIB = OUT / "libpie_kernels.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found")
    return cand


def _newer(src_paths, target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(p).stat().st_mtime > t for p in src_paths)


def _run(cmd, log_name: str) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    (OUT / "logs").mkdir(parents=True, exist_ok=True)
    (OUT / "logs" / f"{log_name}.log").write_text(" ".join(map(str, cmd)) + "\n" + proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(map(str, cmd))}\n{proc.stdout}\n{proc.stderr}")


def build_kernels(verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile csrc/kernels/*.cu for sm_100a and link libpie_kernels.so."""
    OUT.mkdir(exist_ok=True)
    kdir = CSRC / "kernels"
    headers = list(kdir.glob("*.cuh")) + list(kdir.glob("*.h"))
    sources = sorted(kdir.glob("*.cu"))
    objs = []
    jobs = []
    for src in sources:
        obj = OUT / (src.stem + ".o")
        objs.append(obj)
        if _newer([src, *headers], obj):
            cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(kdir), "-c", str(src), "-o", str(obj)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append((cmd, src.stem))
    if jobs:
        if verbose:
            print(f"[pie_b200] compiling {len(jobs)} CUDA source(s) for sm_100a", file=sys.stderr)
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda j: _run(*j), jobs))
    if jobs or _newer(objs, KERNEL_LIB):
        # link beside the target and rename: a reader (or a snapshot of the tree) never sees a half-written library
        tmp = KERNEL_LIB.with_suffix(".so.tmp")
        _run([_nvcc(), "-shared", "-o", str(tmp), *map(str, objs), "-Xcompiler", "-fPIC"], "link_kernels")
        os.replace(tmp, KERNEL_LIB)
    return KERNEL_LIB


def host_module_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return OUT / f"pie_host{suffix}"


def build_host(verbose: bool = False) -> Path:
    """Compile the C++ host runtime into a pybind11 extension module."""
    import pybind11

    OUT.mkdir(exist_ok=True)
    hdir = CSRC / "host"
    sources = sorted(hdir.glob("*.cpp"))
    headers = list(hdir.glob("*.hpp")) + list(hdir.glob("*.h"))
    target = host_module_path()
    if not sources:
        return target
    objs = []
    jobs = []
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", str(hdir)]
    for src in sources:
        obj = OUT / ("host_" + src.stem + ".o")
        objs.append(obj)
        if _newer([src, *headers], obj):
            jobs.append((["g++", "-O2", "-std=c++20", "-fPIC", "-fvisibility=hidden", "-pthread", *inc,
                          "-c", str(src), "-o", str(obj)], "host_" + src.stem))
    if jobs:
        if verbose:
            print(f"[pie_b200] compiling {len(jobs)} C++ host source(s)", file=sys.stderr)
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda j: _run(*j), jobs))
    if jobs or _newer(objs, target):
        tmp = target.with_name(target.name + ".tmp")
        _run(["g++", "-shared", "-pthread", "-o", str(tmp), *map(str, objs)], "link_host")
        os.replace(tmp, target)
    return target


def build_all(verbose: bool = True) -> None:
    build_kernels(verbose=verbose)
    build_host(verbose=verbose)


if __name__ == "__main__":
    build_kernels(verbose=True, ptxas_info="--ptxas" in sys.argv)
    build_host(verbose=True)
    print("built:", KERNEL_LIB, host_module_path())
