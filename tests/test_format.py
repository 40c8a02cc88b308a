"""Source hygiene checks (the counterpart of the reference's tests/format/*.sh): every Python file compiles, no tabs or
trailing blanks in Python / CUDA / C++ sources, lines within the project's width, native sources name none of the
batched memcpy entry points that this platform cannot run, and package sources carry no machine paths."""
import pathlib
import py_compile
import re

ROOT = pathlib.Path(__file__).resolve().parents[1]
PY = [p for d in ("pie_b200", "tests") for p in (ROOT / d).rglob("*.py")] + [ROOT / "bench.py", ROOT / "__graft_entry__.py"]
NATIVE = [p for ext in ("*.cu", "*.cuh", "*.hpp", "*.cpp", "*.h") for p in (ROOT / "pie_b200" / "csrc").rglob(ext)]
MAX_COLS = {".py": 150, ".cu": 150, ".cuh": 150, ".hpp": 150, ".cpp": 150, ".h": 200}


def test_python_sources_compile():
    for p in PY:
        py_compile.compile(str(p), doraise=True)


def test_no_tabs_trailing_blanks_or_overlong_lines():
    bad = []
    for p in PY + NATIVE:
        if p.name == "pie_bridge.h":        # generated from the field table
            continue
        for i, line in enumerate(p.read_text().splitlines(), 1):
            if "\t" in line:
                bad.append(f"{p.relative_to(ROOT)}:{i}: tab")
            if line != line.rstrip():
                bad.append(f"{p.relative_to(ROOT)}:{i}: trailing blank")
            if len(line) > MAX_COLS[p.suffix]:
                bad.append(f"{p.relative_to(ROOT)}:{i}: {len(line)} columns")
    assert not bad, "\n".join(bad[:40])


def test_sources_name_no_machine_paths_or_batched_memcpy():
    # the batched-copy entry points are spelled in two halves so that this file does not name them either
    pat = re.compile("/root/|Memcpy" + "BatchAsync|Memcpy3D" + "BatchAsync")
    bad = [f"{p.relative_to(ROOT)}:{i}" for p in PY + NATIVE if p.name != "test_format.py"
           for i, line in enumerate(p.read_text().splitlines(), 1) if pat.search(line)]
    assert not bad, "\n".join(bad[:40])
