"""The WIT files under pie_b200/wit are the inferlet contract; pie_b200.sdk.wit is its native host.
This test parses the WIT text and checks, function by function and resource by resource, that the
host has an entry of the same name (kebab-case -> snake_case) taking the same number of parameters,
and exercises the contract-level calls of one decode step against a mock driver."""
import asyncio
import inspect
import json
import re
from pathlib import Path

import pytest

from pie_b200.driver.mock import CounterBehavior, MockDriver
from pie_b200.inferlets import install_all
from pie_b200.runtime.engine import Engine, EngineConfig
from pie_b200.sdk import wit

WIT_DIR = Path(wit.__file__).resolve().parents[1] / "wit"


def parse_wit(text: str):
    """-> {interface: {"funcs": {name: arity}, "resources": {res: {method: (arity, kind)}}}}"""
    text = re.sub(r"//[^\n]*", "", text)
    out = {}
    for m in re.finditer(r"interface\s+([a-z0-9-]+)\s*\{", text):
        depth, i = 1, m.end()
        while depth:
            depth += {"{": 1, "}": -1}.get(text[i], 0)
            i += 1
        body = text[m.end():i - 1]
        iface = {"funcs": {}, "resources": {}}
        # resources first, then what is left are free functions / types
        rest = body
        for r in re.finditer(r"resource\s+([a-z0-9-]+)\s*\{", body):
            d, j = 1, r.end()
            while d:
                d += {"{": 1, "}": -1}.get(body[j], 0)
                j += 1
            rbody = body[r.end():j - 1]
            rest = rest.replace(body[r.start():j], "")
            methods = {}
            for f in re.finditer(r"([a-z0-9-]+)\s*:\s*(static\s+)?func\s*\(([^)]*)\)", rbody, re.S):
                methods[f.group(1)] = (_arity(f.group(3)), "static" if f.group(2) else "method")
            c = re.search(r"constructor\s*\(([^)]*)\)", rbody, re.S)
            if c:
                methods["constructor"] = (_arity(c.group(1)), "constructor")
            iface["resources"][r.group(1)] = methods
        for f in re.finditer(r"([a-z0-9-]+)\s*:\s*func\s*\(([^)]*)\)", rest, re.S):
            iface["funcs"][f.group(1)] = _arity(f.group(2))
        out[m.group(1)] = iface
    return out


def _arity(params: str) -> int:
    params = params.strip()
    if not params:
        return 0
    depth, n = 0, 1
    for ch in params.rstrip(","):
        depth += {"<": 1, ">": -1}.get(ch, 0)
        if ch == "," and depth == 0:
            n += 1
    return n


def _snake(name: str) -> str:
    return name.replace("-", "_")


def _py_arity(fn, drop_self: bool) -> int:
    ps = [p for p in inspect.signature(fn).parameters.values()
          if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
    return len(ps) - (1 if drop_self else 0)


def contract():
    found = {}
    for pkg_dir in sorted(p for p in WIT_DIR.iterdir() if p.is_dir()):
        pkg = re.search(r"package\s+([a-z:]+)\s*;", (pkg_dir / "imports.wit").read_text()).group(1)
        world = re.findall(r"import\s+([a-z0-9-]+)\s*;", (pkg_dir / "imports.wit").read_text())
        for f in sorted(pkg_dir.glob("*.wit")):
            for name, iface in parse_wit(f.read_text()).items():
                found[f"{pkg}/{name}"] = iface
        for name in world:
            assert f"{pkg}/{name}" in found, f"world imports {pkg}/{name} but no interface defines it"
    return found


def test_every_wit_function_has_a_host_entry_of_the_same_arity():
    spec = contract()
    assert len(spec) >= 18 and "pie:core/inference" in spec and "pie:zo/zo" in spec
    checked = 0
    for key, iface in spec.items():
        if key == "pie:core/run":
            continue                      # the inferlet's export, not a host import
        host_iface = wit.INTERFACES.get(key)
        assert host_iface is not None, f"no host interface for {key}"
        for fname, arity in iface["funcs"].items():
            fn = getattr(host_iface, _snake(fname), None)
            assert callable(fn), f"{key}.{fname} missing in the host"
            assert _py_arity(fn, drop_self=False) == arity, f"{key}.{fname}: arity {_py_arity(fn, False)} != {arity}"
            checked += 1
        for rname, methods in iface["resources"].items():
            cls = getattr(host_iface, _snake(rname), None)
            assert inspect.isclass(cls), f"{key}: resource {rname} missing in the host"
            for mname, (arity, kind) in methods.items():
                if kind == "constructor":
                    got = _py_arity(cls.__init__, drop_self=True)
                else:
                    attr = inspect.getattr_static(cls, _snake(mname), None)
                    assert attr is not None, f"{key}.{rname}.{mname} missing in the host"
                    is_static = isinstance(attr, staticmethod)
                    assert is_static == (kind == "static"), f"{key}.{rname}.{mname}: static mismatch"
                    got = _py_arity(getattr(cls, _snake(mname)), drop_self=not is_static)
                assert got == arity, f"{key}.{rname}.{mname}: arity {got} != {arity}"
                checked += 1
    assert checked >= 120


def test_world_lists_every_package():
    world = (WIT_DIR / "world.wit").read_text()
    for pkg in ("pie:core/imports", "pie:instruct/imports", "pie:mcp/imports", "pie:zo/imports"):
        assert world.count(f"include {pkg};") == 2         # in `imports` and in `inferlet`
    assert (WIT_DIR / "core" / "run.wit").read_text().count("run: func(input: string) -> result<string, error>;") == 1


PROGRAM = '''
import asyncio, json
from pie_b200.sdk import wit

async def main(args):
    m = wit.model.model.load(wit.runtime.models()[0])
    ctx = wit.context.context.create(m)
    ps = ctx.tokens_per_page()
    prompt = list(range(1, ps + 4))
    ctx.reserve_working_pages(2)
    fp = wit.inference.forward_pass(m)
    fp.context(ctx)
    fp.input_tokens(prompt, list(range(len(prompt))))
    fp.sampler([len(prompt) - 1], ("top-p", (0.0, 1.0)))
    fp.sampler([len(prompt) - 1], "entropy")
    fut = fp.execute()
    await fut.pollable().block()
    out = fut.get()
    ctx.commit_working_pages(1)
    fork = ctx.fork()
    name = ctx.snapshot()
    counts = [ctx.committed_page_count(), ctx.working_page_count(), ctx.working_page_token_count(),
              fork.committed_page_count()]
    ctx.truncate_working_page_tokens(1)
    after = ctx.working_page_token_count()
    wit.context.context.delete(m, name)
    fork.destroy(); ctx.destroy()
    tok = m.tokenizer()
    wit.session.send("hi")
    wit.messaging.push("q", "x")
    f = wit.messaging.pull("q")
    await f.pollable().block()
    return json.dumps({"slots": [s[0] for s in out["slots"]], "token": out["slots"][0][1], "counts": counts,
                       "after": after, "roundtrip": tok.decode(tok.encode("ab")), "pulled": f.get(),
                       "price": wit.scheduling.price(), "user": wit.runtime.username()})
'''


def test_contract_level_decode_step_against_the_mock_driver():
    from pie_b200.runtime.program import Manifest, ProgramStore
    eng = Engine(EngineConfig(watchdog_interval_s=0.1))
    from pie_b200.runtime.tokenizer import ByteTokenizer
    eng.add_model("mock", MockDriver(CounterBehavior(), total_pages=64), tokenizer=ByteTokenizer(512))
    install_all(eng)
    try:
        ProgramStore(eng).install(PROGRAM, Manifest.parse('[package]\nname = "wit-level"\nversion = "0.1.0"\n'), persist=False)
        res = json.loads(eng.run("wit-level", {}, timeout=60))
        assert res["slots"] == ["token", "entropy"]
        ps = 16
        assert res["token"] == ps + 4                       # the counter driver answers last token + 1
        assert res["counts"] == [1, 1, 3, 1] and res["after"] == 2
        assert res["roundtrip"] == "ab" and res["pulled"] == "x" and res["price"] == 1.0
    finally:
        eng.shutdown()
