"""Example inferlets shipped with the engine (native Python programs against pie_b200.sdk).

`install_all(engine)` registers every program under the name its reference counterpart has
in the reference's `inferlets/` directory.
"""
from __future__ import annotations

import importlib
import pkgutil


def install_all(engine) -> list:
    names = []
    for m in pkgutil.iter_modules(__path__):
        mod = importlib.import_module(f"{__name__}.{m.name}")
        if hasattr(mod, "main"):
            name = getattr(mod, "NAME", m.name.replace("_", "-"))
            engine.register_program(name, mod.main, getattr(mod, "MANIFEST", None))
            names.append(name)
    return names
