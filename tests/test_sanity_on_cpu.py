"""Sanity tier: every module of the package (and its ``verl`` alias) imports on a CPU-only box, public names resolve,
and the native sources carry a binding for every exported entry point that Python calls."""

import importlib
import pkgutil
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_every_module_imports():
    import verl_b200

    failed = []
    for m in pkgutil.walk_packages(verl_b200.__path__, "verl_b200."):
        if m.name.endswith("__main__"):
            continue
        try:
            importlib.import_module(m.name)
        except BaseException as e:  # noqa: BLE001
            failed.append((m.name, repr(e)[:200]))
    assert not failed, failed


def test_alias_covers_every_module():
    import verl  # noqa: F401
    import verl_b200

    for m in pkgutil.walk_packages(verl_b200.__path__, "verl_b200."):
        if m.name.endswith("__main__") or "._" in m.name:
            continue
        alias = importlib.import_module("verl." + m.name[len("verl_b200."):])
        real = importlib.import_module(m.name)
        if alias is not real:  # a package-shaped view (the reference splits this module into sub-modules)
            for k, v in vars(real).items():
                if not k.startswith("_"):
                    assert getattr(alias, k) is v, (m.name, k)


def test_python_calls_only_exported_native_functions():
    """Every ``vb_*`` name used from Python exists as an ``extern "C"`` definition in the native sources."""
    defined = set()
    for src in list((ROOT / "verl_b200" / "csrc").glob("*.cu")) + list((ROOT / "verl_b200" / "csrc").glob("*.cpp")):
        defined |= set(re.findall(r"\b(vb_[a-z0-9_]+)\s*\(", src.read_text()))
    used = set()
    for py in (ROOT / "verl_b200").rglob("*.py"):
        used |= set(re.findall(r"""["'.](vb_[a-z0-9_]+)""", py.read_text()))
    missing = sorted(u for u in used if u not in defined)
    assert not missing, missing
