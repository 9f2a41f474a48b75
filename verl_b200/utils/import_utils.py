"""Import helpers (role of verl/utils/import_utils.py)."""

from __future__ import annotations

import importlib
import importlib.util
from functools import cache
from typing import Optional

from .py_functional import load_extern_object  # noqa: F401  (same loader, historical location)


@cache
def is_package_available(name: str) -> bool:
    return importlib.util.find_spec(name) is not None


def is_vllm_available() -> bool:
    return is_package_available("vllm")


def is_sglang_available() -> bool:
    return is_package_available("sglang")


def is_megatron_core_available() -> bool:
    return is_package_available("megatron.core") if is_package_available("megatron") else False


def import_external_libs(external_libs=None) -> None:
    """Import user modules listed in ``model.external_lib`` (they register models / rewards on import)."""
    if not external_libs:
        return
    if isinstance(external_libs, str):
        external_libs = [external_libs]
    for lib in external_libs:
        importlib.import_module(lib)


def load_extern_type(file_path: str, type_name: str):
    return load_extern_object(file_path, type_name)


def deprecated(replacement: str = ""):
    import functools
    import warnings

    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*a, **k):
            warnings.warn(f"{fn.__qualname__} is deprecated" + (f"; use {replacement}" if replacement else ""),
                          DeprecationWarning, stacklevel=2)
            return fn(*a, **k)

        return wrapper

    return deco


def is_version_in_range(package: str, min_version: Optional[str] = None, max_version: Optional[str] = None) -> bool:
    """Installed version of ``package`` within ``[min_version, max_version]`` (either bound may be None)."""
    import importlib.metadata

    from packaging import version

    try:
        v = version.parse(importlib.metadata.version(package))
    except importlib.metadata.PackageNotFoundError as e:
        raise ModuleNotFoundError(f"The `{package}` package is not installed.") from e
    return (min_version is None or version.parse(min_version) <= v) and (max_version is None or v <= version.parse(max_version))


def is_transformers_version_in_range(min_version: Optional[str] = None, max_version: Optional[str] = None) -> bool:
    """verl/utils/transformers_compat.py:41-60."""
    return is_version_in_range("transformers", min_version, max_version)


def is_version_ge(pkg: str = "transformers", minver: str = "0") -> bool:
    return is_version_in_range(pkg, min_version=minver)


def load_module(module_path: str, module_name: Optional[str] = None):
    """A module from a file path (``pkg://a.b`` or a dotted name imports a module by name)."""
    if not module_path:
        return None
    if module_path.startswith("pkg://"):
        return importlib.import_module(module_path[len("pkg://"):])
    import os
    import sys

    if not os.path.exists(module_path):
        return importlib.import_module(module_path)
    name = module_name or f"custom_module_{abs(hash(os.path.abspath(module_path)))}"
    spec = importlib.util.spec_from_file_location(name, module_path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def load_class_from_fqn(fqn: str, description: str = "class"):
    """``package.module.Class`` -> the class object."""
    mod, _, name = str(fqn).rpartition(".")
    if not mod:
        raise ValueError(f"Invalid {description} name {fqn!r}: expected package.module.Name")
    try:
        return getattr(importlib.import_module(mod), name)
    except (ImportError, AttributeError) as e:
        raise ImportError(f"Cannot load {description} {fqn!r}: {e}") from e


def is_nvtx_available() -> bool:
    return is_package_available("nvtx")


def is_trl_available() -> bool:
    return is_package_available("trl")
