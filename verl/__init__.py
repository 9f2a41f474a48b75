"""``import verl`` compatibility: every ``verl.x.y`` resolves to ``verl_b200.x.y`` (the same module objects, so
``verl.protocol.DataProto is verl_b200.protocol.DataProto``). Code written against the reference's import paths
(``from verl import DataProto``, ``from verl.trainer.ppo import core_algos``, ``verl.single_controller.base``...)
runs unchanged on this framework.
"""

import importlib
import importlib.abc
import importlib.util
import sys

import verl_b200 as _impl

_PREFIX, _TARGET = "verl.", "verl_b200."


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target: str):
        self.target = target

    def create_module(self, spec):
        return importlib.import_module(self.target)

    def exec_module(self, module):  # already executed under its real name
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        real = _TARGET + fullname[len(_PREFIX):]
        try:
            if importlib.util.find_spec(real) is None:
                return None
        except (ImportError, ValueError):
            return None
        is_pkg = hasattr(importlib.import_module(real), "__path__")
        return importlib.util.spec_from_loader(fullname, _AliasLoader(real), is_package=is_pkg)


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

# names the reference exports at the top level
DataProto = _impl.DataProto
__version__ = getattr(_impl, "__version__", "0.0.0")


def __getattr__(name):
    return getattr(_impl, name)
