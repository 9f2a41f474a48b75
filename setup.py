"""``pip install -e .`` support: the native library is built in-tree for sm_100a (``verl_b200/_build.py``) when nvcc is
present, so that an installed package finds ``verl_b200/lib/libverl_b200.so`` beside its sources."""

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildWithNative(build_py):
    def run(self):
        try:
            import importlib.util
            import pathlib

            spec = importlib.util.spec_from_file_location("_vb_build", pathlib.Path(__file__).parent / "verl_b200" / "_build.py")
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.build()
        except Exception as e:  # no nvcc: the Python layer still installs; GPU ops raise on first use
            print(f"[verl_b200] native library not built: {e}")
        super().run()


setup(cmdclass={"build_py": BuildWithNative})
