"""Packaging.  The native extensions are compiled by ``stellatrain_b200/_build.py`` (nvcc for sm_100a, g++ for the
CPU tier) next to the Python sources and shipped as package data; ``python setup.py build_ext --inplace`` and
``python __graft_entry__.py`` do the same build.  The reference builds with CMake (backend/CMakeLists.txt:1-110)."""
import importlib.util
from pathlib import Path

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

ROOT = Path(__file__).resolve().parent


def _build_native() -> None:
    spec = importlib.util.spec_from_file_location("_st_build", ROOT / "stellatrain_b200" / "_build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build_all()


class BuildExt(Command):
    description = "compile the native extensions in-tree"
    user_options = [("inplace", "i", "accepted for compatibility; the build is always in-tree")]

    def initialize_options(self):
        self.inplace = True

    def finalize_options(self):
        pass

    def run(self):
        _build_native()


class BuildPy(build_py):
    def run(self):
        _build_native()
        super().run()


setup(
    packages=find_packages(include=["stellatrain_b200", "stellatrain_b200.*"]),
    package_data={"stellatrain_b200": ["*.so", "*.pyi", "csrc/**/*", "utils/*.txt", "control/profiles/*.json"]},
    cmdclass={"build_ext": BuildExt, "build_py": BuildPy},
)
