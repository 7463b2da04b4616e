"""Packaging entry: ``python setup.py build_ext --inplace`` (or ``pip install -e . --no-build-isolation``) compiles
the native module in-tree with nvcc + g++ for sm_100a through ``flexkv_b200/_build.py``; there is no other
build system and no torch C++ dependency."""
import importlib.util
import os

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


def _native_build():
    spec = importlib.util.spec_from_file_location("_flexkv_build", os.path.join(HERE, "flexkv_b200", "_build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build(verbose=True)


class BuildNative(Command):
    description = "compile flexkv_b200._C in-tree (sm_100a)"
    user_options = [("inplace", "i", "accepted for compatibility; the module is always built in-tree")]

    def initialize_options(self):
        self.inplace = True

    def finalize_options(self):
        pass

    def run(self):
        print("built", _native_build())


class BuildPyWithNative(build_py):
    def run(self):
        _native_build()
        super().run()


setup(
    name="flexkv_b200",
    version="0.1.0",
    description="Blackwell-native multi-tier KV-cache manager (HBM / host / SSD / remote / NVLink peers)",
    packages=find_packages(include=["flexkv_b200", "flexkv_b200.*"]),
    package_data={"flexkv_b200": ["_C*.so", "csrc/*.h", "csrc/*.cpp", "csrc/kernels/*"]},
    python_requires=">=3.10",
    install_requires=["numpy", "torch", "pyzmq", "pybind11", "pyyaml"],
    cmdclass={"build_ext": BuildNative, "build_py": BuildPyWithNative},
)
