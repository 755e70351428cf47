"""Packaging (the counterpart of the reference's rockspec, sharedtensor-scm-1.rockspec:19-26, which builds its one C
file): ``pip install .`` compiles the two native modules in-tree with the same commands as
``python -m sharedtensor_b200._build`` (g++ for the host core, nvcc for sm_100a) and installs them with the package.
"""
from pathlib import Path

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py


class BuildNative(build_py):
    def run(self):
        import importlib.util

        spec = importlib.util.spec_from_file_location("_st_build", Path(__file__).parent / "sharedtensor_b200" / "_build.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build_core()
        mod.build_cuda()
        super().run()


setup(
    name="sharedtensor_b200",
    version="0.1.0",
    description="Asynchronous shared tensor for data-parallel training: reference-compatible TCP tree, NVLink peer-memory rings on B200",
    packages=find_packages(include=["sharedtensor_b200", "sharedtensor_b200.*"]),
    py_modules=["sharedtensor"],
    package_data={"sharedtensor_b200": ["*.so", "csrc/**/*"]},
    cmdclass={"build_py": BuildNative},
    python_requires=">=3.10",
    install_requires=["torch", "pybind11"],
)
