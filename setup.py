"""Build hook: compile the sm_100a library before the package files are collected, when nvcc is there.

Everything else is declared in pyproject.toml.  Without nvcc the install succeeds without the library; build it later
with ``python -m b200moe.build`` (the ops raise a clear error on a GPU until then).
"""
import importlib.util
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildWithKernels(build_py):
    def run(self):
        if os.environ.get("B200MOE_SKIP_KERNELS", "0") in ("", "0"):
            try:
                # loaded by path: the package's __init__ imports torch, which a build environment may not have
                spec = importlib.util.spec_from_file_location("_b200moe_build", os.path.join(HERE, "b200moe", "build.py"))
                builder = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(builder)
                builder.build_all(verbose=True)
            except Exception as error:      # no nvcc, or a compile error: say so and carry on without the library
                print(f"[b200moe] CUDA library not built ({error}); run `python -m b200moe.build` later", file=sys.stderr)
        super().run()


setup(cmdclass={"build_py": BuildWithKernels})
