"""Wheel build: compiles the host module (g++) and the sm_100a kernels (nvcc) into ksanallm_b200/_lib before the
package files are collected. ``python __graft_entry__.py`` does the same in place without packaging."""
import importlib.util
import os

from setuptools import setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildNative(build_py):
    def run(self):
        spec = importlib.util.spec_from_file_location("_ksana_build", os.path.join(HERE, "ksanallm_b200", "_build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build_all()
        super().run()


setup(cmdclass={"build_py": BuildNative})
