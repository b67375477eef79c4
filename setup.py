"""Packaging: the native libraries are built in-tree by build.py (nvcc for sm_100a, g++ / pybind11) before the package
is collected, so a wheel carries libffk.so and _ffcore next to the Python sources."""
import os
import subprocess
import sys

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildNative(build_py):
    def run(self):
        root = os.path.dirname(os.path.abspath(__file__))
        subprocess.check_call([sys.executable, os.path.join(root, "build.py")], cwd=root)
        super().run()


setup(cmdclass={"build_py": BuildNative})
