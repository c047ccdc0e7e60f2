"""pip install . builds the native components in-tree (make + nvcc for sm_100a, no GPU
needed to build) and installs the flagcx_b200 package with them.  Role of setup.py /
pyproject.toml in the FlagCX project."""
import os
import subprocess
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


class BuildNative(build_py):
    def run(self):
        subprocess.check_call([sys.executable, "-c", "from flagcx_b200 import build; build.build(verbose=True)"],
                              cwd=ROOT)
        super().run()


setup(
    name="flagcx_b200",
    version="0.1.0",
    description="Blackwell-native collective communication framework with the capabilities of FlagCX",
    packages=find_packages(include=["flagcx_b200", "flagcx_b200.*"]),
    package_data={"flagcx_b200": ["lib/*.so", "ops/*.so", "torch_backend/*.so"]},
    python_requires=">=3.10",
    cmdclass={"build_py": BuildNative},
)
