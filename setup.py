"""``pip install -e .`` (development install: the native library stays in the source tree) or
``pip install .``.  The CUDA library is built by ``python -m necklace_b200._build`` (nvcc, sm_100a);
``build_py`` runs it first when nvcc is there, and it is built on first use otherwise."""
import os
import shutil
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildWithNative(build_py):
    def run(self):
        if shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc"):
            sys.path.insert(0, HERE)
            try:
                from necklace_b200 import _build
                _build.build()
            except Exception as e:  # noqa: BLE001
                print(f"necklace_b200: native library not built ({e}); it is built on first use")
        super().run()


def _version():
    for line in open(os.path.join(HERE, "necklace_b200", "__init__.py")):
        if line.startswith("__version__"):
            return line.split("=")[1].strip().strip('"')
    return "0"


setup(
    name="necklace_b200",
    version=_version(),
    description="Hybrid-parallel training framework with hand-written sm_100a kernels and "
                "peer-memory collectives; API of lancelee82/necklace",
    packages=find_packages(include=["necklace_b200", "necklace_b200.*"]),
    package_data={"necklace_b200": ["csrc/*.cu", "csrc/*.cuh", "csrc/*.h", "*.so",
                                   "_alias/necklace/*.py"]},
    python_requires=">=3.10",
    install_requires=["torch", "numpy", "pyzmq", "msgpack"],
    cmdclass={"build_py": BuildWithNative},
)
