"""Wheel build of umdk_original_b200.

``pip wheel . --no-build-isolation`` (or ``python setup.py bdist_wheel``) compiles the CUDA kernels and
the C runtime into ``umdk_original_b200/lib/libumdk_cam.so`` and the PyTorch bindings into
``umdk_original_b200/_C*.so`` with ``umdk_original_b200._build`` (nvcc, sm_100a only) and packs both
next to the Python sources.  The role of the reference's ``pybind/setup.py:55-106`` and its custom
``bdist_wheel`` (``pybind/pytorch_extension/bdist_wheel_build.py``); ``UMDK_CAM_DEBUG=1`` builds the
host code with ``-O0 -g``, like the reference's ``BUILD_TYPE=Debug`` (the device-side range checks are in
every build).
"""
import importlib.util
import os
from pathlib import Path

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

ROOT = Path(__file__).resolve().parent


def _load_build():
    spec = importlib.util.spec_from_file_location("_umdk_build", ROOT / "umdk_original_b200" / "_build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class BuildNative(build_py):
    def run(self):
        _load_build().build_all(debug=os.environ.get("UMDK_CAM_DEBUG") == "1")
        super().run()


setup(
    name="umdk_original_b200",
    version=os.environ.get("CAM_WHL_VERSION", "0.1.0"),
    description="MoE expert-parallel dispatch / combine / fused expert MLP kernels for NVIDIA B200 (sm_100a)",
    packages=find_packages(include=["umdk_original_b200", "umdk_original_b200.*"]),
    package_data={"umdk_original_b200": ["lib/*.so", "_C*.so", "csrc/**/*"]},
    include_package_data=True,
    python_requires=">=3.10",
    install_requires=["torch"],
    cmdclass={"build_py": BuildNative},
    zip_safe=False,
)
