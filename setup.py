"""Packaging for dion_b200.  The CUDA kernels are compiled for sm_100a into ``dion_b200/_lib``
at build time when nvcc is available (``python setup.py build_kernels`` or automatically by
``build_py``); they are also built on first use.  Extras: ``dev`` (tests), ``train`` (data
preparation, logging).  There is no ``triton`` extra: nothing here uses it.  With
``DION_B200_COMPAT=1`` in the environment the forwarding packages ``dion`` and ``models`` of
``compat/`` are installed as well, so code written against the reference's import names runs
unchanged; they are left out by default because they would shadow a real ``dion`` install."""
import os
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


def _build_kernels() -> None:
    sys.path.insert(0, HERE)
    from dion_b200.ops import _backend

    if _backend.nvcc_path() is None:
        print("nvcc not found: kernels will be built on first use", file=sys.stderr)
        return
    _backend.build()


class BuildKernels(Command):
    description = "compile the sm_100a kernel libraries into dion_b200/_lib"
    user_options = []

    def initialize_options(self):
        pass

    def finalize_options(self):
        pass

    def run(self):
        _build_kernels()


class BuildPyWithKernels(build_py):
    def run(self):
        try:
            _build_kernels()
        except Exception as exc:  # a missing toolchain must not break a source install
            print(f"kernel build skipped: {exc}", file=sys.stderr)
        super().run()


def _readme() -> str:
    path = os.path.join(HERE, "README.md")
    return open(path, encoding="utf-8").read() if os.path.exists(path) else ""


_packages = find_packages(include=["dion_b200", "dion_b200.*"])
_package_dir = {}
if os.environ.get("DION_B200_COMPAT", "0") == "1":
    _packages += ["dion", "models"]
    _package_dir = {"dion": "compat/dion", "models": "compat/models"}

setup(
    name="dion_b200",
    version="0.1.0",
    description="Orthonormal-update optimizers (Muon, Dion, Dion2, NorMuon) with sm_100a kernels",
    long_description=_readme(),
    long_description_content_type="text/markdown",
    packages=_packages,
    package_dir=_package_dir,
    package_data={"dion_b200": ["csrc/*.cu", "csrc/*.cuh", "csrc/*.h", "_lib/*.so"]},
    python_requires=">=3.10",
    install_requires=["torch>=2.7", "numpy"],
    extras_require={
        "dev": ["pytest", "pytest-timeout"],
        "train": ["pyyaml", "tiktoken", "datasets", "huggingface_hub", "tqdm", "wandb"],
    },
    cmdclass={"build_kernels": BuildKernels, "build_py": BuildPyWithKernels},
    license="MIT",
)
