"""Packaging of supergrok15_b200 (and of its import aliases ``grokking_optimizers`` / ``grokking_race_v2``).

    pip install --no-build-isolation .          # or: pip install --no-build-isolation -e .

With ``nvcc`` on the machine the native extension is compiled for sm_100a (``supergrok15_b200/_build.py``: every
``csrc/*.cu`` with ``-gencode arch=compute_100a,code=sm_100a``, the binding files with the host compiler) and shipped inside
the package; nvcc cross-compiles, so no GPU has to be visible at build time (the reference's setup.py refuses to build
without one, reference setup.py:19-24).  Without ``nvcc`` the package installs as pure Python: CPU tensors then run the
PyTorch statements of every optimizer (``ops/oracle.py``), CUDA tensors raise with the build instruction.
"""
import os
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildWithNative(build_py):
    def run(self):
        sys.path.insert(0, HERE)
        try:
            from supergrok15_b200 import _build
            if _build._nvcc() is None:
                print("supergrok15_b200: nvcc not found - installing without the native extension (CPU oracle path only)")
            else:
                print("supergrok15_b200: built", _build.build())
        except Exception as exc:  # noqa: BLE001
            if os.environ.get("SG_REQUIRE_NATIVE") == "1":
                raise
            print(f"supergrok15_b200: native build failed ({type(exc).__name__}: {exc}); installing without it")
        finally:
            sys.path.pop(0)
        super().run()


setup(
    name="supergrok15-b200",
    version="2.0.0",
    description="Blackwell-native (sm_100a) grokking optimizers: SuperGrok v1.1 / v1.5 / v2, GrokAdamW, NeuralGrok, Prodigy, Grokfast, "
                "Lion, LookSAM, Muon, AdamW; ZeRO-sharded data-parallel engine with in-kernel collectives; the grokking race driver",
    packages=find_packages(include=["supergrok15_b200", "supergrok15_b200.*", "grokking_optimizers", "grokking_optimizers.*"]),
    py_modules=["grokking_race_v2"],
    package_data={"supergrok15_b200": ["_C*.so", "csrc/*.cu", "csrc/*.cuh", "csrc/*.h", "csrc/*.cpp"]},
    cmdclass={"build_py": BuildWithNative},
    python_requires=">=3.10",
    install_requires=["torch>=2.4", "numpy"],
)
