"""``pip install -e .`` / ``python setup.py build_ext --inplace`` for helix_a2a_b200.

The reference packages one ``CUDAExtension`` compiled for sm_90 / sm_90a / sm_100
(``setup.py:14-44``).  Here the extension is B200-only (``-gencode arch=compute_100a,code=sm_100a``)
and is built by ``helix_a2a_b200/_build.py`` (nvcc for the kernels, g++ against the torch headers
for the bindings); ``build_ext`` just calls it, so the resulting ``_C*.so`` sits inside the
package directory where the tests, the benchmarks and ``import helix_a2a`` (the drop-in alias
package) find it.
"""
import importlib.util
import os

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


def _load_builder():
    spec = importlib.util.spec_from_file_location("_helix_build", os.path.join(ROOT, "helix_a2a_b200", "_build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class BuildExt(Command):
    description = "compile csrc/ into helix_a2a_b200/_C*.so for sm_100a"
    user_options = [("inplace", "i", "accepted for compatibility: the build is always in-tree"), ("force", "f", "rebuild everything")]
    boolean_options = ["inplace", "force"]

    def initialize_options(self):
        self.inplace = True
        self.force = False

    def finalize_options(self):
        pass

    def run(self):
        _load_builder().build(force=bool(self.force), verbose=True)


class BuildPy(build_py):
    def run(self):
        self.run_command("build_ext")
        super().run()


def _version():
    ns = {}
    with open(os.path.join(ROOT, "helix_a2a_b200", "_version.py")) as f:
        exec(f.read(), ns)
    return ns.get("__version__", "0.0.0")


setup(
    name="helix_a2a_b200",
    version=_version(),
    description="Helix context-parallel decode exchange, attention and o_proj kernels for NVIDIA B200 (sm_100a)",
    packages=find_packages(include=["helix_a2a_b200", "helix_a2a_b200.*", "helix_a2a", "helix_a2a.*"]),
    package_data={"helix_a2a_b200": ["_C*.so", "_ll128_host.so"]},
    python_requires=">=3.10",
    install_requires=["torch>=2.6"],
    cmdclass={"build_ext": BuildExt, "build_py": BuildPy},
    zip_safe=False,
)
