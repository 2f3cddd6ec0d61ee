"""Packaging of deepep_b200: ``pip install .`` (or ``pip install -e .``) builds the native extension for sm_100a with the
in-tree builder (nvcc + g++, no GPU needed) and installs the package together with the kernel headers that the run-time
compiler includes.

Build-time switches (read from the environment, like the reference's setup.py:70-89):
``EP_NUM_TOPK_IDX_BITS`` (32 or 64) is baked into ``deepep_b200/envs.py`` as the default dtype of routing indices
(``deepep_b200.topk_idx_t``; the kernels accept both widths at run time), as are ``EP_JIT_CACHE_DIR`` and
``EP_HEAP_BACKEND`` when set. ``CUDA_HOME`` selects the toolkit.

Parity: setup.py:92-218 of the reference (CUDAExtension + persistent environment variables baked at build time).
"""
import os
import sys
from pathlib import Path

from setuptools import Extension, find_packages, setup
from setuptools.command.build_ext import build_ext
from setuptools.command.build_py import build_py

ROOT = Path(__file__).resolve().parent
PERSISTENT_ENVS = ('EP_NUM_TOPK_IDX_BITS', 'EP_JIT_CACHE_DIR', 'EP_HEAP_BACKEND')


class BuildNative(build_ext):
    """Runs the in-tree builder and copies the shared object to where setuptools expects it."""

    def run(self):
        sys.path.insert(0, str(ROOT))
        from deepep_b200 import _build
        target = _build.build()
        for ext in self.extensions:
            dest = Path(self.get_ext_fullpath(ext.name))
            dest.parent.mkdir(parents=True, exist_ok=True)
            if dest.resolve() != Path(target).resolve():
                self.copy_file(str(target), str(dest))


class BuildPy(build_py):
    """Writes the persistent environment defaults next to the package."""

    def run(self):
        lines = ['"""Environment defaults fixed when the package was built (setup.py)."""', 'persistent_envs = {']
        for key in PERSISTENT_ENVS:
            if os.environ.get(key):
                lines.append(f'    {key!r}: {os.environ[key]!r},')
        lines.append('}')
        (ROOT / 'deepep_b200' / 'envs.py').write_text('\n'.join(lines) + '\n')
        super().run()


setup(
    name='deepep_b200',
    version='0.2.0',
    description='B200-native expert-parallel communication library (dispatch / combine over NVLink 5, tcgen05 GEMMs)',
    packages=find_packages(include=['deepep_b200', 'deepep_b200.*']),
    package_data={'deepep_b200': ['csrc/**/*.hpp', 'csrc/**/*.cuh', 'csrc/**/*.h', 'csrc/**/*.cu', 'csrc/**/*.cpp']},
    ext_modules=[Extension('deepep_b200._C', sources=[])],
    cmdclass={'build_ext': BuildNative, 'build_py': BuildPy},
    python_requires='>=3.10',
    install_requires=['torch'],
)
