"""In-tree build of the native extension ``deepep_b200._C`` for sm_100a.

``python -m deepep_b200._build`` compiles every ``csrc/kernels/*.cu`` with nvcc
(``-gencode arch=compute_100a,code=sm_100a``), every ``csrc/runtime/*.cpp`` with g++ against
the PyTorch headers, and links them into ``deepep_b200/_C.<abi>.so`` next to this file.
Objects are cached under ``build/`` keyed by a hash of the source, the headers and the flags,
so a rebuild only recompiles what changed. Nothing is installed outside the repository and no
GPU is needed (nvcc cross-compiles).

Parity: replaces ``setup.py`` / ``CMakeLists.txt`` of the reference (setup.py:92-218); the
reference's JIT compile step (csrc/jit/compiler.hpp) has its counterpart in ``deepep_b200/jit``.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List, Sequence

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / 'csrc'
BUILD = ROOT.parent / 'build' / 'deepep_b200'
EXT_SUFFIX = sysconfig.get_config_var('EXT_SUFFIX')
TARGET = ROOT / f'_C{EXT_SUFFIX}'

NVCC_ARCH = ['-gencode', 'arch=compute_100a,code=sm_100a']
NVCC_FLAGS = NVCC_ARCH + ['-O3', '-std=c++17', '-lineinfo', '--expt-relaxed-constexpr', '-Xcompiler', '-fPIC',
                          '--threads', '2']
CXX_FLAGS = ['-O2', '-std=c++17', '-fPIC', '-Wno-deprecated-declarations']


def cuda_home() -> str:
    for key in ('CUDA_HOME', 'CUDA_PATH'):
        if os.environ.get(key):
            return os.environ[key]
    return '/usr/local/cuda'


def _headers_digest() -> str:
    h = hashlib.sha256()
    for path in sorted(CSRC.rglob('*')):
        if path.suffix in ('.hpp', '.cuh', '.h'):
            h.update(path.relative_to(CSRC).as_posix().encode())
            h.update(path.read_bytes())
    return h.hexdigest()


def _object_for(src: Path, cmd_prefix: Sequence[str], headers: str) -> Path:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    h.update(headers.encode())
    h.update(' '.join(cmd_prefix).encode())
    return BUILD / f'{src.stem}.{h.hexdigest()[:16]}.o'


def _run(cmd: Sequence[str]) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError('build command failed:\n' + ' '.join(cmd) + '\n' + proc.stdout)
    if os.environ.get('EP_BUILD_VERBOSE') and proc.stdout.strip():
        print(proc.stdout)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Builds (or refreshes) the extension and returns the path of the shared object."""
    import torch
    from torch.utils import cpp_extension

    BUILD.mkdir(parents=True, exist_ok=True)
    nvcc = os.path.join(cuda_home(), 'bin', 'nvcc')
    torch_inc = cpp_extension.include_paths()
    py_inc = sysconfig.get_paths()['include']
    cuda_inc = os.path.join(cuda_home(), 'include')
    headers = _headers_digest()

    jobs = []
    for src in sorted((CSRC / 'kernels').glob('*.cu')):
        prefix = [nvcc] + NVCC_FLAGS
        if verbose:
            prefix += ['-Xptxas', '-v']
        obj = _object_for(src, prefix, headers)
        jobs.append((src, obj, prefix + ['-c', str(src), '-o', str(obj)]))
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    for src in sorted((CSRC / 'runtime').glob('*.cpp')):
        prefix = (['g++'] + CXX_FLAGS + [f'-I{p}' for p in torch_inc] + [f'-I{py_inc}', f'-I{cuda_inc}',
                  f'-D_GLIBCXX_USE_CXX11_ABI={abi}', '-DTORCH_EXTENSION_NAME=_C', '-DTORCH_API_INCLUDE_EXTENSION_H'])
        obj = _object_for(src, prefix, headers)
        jobs.append((src, obj, prefix + ['-c', str(src), '-o', str(obj)]))

    todo = [j for j in jobs if force or not j[1].exists()]

    def compile_one(job):
        src, obj, cmd = job
        if verbose:
            print(f'[build] {src.relative_to(ROOT)}', flush=True)
        _run(cmd)

    if todo:
        with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 4)) as pool:
            list(pool.map(compile_one, todo))

    objects = [str(j[1]) for j in jobs]
    link_stamp = BUILD / 'link.stamp'
    stamp = hashlib.sha256(' '.join(objects).encode()).hexdigest()
    if force or todo or not TARGET.exists() or not link_stamp.exists() or link_stamp.read_text() != stamp:
        torch_lib = os.path.join(os.path.dirname(torch.__file__), 'lib')
        cuda_lib = os.path.join(cuda_home(), 'lib64')
        cmd = (['g++', '-shared', '-o', str(TARGET)] + objects +
               [f'-L{torch_lib}', f'-L{cuda_lib}', '-lc10', '-lc10_cuda', '-ltorch_cpu', '-ltorch_cuda', '-ltorch',
                '-ltorch_python', '-lcudart', f'-Wl,-rpath,{torch_lib}', f'-Wl,-rpath,{cuda_lib}'])
        _run(cmd)
        link_stamp.write_text(stamp)
    # old objects of earlier source versions
    live = {j[1].name for j in jobs}
    for old in BUILD.glob('*.o'):
        if old.name not in live:
            old.unlink()
    return TARGET


if __name__ == '__main__':
    path = build(force='--force' in sys.argv, verbose='-v' in sys.argv or '--verbose' in sys.argv)
    print(path)
