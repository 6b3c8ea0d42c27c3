"""Ahead-of-time build of libdgb200.so (all sm_100a kernels + the C-ABI host layer) with nvcc.

Replaces the reference's runtime JIT (csrc/jit/compiler.hpp:100-252): nothing is compiled at call time.
Run as ``python -m deepgemm_b200.build`` or call :func:`build`.
"""
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, 'csrc')
LIB_PATH = os.path.join(PKG_DIR, 'libdgb200.so')

NVCC_FLAGS = [
    '-std=c++17', '-O3', '-lineinfo',
    '-gencode', 'arch=compute_100a,code=sm_100a',
    '-Xcompiler', '-fPIC', '-shared',
    '--expt-relaxed-constexpr',
    '-Xptxas', '-warn-lmem-usage',
]


def _nvcc() -> str:
    cuda_home = os.environ.get('CUDA_HOME', '/usr/local/cuda')
    cand = os.path.join(cuda_home, 'bin', 'nvcc')
    if os.path.exists(cand):
        return cand
    found = shutil.which('nvcc')
    if found is None:
        raise RuntimeError('nvcc not found; set CUDA_HOME')
    return found


def _sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(('.cu', '.cuh', '.h')))


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    lib_mtime = os.path.getmtime(LIB_PATH)
    deps = _sources() + [os.path.join(PKG_DIR, '..', 'include', 'dgb200.h')]
    return any(os.path.getmtime(s) > lib_mtime for s in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if any source is newer than it; returns the path of the shared object."""
    if not force and not is_stale():
        return LIB_PATH
    extra = os.environ.get('DGB200_EXTRA_NVCC_FLAGS', '').split()
    cmd = [_nvcc()] + NVCC_FLAGS + extra + (['-Xptxas', '-v'] if verbose else []) + \
          ['-o', LIB_PATH, os.path.join(CSRC, 'dgb200.cu')]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError('nvcc failed building libdgb200.so')
    return LIB_PATH


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='-v' in sys.argv))
