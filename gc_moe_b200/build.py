"""Build libgcmoe_sm100.so in-tree with nvcc for sm_100a.

    python -m gc_moe_b200.build

The library is the only native artefact of the package; it is loaded with
ctypes by ``gc_moe_b200._native`` and is never rebuilt implicitly at import.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

PACKAGE_DIR = os.path.dirname(os.path.abspath(__file__))
SOURCE = os.path.join(PACKAGE_DIR, 'csrc', 'gcmoe.cu')
LIBRARY = os.path.join(PACKAGE_DIR, 'libgcmoe_sm100.so')


def _newest_source_mtime() -> float:
    roots = [os.path.join(PACKAGE_DIR, 'csrc'), os.path.join(PACKAGE_DIR, '..', 'include')]
    return max(os.path.getmtime(os.path.join(r, f)) for r in roots for f in os.listdir(r))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources."""
    if (not force and os.path.exists(LIBRARY)
            and os.path.getmtime(LIBRARY) >= _newest_source_mtime()):
        return LIBRARY
    nvcc = shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'
    if not os.path.exists(nvcc):
        raise RuntimeError('nvcc not found; libgcmoe_sm100.so cannot be built')
    cmd = [nvcc, '-gencode', 'arch=compute_100a,code=sm_100a', '-O3', '-std=c++17',
           '-lineinfo', '--shared', '-Xcompiler', '-fPIC', '-Xptxas', '-v' if verbose else '-O3',
           '-cudart', 'shared', '-o', LIBRARY, SOURCE]
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError('nvcc failed:\n' + result.stdout + result.stderr)
    if verbose:
        print(result.stderr)
    return LIBRARY


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='-v' in sys.argv))
