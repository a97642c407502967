"""Build recipe of the CUDA library (sm_100a only).

``python -m nha_b200.build`` compiles every ``csrc/*.cu`` with nvcc into
``nha_b200/libnha_b200.so`` (in-tree, so the built library travels with the
source tree).  There is no other backend and no fallback: if the library
is missing and cannot be built, importing the ops raises.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, 'csrc')
LIB = os.path.join(HERE, 'libnha_b200.so')

NVCC_FLAGS = [
    '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
    '--use_fast_math', '-Xcompiler', '-fPIC', '-shared', '-cudart', 'static',
]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, '*.cu')))


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(CSRC, '*.cuh')) + glob.glob(os.path.join(HERE, '..', 'include', '*.h'))
    return any(os.path.getmtime(f) > t for f in deps)


def nvcc_path():
    return shutil.which('nvcc') or ('/usr/local/cuda/bin/nvcc' if os.path.exists('/usr/local/cuda/bin/nvcc') else None)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; return its path."""
    if not force and not is_stale():
        return LIB
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError('nha_b200: nvcc not found and libnha_b200.so is missing or stale; '
                           'there is no fallback implementation')
    objs = []
    # objects and the linked library under names of this process: several ranks that find the library stale at the same
    # time each build their own and the last rename wins, instead of linking each other's half-written objects
    tmp = os.path.join(HERE, 'build', f'p{os.getpid()}')
    os.makedirs(tmp, exist_ok=True)
    procs = []
    for src in sources():
        obj = os.path.join(tmp, os.path.basename(src)[:-3] + '.o')
        objs.append(obj)
        cmd = [nvcc] + [f for f in NVCC_FLAGS if f not in ('-shared',)] + os.environ.get('NHA_B200_NVCC_FLAGS', '').split() \
            + ['-c', src, '-o', obj]
        if verbose:
            cmd.insert(1, '-Xptxas=-v')
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if verbose and out:
            print(out)
        if p.returncode != 0:
            raise RuntimeError(f'nvcc failed on {src}:\n{out}')
    out = f'{LIB}.{os.getpid()}.tmp'
    link = [nvcc, '-shared', '-cudart', 'static', '-gencode', 'arch=compute_100a,code=sm_100a', '-o', out] + objs
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f'link failed:\n{r.stdout}')
    os.replace(out, LIB)
    shutil.rmtree(tmp, ignore_errors=True)
    return LIB


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='-v' in sys.argv))
