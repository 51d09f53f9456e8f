"""Builds libb200handler.so in-tree with nvcc for sm_100a.

    python -m brainstorm_b200.build [--force] [--verbose]

Objects are rebuilt only when their source (or a header) is newer.  nvcc
cross-compiles without a GPU, so this also runs on a CPU-only machine.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, 'csrc')
OBJ = os.path.join(CSRC, 'build')
LIB = os.path.join(PKG, 'libb200handler.so')
NVCC = os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')

NVCC_FLAGS = [
    '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3',
    '-std=c++17', '-Xcompiler', '-fPIC,-fvisibility=hidden', '-Xptxas', '-v',
    '--expt-relaxed-constexpr',
]  # deliberately no --use_fast_math: expf/tanhf/logf/division stay IEEE-accurate


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith('.cu'))


def _newest_header():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(('.cuh', '.h'))]
    return max([os.path.getmtime(h) for h in hs] + [os.path.getmtime(__file__)])


def _compile(src, verbose):
    obj = os.path.join(OBJ, src[:-3] + '.o')
    cmd = [NVCC] + NVCC_FLAGS + ['-c', os.path.join(CSRC, src), '-o', obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    with open(obj + '.log', 'w') as f:
        f.write(' '.join(cmd) + '\n' + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError('nvcc failed for %s:\n%s' % (src, r.stderr[-4000:]))
    if verbose:
        print(r.stderr)
    return obj


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    hdr = _newest_header()
    todo, objs = [], []
    for src in sources():
        obj = os.path.join(OBJ, src[:-3] + '.o')
        objs.append(obj)
        if (force or not os.path.exists(obj) or
                os.path.getmtime(obj) < max(os.path.getmtime(os.path.join(CSRC, src)), hdr)):
            todo.append(src)
    if todo:
        with ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            list(ex.map(lambda s: _compile(s, verbose), todo))
    if todo or not os.path.exists(LIB):
        cmd = [NVCC, '-shared', '-o', LIB] + objs + ['-lcudart_static', '-ldl', '-lpthread', '-lrt']
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError('link failed:\n' + r.stderr[-4000:])
    return LIB


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='--verbose' in sys.argv))
