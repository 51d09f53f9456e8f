"""ctypes binding of libb200handler.so.

Prototypes are read from ``include/b200_handler.h`` so that the Python side can
never drift from the declared C-ABI.  There is no fallback: if the shared
library is missing the import fails with instructions to build it.
"""
from __future__ import annotations

import ctypes
import os
import re

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
LIB_PATH = os.path.join(PKG, 'libb200handler.so')
HEADER = os.path.join(ROOT, 'include', 'b200_handler.h')

_CTYPES = {
    'int': ctypes.c_int, 'float': ctypes.c_float, 'int64_t': ctypes.c_int64,
    'uint64_t': ctypes.c_uint64, 'void': None,
}


class B200Error(RuntimeError):
    """A call into libb200handler.so returned a non-zero status."""


def parse_header(path=HEADER):
    """Returns {name: (restype, [argtypes])} for every function declared."""
    with open(path) as f:
        text = f.read()
    text = re.sub(r'/\*.*?\*/', ' ', text, flags=re.S)
    text = re.sub(r'//[^\n]*', ' ', text)
    text = re.sub(r'^\s*#.*$', ' ', text, flags=re.M)
    text = text.replace('extern "C" {', ' ').replace('}', ' ')
    protos = {}
    for decl in text.split(';'):
        decl = ' '.join(decl.split())
        m = re.match(r'^(.*?)\b(b200_\w+)\s*\((.*)\)$', decl)
        if not m:
            continue
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        protos[name] = (_ctype_of(ret), [] if args in ('', 'void') else
                        [_ctype_of(a.strip(), is_arg=True) for a in args.split(',')])
    return protos


def _ctype_of(decl, is_arg=False):
    if '*' in decl:
        if not is_arg and 'char' in decl:
            return ctypes.c_char_p
        return ctypes.c_void_p
    toks = [t for t in decl.replace('const', ' ').split()]
    base = toks[0] if toks else 'void'
    return _CTYPES[base]


def load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            'libb200handler.so has not been built: run '
            '`python -m brainstorm_b200.build` (needs nvcc). '
            'There is no CPU fallback.')
    lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
    protos = parse_header()
    for name, (restype, argtypes) in protos.items():
        fn = getattr(lib, name)  # AttributeError if the .so lacks a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    return lib, protos


lib, PROTOTYPES = load()


def check(rc):
    if rc:
        raise B200Error(lib.b200_last_error().decode('utf-8', 'replace'))
